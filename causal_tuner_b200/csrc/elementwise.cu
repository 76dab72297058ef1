// HBM-bound elementwise kernels of the projection / MLP path: dtype casts of the
// LoRA factors, the SwiGLU product and its in-place backward, adjacent-pair
// RoPE, the residual add and the ordered reduction of split-contraction
// partial sums. All are grid-stride loops over 16-byte vectors where the
// buffers allow it.
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace ct {
namespace {

constexpr int kThreads = 256;

// Grid of an elementwise kernel: one CTA per kThreads * per_thread work items, i.e. every thread makes one pass
// (the kernels are grid-stride loops, so any grid is correct). Measured on B200 against a persistent grid of
// exactly the resident CTAs: the SwiGLU forward runs 21 % faster (205 vs 260 us at 16384 x 14336) and its
// in-place backward 14 % (416 vs 481 us) - the hardware's block scheduler keeps more loads in flight than a
// loop whose next iteration waits for this one's stores. CT_B200_ELEMENTWISE_PERSISTENT=1 restores the
// persistent grid for comparison runs.
template <typename Kernel>
unsigned grid_for(Kernel kernel, int64_t work_items, int per_thread = 1) {
  static const bool persistent = [] {
    const char* text = getenv("CT_B200_ELEMENTWISE_PERSISTENT");
    return text && text[0] == '1';
  }();
  int64_t blocks = (work_items + static_cast<int64_t>(kThreads) * per_thread - 1) / (static_cast<int64_t>(kThreads) * per_thread);
  if (persistent) {
    static std::mutex mutex;
    static std::unordered_map<const void*, int> resident;      // kernel -> resident CTAs on the current device type
    std::lock_guard<std::mutex> lock(mutex);
    const void* key = reinterpret_cast<const void*>(kernel);
    auto found = resident.find(key);
    if (found == resident.end()) {
      int device = 0, sms = 0, per_sm = 0;
      if (cudaGetDevice(&device) != cudaSuccess ||
          cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess || sms <= 0 ||
          per_sm <= 0) {
        cudaGetLastError();
        sms = 148;
        per_sm = 4;
      }
      found = resident.emplace(key, sms * per_sm).first;
    }
    if (blocks > found->second) blocks = found->second;
  }
  if (blocks > (1LL << 30)) blocks = 1LL << 30;
  if (blocks < 1) blocks = 1;
  return static_cast<unsigned>(blocks);
}

// ---- cast ---------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
cast_kernel(const void* src, int src_dtype, int64_t ld_src, void* dst, int dst_dtype, int64_t ld_dst,
            int64_t rows, int64_t cols) {
  const int64_t total = rows * cols;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t r = i / cols, c = i - r * cols;
    store_from_float(dst, r * ld_dst + c, dst_dtype, load_as_float(src, r * ld_src + c, src_dtype));
  }
}

// fp32 -> bf16, contiguous, 8 elements per thread per step.
__global__ void __launch_bounds__(kThreads)
cast_f32_bf16_vec_kernel(const float4* __restrict__ src, uint4* __restrict__ dst, int64_t groups) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < groups;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const float4 lo = __ldg(src + 2 * i), hi = __ldg(src + 2 * i + 1);
    __nv_bfloat162 p0 = __floats2bfloat162_rn(lo.x, lo.y), p1 = __floats2bfloat162_rn(lo.z, lo.w);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(hi.x, hi.y), p3 = __floats2bfloat162_rn(hi.z, hi.w);
    dst[i] = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                        *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
  }
}

// Several contiguous tensors in one launch (the per-call casts of an operator's adapters): the
// pointer table travels as the kernel argument, a block walks 2048-element chunks of the
// concatenation. `vec`: fp32 -> bf16 with every pointer 16-byte aligned and every size a multiple of 8.
constexpr int kCastBatch = 32;
constexpr int kCastChunk = 8 * kThreads;

struct CastBatch {
  const void* src[kCastBatch];
  void* dst[kCastBatch];
  long long size[kCastBatch];
  int first_chunk[kCastBatch + 1];
  int count;
  int vec;
};

__global__ void __launch_bounds__(kThreads)
cast_many_kernel(const __grid_constant__ CastBatch batch, int src_dtype, int dst_dtype) {
  const int chunks = batch.first_chunk[batch.count];
  for (int chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
    int t = 0;
    while (t + 1 < batch.count && batch.first_chunk[t + 1] <= chunk) ++t;
    const long long begin = static_cast<long long>(chunk - batch.first_chunk[t]) * kCastChunk;
    const long long left = batch.size[t] - begin;
    if (batch.vec) {
      const long long i = begin + 8ll * threadIdx.x;
      if (8ll * threadIdx.x < left) {
        const float4* from = reinterpret_cast<const float4*>(static_cast<const float*>(batch.src[t]) + i);
        const float4 lo = __ldg(from), hi = __ldg(from + 1);
        __nv_bfloat162 p0 = __floats2bfloat162_rn(lo.x, lo.y), p1 = __floats2bfloat162_rn(lo.z, lo.w);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(hi.x, hi.y), p3 = __floats2bfloat162_rn(hi.z, hi.w);
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(batch.dst[t]) + i) =
            make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                       *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
      }
    } else {
      const int n = static_cast<int>(left < kCastChunk ? left : kCastChunk);
      for (int j = threadIdx.x; j < n; j += kThreads)
        store_from_float(batch.dst[t], begin + j, dst_dtype, load_as_float(batch.src[t], begin + j, src_dtype));
    }
  }
}

// ---- SwiGLU ---------------------------------------------------------------------
// The element arithmetic (swiglu_element) lives in common.cuh: the GEMM epilogue shares it.
template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_kernel(const T* gate, const T* up, const T* grad, T* out, T* dg, T* du, int64_t n, int reconstruct) {
  const bool backward = grad != nullptr;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const float g = to_float<T>(gate[i]), u = to_float<T>(up[i]);
    const float gr = backward ? to_float<T>(grad[i]) : 0.0f;
    float h = 0.f, a = 0.f, b = 0.f;
    swiglu_element<T>(g, u, gr, backward, reconstruct != 0, h, a, b);
    if (backward) {
      dg[i] = from_float<T>(a);
      du[i] = from_float<T>(b);
    }
    if (reconstruct) out[i] = from_float<T>(h);
  }
}

// bf16, 8 elements (16 bytes) per vector; every buffer 16-byte aligned, n % 8 == 0. A thread handles kSwigluUnroll
// vectors per step and issues all of their loads before the first use: the outputs may alias the inputs
// element for element (the in-place backward), so the compiler cannot move the next vector's loads above
// this vector's stores by itself, and one vector in flight per thread leaves HBM latency exposed.
constexpr int kSwigluUnroll = 2;

__device__ __forceinline__ void swiglu_vector(const uint4& gv, const uint4& uv, const uint4& rv, bool backward,
                                              bool reconstruct, uint4& hv, uint4& av, uint4& bv) {
  const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
  const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
  uint32_t hw[4], aw[4], bw[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[j]));
    const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[j]));
    const float2 r = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw[j]));
    float h0 = 0.f, h1 = 0.f, a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
    swiglu_element<__nv_bfloat16>(g.x, u.x, r.x, backward, reconstruct, h0, a0, b0);
    swiglu_element<__nv_bfloat16>(g.y, u.y, r.y, backward, reconstruct, h1, a1, b1);
    __nv_bfloat162 hp = __floats2bfloat162_rn(h0, h1), ap = __floats2bfloat162_rn(a0, a1),
                   bp = __floats2bfloat162_rn(b0, b1);
    hw[j] = *reinterpret_cast<uint32_t*>(&hp);
    aw[j] = *reinterpret_cast<uint32_t*>(&ap);
    bw[j] = *reinterpret_cast<uint32_t*>(&bp);
  }
  hv = make_uint4(hw[0], hw[1], hw[2], hw[3]);
  av = make_uint4(aw[0], aw[1], aw[2], aw[3]);
  bv = make_uint4(bw[0], bw[1], bw[2], bw[3]);
}

template <bool BACKWARD>
__global__ void __launch_bounds__(kThreads)
swiglu_bf16_vec_kernel(const uint4* gate, const uint4* up, const uint4* grad, uint4* out, uint4* dg, uint4* du,
                       int64_t groups, int reconstruct) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; base < groups;
       base += stride * kSwigluUnroll) {
    uint4 gv[kSwigluUnroll], uv[kSwigluUnroll], rv[kSwigluUnroll];
#pragma unroll
    for (int k = 0; k < kSwigluUnroll; ++k) {
      const int64_t i = base + k * stride;
      const bool live = i < groups;
      gv[k] = live ? gate[i] : make_uint4(0, 0, 0, 0);
      uv[k] = live ? up[i] : make_uint4(0, 0, 0, 0);
      rv[k] = (BACKWARD && live) ? grad[i] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < kSwigluUnroll; ++k) {
      const int64_t i = base + k * stride;
      if (i >= groups) break;
      uint4 hv, av, bv;
      swiglu_vector(gv[k], uv[k], rv[k], BACKWARD, reconstruct != 0, hv, av, bv);
      if (BACKWARD) {
        dg[i] = av;
        du[i] = bv;
      }
      if (reconstruct) out[i] = hv;
    }
  }
}

// ---- RoPE -----------------------------------------------------------------------
// One thread per (row, head, pair). kernels/core_cuda.py:134-164.
template <typename T>
__global__ void __launch_bounds__(kThreads)
rope_kernel(const T* x, const T* cosine, const T* sine, T* y, int64_t rows, int heads, int head_dim, int half,
            int inverse) {
  const int pairs_per_head = head_dim / 2;
  const int64_t total = rows * heads * pairs_per_head;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int channel = static_cast<int>(i % pairs_per_head);
    const int64_t token = i / (static_cast<int64_t>(heads) * pairs_per_head);
    const T even_raw = x[2 * i], odd_raw = x[2 * i + 1];
    if (channel < half) {
      const float even = to_float<T>(even_raw), odd = to_float<T>(odd_raw);
      const float c = to_float<T>(cosine[token * half + channel]);
      float s = to_float<T>(sine[token * half + channel]);
      if (inverse) s = -s;
      const float ec = round_to<T>(__fmul_rn(even, c)), os = round_to<T>(__fmul_rn(odd, s));
      const float oc = round_to<T>(__fmul_rn(odd, c)), es = round_to<T>(__fmul_rn(even, s));
      y[2 * i] = from_float<T>(__fsub_rn(ec, os));
      y[2 * i + 1] = from_float<T>(__fadd_rn(oc, es));
    } else {
      y[2 * i] = even_raw;
      y[2 * i + 1] = odd_raw;
    }
  }
}

// 16-bit types, 8 elements (4 pairs) per thread: one 16-byte load/store of x and one 8-byte load each of
// cos and sin. Needs head_dim % 8 == 0, half % 4 == 0 and 16-byte aligned x / y (8-byte cos / sin).
// `rotated_only`: y aliases x, so the pass-through part of every head is left alone.
template <typename T>
__global__ void __launch_bounds__(kThreads)
rope_vec_kernel(const T* x, const T* cosine, const T* sine, T* y, int64_t rows, int heads, int head_dim, int half,
                int inverse, int rotated_only) {
  const int chunks_per_head = head_dim / 8, rotated_chunks = half / 4;
  const int per_head = rotated_only ? rotated_chunks : chunks_per_head;
  const int64_t total = rows * heads * per_head;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int chunk = static_cast<int>(i % per_head);
    const int64_t head_index = i / per_head;             // token * heads + head
    const int64_t token = head_index / heads;
    const int64_t offset = head_index * head_dim + chunk * 8;
    const uint4 raw = *reinterpret_cast<const uint4*>(x + offset);
    if (chunk >= rotated_chunks) {
      *reinterpret_cast<uint4*>(y + offset) = raw;
      continue;
    }
    const uint2 craw = __ldg(reinterpret_cast<const uint2*>(cosine + token * half + chunk * 4));
    const uint2 sraw = __ldg(reinterpret_cast<const uint2*>(sine + token * half + chunk * 4));
    const T* xv = reinterpret_cast<const T*>(&raw);
    const T* cv = reinterpret_cast<const T*>(&craw);
    const T* sv = reinterpret_cast<const T*>(&sraw);
    uint4 result;
    T* yv = reinterpret_cast<T*>(&result);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float even = to_float<T>(xv[2 * j]), odd = to_float<T>(xv[2 * j + 1]);
      const float c = to_float<T>(cv[j]);
      const float sn = inverse ? -to_float<T>(sv[j]) : to_float<T>(sv[j]);
      const float ec = round_to<T>(__fmul_rn(even, c)), os = round_to<T>(__fmul_rn(odd, sn));
      const float oc = round_to<T>(__fmul_rn(odd, c)), es = round_to<T>(__fmul_rn(even, sn));
      yv[2 * j] = from_float<T>(__fsub_rn(ec, os));
      yv[2 * j + 1] = from_float<T>(__fadd_rn(oc, es));
    }
    *reinterpret_cast<uint4*>(y + offset) = result;
  }
}

// ---- residual add -----------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) add_kernel(T* y, const T* r, int64_t n) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * kThreads)
    y[i] = from_float<T>(__fadd_rn(to_float<T>(y[i]), to_float<T>(r[i])));
}

__global__ void __launch_bounds__(kThreads) add_bf16_vec_kernel(uint4* y, const uint4* r, int64_t groups) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < groups;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const uint4 a = y[i], b = __ldg(r + i);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t ow[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[j]));
      const float2 q = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[j]));
      __nv_bfloat162 o = __floats2bfloat162_rn(__fadd_rn(p.x, q.x), __fadd_rn(p.y, q.y));
      ow[j] = *reinterpret_cast<uint32_t*>(&o);
    }
    y[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

// ---- ordered reduction of split-contraction partial sums ---------------------------
__global__ void __launch_bounds__(kThreads)
reduce_partials_kernel(const float* __restrict__ partials, int slices, int64_t rows, int64_t cols,
                       int64_t ld_partial, float* out, int64_t ld_out, int add) {
  const int64_t total = rows * cols;
  const int64_t slice_stride = rows * ld_partial;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t r = i / cols, c = i - r * cols;
    float acc = add ? out[r * ld_out + c] : 0.0f;
    const float* p = partials + r * ld_partial + c;
    for (int s = 0; s < slices; ++s) acc = __fadd_rn(acc, p[s * slice_stride]);
    out[r * ld_out + c] = acc;
  }
}

// cos / sin of position * inverse frequency: fp32 product, full-range evaluation, rounded to T.
template <typename T>
__global__ void __launch_bounds__(kThreads)
position_values_kernel(const int64_t* __restrict__ positions, const float* __restrict__ inverse, T* __restrict__ cosine,
                       T* __restrict__ sine, int64_t total, int half) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const float angle = __fmul_rn(static_cast<float>(positions[i / half]), inverse[i % half]);
    cosine[i] = from_float<T>(cosf(angle));
    sine[i] = from_float<T>(sinf(angle));
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int reduce_partials(const float* partials, int slices, int64_t rows, int64_t cols, int64_t ld_partial, float* out,
                    int64_t ld_out, int add, cudaStream_t stream) {
  if (rows * cols == 0) return CT_OK;
  reduce_partials_kernel<<<grid_for(reduce_partials_kernel, rows * cols), kThreads, 0, stream>>>(partials, slices, rows, cols, ld_partial, out,
                                                                        ld_out, add);
  count_launch(false);
  return check_launch("reduce_partials");
}

}  // namespace ct

using namespace ct;

extern "C" int ct_cast(const void* src, int src_dtype, int64_t ld_src, void* dst, int dst_dtype, int64_t ld_dst,
                       int64_t rows, int64_t cols, void* stream) {
  if (rows < 0 || cols < 0) return fail(CT_ERR_ARG, "ct_cast: negative size");
  if (rows * cols == 0) return CT_OK;
  if (!src || !dst) return fail(CT_ERR_ARG, "ct_cast: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * cols;
  if (src_dtype == CT_F32 && dst_dtype == CT_BF16 && ld_src == cols && ld_dst == cols && total % 8 == 0 &&
      aligned16(src) && aligned16(dst)) {
    cast_f32_bf16_vec_kernel<<<grid_for(cast_f32_bf16_vec_kernel, total / 8), kThreads, 0, s>>>(static_cast<const float4*>(src),
                                                                     static_cast<uint4*>(dst), total / 8);
  } else {
    cast_kernel<<<grid_for(cast_kernel, total), kThreads, 0, s>>>(src, src_dtype, ld_src, dst, dst_dtype, ld_dst, rows, cols);
  }
  count_launch(false);
  return check_launch("ct_cast");
}

extern "C" int ct_cast_many(int count, const void* const* src, void* const* dst, const int64_t* sizes, int src_dtype,
                            int dst_dtype, void* stream) {
  if (count < 0) return fail(CT_ERR_ARG, "ct_cast_many: count=%d", count);
  if (count == 0) return CT_OK;
  if (!src || !dst || !sizes) return fail(CT_ERR_ARG, "ct_cast_many: null table");
  if (src_dtype < CT_F32 || src_dtype > CT_F16 || dst_dtype < CT_F32 || dst_dtype > CT_F16)
    return fail(CT_ERR_ARG, "ct_cast_many: dtype %d -> %d", src_dtype, dst_dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int first = 0; first < count; first += kCastBatch) {
    CastBatch batch{};
    batch.count = 0;
    batch.vec = src_dtype == CT_F32 && dst_dtype == CT_BF16;
    batch.first_chunk[0] = 0;
    for (int i = first; i < count && i < first + kCastBatch; ++i) {
      if (sizes[i] < 0) return fail(CT_ERR_ARG, "ct_cast_many: negative size at %d", i);
      if (sizes[i] == 0) continue;
      if (!src[i] || !dst[i]) return fail(CT_ERR_ARG, "ct_cast_many: null tensor at %d", i);
      const int j = batch.count++;
      batch.src[j] = src[i];
      batch.dst[j] = dst[i];
      batch.size[j] = sizes[i];
      const long long chunks = (sizes[i] + kCastChunk - 1) / kCastChunk;
      if (batch.first_chunk[j] + chunks > 0x7fffffffLL) return fail(CT_ERR_UNSUPPORTED, "ct_cast_many: tensor too large");
      batch.first_chunk[j + 1] = batch.first_chunk[j] + static_cast<int>(chunks);
      if (sizes[i] % 8 || !aligned16(src[i]) || !aligned16(dst[i])) batch.vec = 0;
    }
    if (batch.count == 0) continue;
    cast_many_kernel<<<grid_for(cast_many_kernel, static_cast<int64_t>(batch.first_chunk[batch.count]) * kThreads), kThreads, 0, s>>>(
        batch, src_dtype, dst_dtype);
    count_launch(false);
  }
  return check_launch("ct_cast_many");
}

extern "C" int ct_swiglu(const void* gate, const void* up, const void* grad, void* out, void* dg, void* du, int64_t n,
                         int dtype, int reconstruct, void* stream) {
  if (n < 0) return fail(CT_ERR_ARG, "ct_swiglu: negative size");
  if (n == 0) return CT_OK;
  if (!gate || !up || (reconstruct && !out) || (grad && (!dg || !du))) return fail(CT_ERR_ARG, "ct_swiglu: null pointer");
  if (!grad && !reconstruct) return fail(CT_ERR_ARG, "ct_swiglu: nothing to compute");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == CT_BF16) {
    const bool vec = n % 8 == 0 && aligned16(gate) && aligned16(up) && (!grad || aligned16(grad)) &&
                     (!reconstruct || aligned16(out)) && (!grad || (aligned16(dg) && aligned16(du)));
    if (vec) {
      const unsigned blocks =
          grid_for(grad ? swiglu_bf16_vec_kernel<true> : swiglu_bf16_vec_kernel<false>, n / 8, kSwigluUnroll);
      (grad ? swiglu_bf16_vec_kernel<true> : swiglu_bf16_vec_kernel<false>)<<<blocks, kThreads, 0, s>>>(
          static_cast<const uint4*>(gate), static_cast<const uint4*>(up), static_cast<const uint4*>(grad),
          static_cast<uint4*>(out), static_cast<uint4*>(dg), static_cast<uint4*>(du), n / 8, reconstruct);
    } else
      swiglu_kernel<__nv_bfloat16><<<grid_for(swiglu_kernel<__nv_bfloat16>, n), kThreads, 0, s>>>(
          static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
          static_cast<const __nv_bfloat16*>(grad), static_cast<__nv_bfloat16*>(out),
          static_cast<__nv_bfloat16*>(dg), static_cast<__nv_bfloat16*>(du), n, reconstruct);
  } else if (dtype == CT_F32) {
    swiglu_kernel<float><<<grid_for(swiglu_kernel<float>, n), kThreads, 0, s>>>(static_cast<const float*>(gate), static_cast<const float*>(up),
                                                          static_cast<const float*>(grad), static_cast<float*>(out),
                                                          static_cast<float*>(dg), static_cast<float*>(du), n,
                                                          reconstruct);
  } else if (dtype == CT_F16) {
    swiglu_kernel<__half><<<grid_for(swiglu_kernel<__half>, n), kThreads, 0, s>>>(static_cast<const __half*>(gate),
                                                           static_cast<const __half*>(up),
                                                           static_cast<const __half*>(grad), static_cast<__half*>(out),
                                                           static_cast<__half*>(dg), static_cast<__half*>(du), n,
                                                           reconstruct);
  } else {
    return fail(CT_ERR_ARG, "ct_swiglu: dtype %d", dtype);
  }
  count_launch(false);
  return check_launch("ct_swiglu");
}

extern "C" int ct_rope(const void* x, const void* cosine, const void* sine, void* y, int64_t rows, int heads,
                       int head_dim, int half, int inverse, int dtype, void* stream) {
  if (rows < 0 || heads <= 0 || head_dim <= 0 || (head_dim & 1) || half < 0 || 2 * half > head_dim)
    return fail(CT_ERR_ARG, "ct_rope: rows=%lld heads=%d head_dim=%d half=%d", (long long)rows, heads, head_dim, half);
  if (rows == 0) return CT_OK;
  if (!x || !y || (half && (!cosine || !sine))) return fail(CT_ERR_ARG, "ct_rope: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * heads * (head_dim / 2);
  const bool vec = dtype != CT_F32 && head_dim % 8 == 0 && half % 4 == 0 && half > 0 && aligned16(x) && aligned16(y) &&
                   (reinterpret_cast<uintptr_t>(cosine) & 7) == 0 && (reinterpret_cast<uintptr_t>(sine) & 7) == 0;
  if (vec) {
    const int rotated_only = x == y;
    const int64_t work = rows * heads * (rotated_only ? half / 4 : head_dim / 8);
    if (dtype == CT_BF16)
      rope_vec_kernel<__nv_bfloat16><<<grid_for(rope_vec_kernel<__nv_bfloat16>, work), kThreads, 0, s>>>(
          static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(cosine),
          static_cast<const __nv_bfloat16*>(sine), static_cast<__nv_bfloat16*>(y), rows, heads, head_dim, half, inverse,
          rotated_only);
    else
      rope_vec_kernel<__half><<<grid_for(rope_vec_kernel<__half>, work), kThreads, 0, s>>>(
          static_cast<const __half*>(x), static_cast<const __half*>(cosine), static_cast<const __half*>(sine),
          static_cast<__half*>(y), rows, heads, head_dim, half, inverse, rotated_only);
    count_launch(false);
    return check_launch("ct_rope");
  }
  if (dtype == CT_BF16)
    rope_kernel<__nv_bfloat16><<<grid_for(rope_kernel<__nv_bfloat16>, total), kThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(cosine),
        static_cast<const __nv_bfloat16*>(sine), static_cast<__nv_bfloat16*>(y), rows, heads, head_dim, half, inverse);
  else if (dtype == CT_F32)
    rope_kernel<float><<<grid_for(rope_kernel<float>, total), kThreads, 0, s>>>(static_cast<const float*>(x),
                                                            static_cast<const float*>(cosine),
                                                            static_cast<const float*>(sine), static_cast<float*>(y),
                                                            rows, heads, head_dim, half, inverse);
  else if (dtype == CT_F16)
    rope_kernel<__half><<<grid_for(rope_kernel<__half>, total), kThreads, 0, s>>>(static_cast<const __half*>(x),
                                                             static_cast<const __half*>(cosine),
                                                             static_cast<const __half*>(sine), static_cast<__half*>(y),
                                                             rows, heads, head_dim, half, inverse);
  else
    return fail(CT_ERR_ARG, "ct_rope: dtype %d", dtype);
  count_launch(false);
  return check_launch("ct_rope");
}

extern "C" int ct_add_inplace(void* y, const void* r, int64_t n, int dtype, void* stream) {
  if (n < 0) return fail(CT_ERR_ARG, "ct_add_inplace: negative size");
  if (n == 0) return CT_OK;
  if (!y || !r) return fail(CT_ERR_ARG, "ct_add_inplace: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == CT_BF16) {
    if (n % 8 == 0 && aligned16(y) && aligned16(r))
      add_bf16_vec_kernel<<<grid_for(add_bf16_vec_kernel, n / 8), kThreads, 0, s>>>(static_cast<uint4*>(y), static_cast<const uint4*>(r),
                                                               n / 8);
    else
      add_kernel<__nv_bfloat16><<<grid_for(add_kernel<__nv_bfloat16>, n), kThreads, 0, s>>>(static_cast<__nv_bfloat16*>(y),
                                                                 static_cast<const __nv_bfloat16*>(r), n);
  } else if (dtype == CT_F32) {
    add_kernel<float><<<grid_for(add_kernel<float>, n), kThreads, 0, s>>>(static_cast<float*>(y), static_cast<const float*>(r), n);
  } else if (dtype == CT_F16) {
    add_kernel<__half><<<grid_for(add_kernel<__half>, n), kThreads, 0, s>>>(static_cast<__half*>(y), static_cast<const __half*>(r), n);
  } else {
    return fail(CT_ERR_ARG, "ct_add_inplace: dtype %d", dtype);
  }
  count_launch(false);
  return check_launch("ct_add_inplace");
}

extern "C" int ct_position_values(const int64_t* positions, const float* inverse, void* cosine, void* sine,
                                  int64_t count, int half, int dtype, void* stream) {
  if (count < 0 || half < 0) return fail(CT_ERR_ARG, "ct_position_values: count=%lld half=%d", (long long)count, half);
  if (count == 0 || half == 0) return CT_OK;
  if (!positions || !inverse || !cosine || !sine) return fail(CT_ERR_ARG, "ct_position_values: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t total = count * half;
  if (dtype == CT_BF16)
    position_values_kernel<__nv_bfloat16><<<grid_for(position_values_kernel<__nv_bfloat16>, total), kThreads, 0, s>>>(
        positions, inverse, static_cast<__nv_bfloat16*>(cosine), static_cast<__nv_bfloat16*>(sine), total, half);
  else if (dtype == CT_F16)
    position_values_kernel<__half><<<grid_for(position_values_kernel<__half>, total), kThreads, 0, s>>>(
        positions, inverse, static_cast<__half*>(cosine), static_cast<__half*>(sine), total, half);
  else if (dtype == CT_F32)
    position_values_kernel<float><<<grid_for(position_values_kernel<float>, total), kThreads, 0, s>>>(
        positions, inverse, static_cast<float*>(cosine), static_cast<float*>(sine), total, half);
  else
    return fail(CT_ERR_ARG, "ct_position_values: dtype %d", dtype);
  count_launch(false);
  return check_launch("ct_position_values");
}
