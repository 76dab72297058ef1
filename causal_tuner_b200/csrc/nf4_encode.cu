// NF4 encode: the inverse of nf4.cu, run once per frozen weight when a checkpoint is installed.
//
//   absmax[g]  = max |w| over block g (blocksize consecutive elements of the flattened weight)
//   index      = number of midpoints between adjacent code levels that lie strictly below
//                w / max(absmax[g], FLT_MIN)  (= nearest level, the lower one on a tie)
//   packed[j]  = index(2j) << 4 | index(2j + 1); elements past n count as 0.0
// and, for nested statistics,
//   offset     = mean(absmax) accumulated in fp64 in a fixed order, rounded to fp32
//   absmax2[h] = max |absmax - offset| over group h (blocksize2 consecutive blocks)
//   absmax_q   = 8-bit index of (absmax - offset) / max(absmax2[h], FLT_MIN) in the 256-level table,
//                by the same midpoint rule.
// The reference leaves this arithmetic to bitsandbytes (modeling/lora.py:41-56); the rule here is
// the library's own (quant.py), which the decoder inverts exactly.
//
// One thread owns 8 consecutive elements (one 16-byte load of a 16-bit weight, one 4-byte store of
// nibbles); the blocksize / 8 threads of a block combine their maxima by warp shuffles, so a
// block never straddles a warp. Pure HBM streaming: 2 B read + 0.5625 B written per bf16 element.
#include <cfloat>

#include "common.cuh"

namespace ct {
namespace {

constexpr int kEncThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kEncThreads) nf4_encode_kernel(const T* __restrict__ w, int64_t n, int64_t padded,
                                                                 int lanes, const float* __restrict__ code,
                                                                 uint8_t* __restrict__ packed,
                                                                 float* __restrict__ absmax, int vec) {
  float mid[15];
#pragma unroll
  for (int i = 0; i < 15; ++i) mid[i] = (__ldg(code + i + 1) + __ldg(code + i)) / 2.f;
  const int64_t thread = static_cast<int64_t>(blockIdx.x) * kEncThreads + threadIdx.x;
  const int64_t e = thread * 8;
  float v[8];
  if (vec && e + 8 <= n) {
    if constexpr (sizeof(T) == 2) {
      const uint4 q = *reinterpret_cast<const uint4*>(w + e);
      const T* h = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = to_float<T>(h[i]);
    } else {
      const float4 a = *reinterpret_cast<const float4*>(w + e), b = *reinterpret_cast<const float4*>(w + e + 4);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = e + i < n ? to_float<T>(w[e + i]) : 0.f;
  }
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
  for (int offset = lanes >> 1; offset > 0; offset >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, offset));
  if (e >= padded) return;
  if ((thread & (lanes - 1)) == 0) absmax[thread / lanes] = m;
  const float scale = fmaxf(m, FLT_MIN);
  uint32_t word = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float s = __fdiv_rn(v[i], scale);
    uint32_t index = 0;
#pragma unroll
    for (int j = 0; j < 15; ++j) index += mid[j] < s ? 1u : 0u;
    // element e+i: byte i/2, high nibble when i is even
    word |= index << (8 * (i >> 1) + ((i & 1) ? 0 : 4));
  }
  const int64_t bytes = (n + 1) / 2, at = e / 2;
  if (vec && at + 4 <= bytes) {
    *reinterpret_cast<uint32_t*>(packed + at) = word;
  } else {
    for (int i = 0; i < 4; ++i)
      if (at + i < bytes) packed[at + i] = static_cast<uint8_t>(word >> (8 * i));
  }
}

// One block: mean of `count` floats, accumulated in fp64 (each thread a strided subsequence, then a
// fixed tree), rounded to fp32.
__global__ void __launch_bounds__(1024) mean_kernel(const float* __restrict__ values, int64_t count,
                                                    float* __restrict__ mean) {
  __shared__ double shared[1024];
  double acc = 0.0;
  for (int64_t i = threadIdx.x; i < count; i += 1024) acc += static_cast<double>(values[i]);
  shared[threadIdx.x] = acc;
  __syncthreads();
  for (int offset = 512; offset > 0; offset >>= 1) {
    if (threadIdx.x < offset) shared[threadIdx.x] += shared[threadIdx.x + offset];
    __syncthreads();
  }
  if (threadIdx.x == 0) *mean = static_cast<float>(shared[0] / static_cast<double>(count));
}

// One block per group of blocksize2 absmax values.
__global__ void __launch_bounds__(kEncThreads) nest_kernel(const float* __restrict__ absmax, int64_t blocks,
                                                           int blocksize2, const float* __restrict__ code2,
                                                           const float* __restrict__ offset,
                                                           uint8_t* __restrict__ quantised,
                                                           float* __restrict__ absmax2) {
  __shared__ float mid[255];
  __shared__ float partial[kEncThreads / 32];
  __shared__ float group_max;
  for (int i = threadIdx.x; i < 255; i += kEncThreads) mid[i] = (code2[i + 1] + code2[i]) / 2.f;
  const float off = *offset;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blocksize2;
  float m = 0.f;
  for (int i = threadIdx.x; i < blocksize2; i += kEncThreads)
    if (first + i < blocks) m = fmaxf(m, fabsf(absmax[first + i] - off));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < kEncThreads / 32; ++i) total = fmaxf(total, partial[i]);
    group_max = total;
    absmax2[blockIdx.x] = total;
  }
  __syncthreads();
  const float scale = fmaxf(group_max, FLT_MIN);
  for (int i = threadIdx.x; i < blocksize2; i += kEncThreads) {
    if (first + i >= blocks) break;
    const float s = __fdiv_rn(absmax[first + i] - off, scale);
    int lo = 0, hi = 255;           // number of midpoints strictly below s
    while (lo < hi) {
      const int middle = (lo + hi) >> 1;
      if (mid[middle] < s) lo = middle + 1; else hi = middle;
    }
    quantised[first + i] = static_cast<uint8_t>(lo);
  }
}

}  // namespace
}  // namespace ct

using namespace ct;

extern "C" int ct_nf4_encode(const void* weight, int64_t n, int dtype, int blocksize, const float* code,
                             uint8_t* packed, float* absmax, void* stream) {
  if (n < 0) return fail(CT_ERR_ARG, "ct_nf4_encode: n=%lld", (long long)n);
  if (blocksize < 8 || blocksize > 256 || (blocksize & (blocksize - 1)))
    return fail(CT_ERR_UNSUPPORTED, "ct_nf4_encode: blocksize %d (powers of two from 8 to 256)", blocksize);
  if (dtype < CT_F32 || dtype > CT_F16) return fail(CT_ERR_ARG, "ct_nf4_encode: dtype %d", dtype);
  if (n == 0) return CT_OK;
  if (!weight || !code || !packed || !absmax) return fail(CT_ERR_ARG, "ct_nf4_encode: null pointer");
  const int64_t padded = (n + blocksize - 1) / blocksize * blocksize;
  const int64_t threads = padded / 8;
  const int64_t grid = (threads + kEncThreads - 1) / kEncThreads;
  if (grid > 0x7fffffffLL) return fail(CT_ERR_UNSUPPORTED, "ct_nf4_encode: n too large");
  const int vec = (reinterpret_cast<uintptr_t>(weight) & 15) == 0 && (reinterpret_cast<uintptr_t>(packed) & 3) == 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int lanes = blocksize / 8;
  if (dtype == CT_BF16)
    nf4_encode_kernel<__nv_bfloat16><<<static_cast<unsigned>(grid), kEncThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(weight), n, padded, lanes, code, packed, absmax, vec);
  else if (dtype == CT_F16)
    nf4_encode_kernel<__half><<<static_cast<unsigned>(grid), kEncThreads, 0, s>>>(
        static_cast<const __half*>(weight), n, padded, lanes, code, packed, absmax, vec);
  else
    nf4_encode_kernel<float><<<static_cast<unsigned>(grid), kEncThreads, 0, s>>>(
        static_cast<const float*>(weight), n, padded, lanes, code, packed, absmax, vec);
  count_launch(false);
  return check_launch("ct_nf4_encode");
}

extern "C" int ct_nf4_nest(const float* absmax, int64_t blocks, int blocksize2, const float* code2,
                           uint8_t* quantised, float* absmax2, float* offset, void* stream) {
  if (blocks < 0 || blocksize2 <= 0) return fail(CT_ERR_ARG, "ct_nf4_nest: blocks=%lld blocksize2=%d", (long long)blocks, blocksize2);
  if (blocks == 0) return CT_OK;
  if (!absmax || !code2 || !quantised || !absmax2 || !offset) return fail(CT_ERR_ARG, "ct_nf4_nest: null pointer");
  const int64_t groups = (blocks + blocksize2 - 1) / blocksize2;
  if (groups > 0x7fffffffLL) return fail(CT_ERR_UNSUPPORTED, "ct_nf4_nest: too many groups");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  mean_kernel<<<1, 1024, 0, s>>>(absmax, blocks, offset);
  count_launch(false);
  nest_kernel<<<static_cast<unsigned>(groups), kEncThreads, 0, s>>>(absmax, blocks, blocksize2, code2, offset, quantised,
                                                                    absmax2);
  count_launch(false);
  return check_launch("ct_nf4_nest");
}
