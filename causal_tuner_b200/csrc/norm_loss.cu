// Row-wise kernels next to the projection path: RMSNorm forward / input gradient and the
// weighted cross-entropy that turns a tile of logits into per-row losses and, in place, into
// the gradient of those losses. All HBM-bound: one CTA per row, 16-byte vectors where the row
// allows it, fp32 arithmetic, the rounding points of the reference kernels
// (kernels/core_cuda.py:30-82, kernels/loss_cuda.py:12-55).
#include "common.cuh"

namespace ct {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) total += scratch[w];
  return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = -INFINITY;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) total = fmaxf(total, scratch[w]);
  return total;
}

// y = round(x * rstd) * round(w); rstd = rsqrt(mean(x^2) + eps) is kept for the backward pass.
template <typename T, typename W>
__global__ void __launch_bounds__(kThreads)
rms_forward_kernel(const T* x, const W* w, T* y, float* rstd, int64_t width, float eps) {
  __shared__ float scratch[kThreads / 32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * width;
  float sum = 0.f;
  for (int64_t c = threadIdx.x; c < width; c += kThreads) {
    const float v = to_float<T>(xr[c]);
    sum += v * v;
  }
  const float inverse = rsqrtf(block_sum(sum, scratch) / static_cast<float>(width) + eps);
  if (threadIdx.x == 0) rstd[row] = inverse;
  T* yr = y + row * width;
  for (int64_t c = threadIdx.x; c < width; c += kThreads) {
    const float normalized = round_to<T>(to_float<T>(xr[c]) * inverse);
    const float weight = round_to<T>(to_float<W>(w[c]));
    yr[c] = from_float<T>(normalized * weight);
  }
}

// gx = rstd * (g - x * rstd^2 * mean(g * x)) with g = round(go * round(w)); gx may alias go.
// With `add`: gx = round(gx) + add, the sum autograd would form when x also feeds a residual path.
// FROM_OUTPUT: `x` holds the norm's OUTPUT y instead of its input; the normalised row is rebuilt as
// n = y / round(w) and gx = rstd * (g - n * mean(g * n)) (kernels/core_cuda.py:56-59).
template <typename T, typename W, bool FROM_OUTPUT>
__global__ void __launch_bounds__(kThreads)
rms_backward_kernel(const T* x, const W* w, const float* rstd, const T* go, const T* add, T* gx, int64_t width) {
  __shared__ float scratch[kThreads / 32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * width;
  const T* gr = go + row * width;
  float sum = 0.f;
  for (int64_t c = threadIdx.x; c < width; c += kThreads) {
    const float weight = round_to<T>(to_float<W>(w[c]));
    const float gradient = round_to<T>(to_float<T>(gr[c]) * weight);
    sum += gradient * (FROM_OUTPUT ? __fdividef(to_float<T>(xr[c]), weight) : to_float<T>(xr[c]));
  }
  const float projection = block_sum(sum, scratch) / static_cast<float>(width);
  const float inverse = rstd[row];
  T* out = gx + row * width;
  for (int64_t c = threadIdx.x; c < width; c += kThreads) {
    const float weight = round_to<T>(to_float<W>(w[c]));
    const float gradient = round_to<T>(to_float<T>(gr[c]) * weight);
    float value = FROM_OUTPUT ? inverse * (gradient - __fdividef(to_float<T>(xr[c]), weight) * projection)
                              : inverse * (gradient - to_float<T>(xr[c]) * (inverse * inverse * projection));
    if (add) value = __fadd_rn(round_to<T>(value), to_float<T>(add[row * width + c]));
    out[c] = from_float<T>(value);
  }
}

// 16-bit activations, width % 8 == 0, 16-byte aligned rows and weights: the same arithmetic with 16-byte loads and
// stores. Rows of up to kHeld * kThreads chunks (4096 elements) stay in registers between the two
// passes, and all of a thread's loads are issued before the first use; longer rows are read again
// (from L1).
constexpr int kHeld = 2;

// Eight consecutive weights, rounded to the activation type T, from one or two 16-byte loads.
template <typename T, typename W>
__device__ __forceinline__ void load_weights(const W* w, int64_t c, float (&out)[8]) {
  if constexpr (sizeof(W) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4*>(w + c * 8);
    const W* v = reinterpret_cast<const W*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = round_to<T>(to_float<W>(v[j]));
  } else {
    const float4 lo = *reinterpret_cast<const float4*>(w + c * 8), hi = *reinterpret_cast<const float4*>(w + c * 8 + 4);
    const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = round_to<T>(v[j]);
  }
}

template <typename T, typename W>
__global__ void __launch_bounds__(kThreads, 8)             // 32 registers, no spills: full occupancy
rms_forward_vec_kernel(const T* x, const W* w, T* y, float* rstd, int64_t width, float eps) {
  __shared__ float scratch[kThreads / 32];
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * width);
  const int64_t chunks = width / 8;
  const bool held = chunks <= kHeld * kThreads;
  uint4 kept[kHeld];
  float sum = 0.f;
  auto square = [&](const uint4& raw) {
    const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = to_float<T>(v[j]);
      sum += f * f;
    }
  };
  if (held) {
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int64_t c = threadIdx.x + i * kThreads;
      kept[i] = c < chunks ? xr[c] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kHeld; ++i) square(kept[i]);
  } else {
    for (int64_t c = threadIdx.x; c < chunks; c += kThreads) square(xr[c]);
  }
  const float inverse = rsqrtf(block_sum(sum, scratch) / static_cast<float>(width) + eps);
  if (threadIdx.x == 0) rstd[row] = inverse;
  uint4* yr = reinterpret_cast<uint4*>(y + row * width);
  auto emit = [&](const uint4& raw, int64_t c) {
    const T* v = reinterpret_cast<const T*>(&raw);
    uint4 out;
    T* o = reinterpret_cast<T*>(&out);
    float weight[8];
    load_weights<T, W>(w, c, weight);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float normalized = round_to<T>(to_float<T>(v[j]) * inverse);
      o[j] = from_float<T>(normalized * weight[j]);
    }
    yr[c] = out;
  };
  if (held) {
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int64_t c = threadIdx.x + i * kThreads;
      if (c < chunks) emit(kept[i], c);
    }
  } else {
    for (int64_t c = threadIdx.x; c < chunks; c += kThreads) emit(xr[c], c);
  }
}

template <typename T, typename W, bool ADD, bool FROM_OUTPUT>
__global__ void __launch_bounds__(kThreads, ADD ? 4 : 6)   // 40 registers without spills (plain), 64 with the add
rms_backward_vec_kernel(const T* x, const W* w, const float* rstd, const T* go, const T* add, T* gx, int64_t width) {
  __shared__ float scratch[kThreads / 32];
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * width);
  const uint4* gr = reinterpret_cast<const uint4*>(go + row * width);
  const int64_t chunks = width / 8;
  const bool held = chunks <= kHeld * kThreads;
  const uint4* extra = ADD ? reinterpret_cast<const uint4*>(add + row * width) : nullptr;
  uint4 kept_x[kHeld], kept_g[kHeld], kept_a[ADD ? kHeld : 1];
  float sum = 0.f;
  auto project = [&](const uint4& xraw, const uint4& graw, int64_t c) {
    const T* xv = reinterpret_cast<const T*>(&xraw);
    const T* gv = reinterpret_cast<const T*>(&graw);
    float weight[8];
    load_weights<T, W>(w, c, weight);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      sum += round_to<T>(to_float<T>(gv[j]) * weight[j]) *
             (FROM_OUTPUT ? __fdividef(to_float<T>(xv[j]), weight[j]) : to_float<T>(xv[j]));
  };
  if (held) {
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int64_t c = threadIdx.x + i * kThreads;
      kept_x[i] = c < chunks ? xr[c] : make_uint4(0, 0, 0, 0);
      kept_g[i] = c < chunks ? gr[c] : make_uint4(0, 0, 0, 0);
      if constexpr (ADD) kept_a[i] = c < chunks ? extra[c] : make_uint4(0, 0, 0, 0);   // in flight with x and g
    }
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int64_t c = threadIdx.x + i * kThreads;
      if (c < chunks) project(kept_x[i], kept_g[i], c);
    }
  } else {
    for (int64_t c = threadIdx.x; c < chunks; c += kThreads) project(xr[c], gr[c], c);
  }
  const float projection = block_sum(sum, scratch) / static_cast<float>(width);
  const float inverse = rstd[row];
  const float factor = inverse * inverse * projection;
  uint4* out = reinterpret_cast<uint4*>(gx + row * width);
  auto emit = [&](const uint4& xraw, const uint4& graw, const uint4& other, int64_t c) {
    const T* xv = reinterpret_cast<const T*>(&xraw);
    const T* gv = reinterpret_cast<const T*>(&graw);
    uint4 result;
    const T* av = reinterpret_cast<const T*>(&other);
    T* o = reinterpret_cast<T*>(&result);
    float weight[8];
    load_weights<T, W>(w, c, weight);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gradient = round_to<T>(to_float<T>(gv[j]) * weight[j]);
      float value = FROM_OUTPUT ? inverse * (gradient - __fdividef(to_float<T>(xv[j]), weight[j]) * projection)
                                : inverse * (gradient - to_float<T>(xv[j]) * factor);
      if constexpr (ADD) value = __fadd_rn(round_to<T>(value), to_float<T>(av[j]));
      o[j] = from_float<T>(value);
    }
    out[c] = result;
  };
  if (held) {
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int64_t c = threadIdx.x + i * kThreads;
      if (c < chunks) emit(kept_x[i], kept_g[i], kept_a[ADD ? i : 0], c);
    }
  } else {
    for (int64_t c = threadIdx.x; c < chunks; c += kThreads)
      emit(xr[c], gr[c], ADD ? extra[c] : make_uint4(0, 0, 0, 0), c);
  }
}

// Trainable norm weight (kernels/core_cuda.py:43-91): a CTA walks `rows_per_group` consecutive rows; per row it
// optionally writes the input gradient (never in reconstruction mode, never over `go`) and adds
// go * round(x * rstd) to one fp32 sum per column. The sums of a group go to partials[group, :];
// rms_weight_reduce_kernel then adds the groups in index order. Rows are visited in order and every
// column belongs to one thread, so the result does not depend on scheduling.
constexpr size_t kWeightGradSharedLimit = 200 * 1024;

template <typename T, typename W>
__global__ void __launch_bounds__(kThreads)
rms_weight_gradient_kernel(const T* x, const W* w, const float* rstd, const T* go, T* gx, float* partials, int64_t rows,
                           int64_t width, int64_t rows_per_group, int in_shared) {
  extern __shared__ float column_sums[];
  __shared__ float scratch[kThreads / 32];
  const int64_t group = blockIdx.x;
  float* sums = in_shared ? column_sums : partials + group * width;
  for (int64_t c = threadIdx.x; c < width; c += kThreads) sums[c] = 0.f;
  const int64_t first = group * rows_per_group;
  const int64_t last = first + rows_per_group < rows ? first + rows_per_group : rows;
  for (int64_t row = first; row < last; ++row) {
    const T* xr = x + row * width;
    const T* gr = go + row * width;
    const float inverse = rstd[row];
    if (gx) {
      float sum = 0.f;
      for (int64_t c = threadIdx.x; c < width; c += kThreads)
        sum += round_to<T>(to_float<T>(gr[c]) * round_to<T>(to_float<W>(w[c]))) * to_float<T>(xr[c]);
      const float projection = block_sum(sum, scratch) / static_cast<float>(width);
      T* out = gx + row * width;
      for (int64_t c = threadIdx.x; c < width; c += kThreads) {
        const float gradient = round_to<T>(to_float<T>(gr[c]) * round_to<T>(to_float<W>(w[c])));
        out[c] = from_float<T>(inverse * (gradient - to_float<T>(xr[c]) * (inverse * inverse * projection)));
      }
    }
    for (int64_t c = threadIdx.x; c < width; c += kThreads)
      sums[c] += to_float<T>(gr[c]) * round_to<T>(to_float<T>(xr[c]) * inverse);
  }
  if (in_shared) {
    float* out = partials + group * width;
    for (int64_t c = threadIdx.x; c < width; c += kThreads) out[c] = sums[c];
  }
}

// dw[c] = sum over groups (in index order within each of 8 interleaved lanes, lanes then added in order).
template <typename W>
__global__ void rms_weight_reduce_kernel(const float* partials, int64_t groups, int64_t width, W* dw) {
  __shared__ float lanes[8][33];
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + threadIdx.x;
  float sum = 0.f;
  if (c < width)
    for (int64_t g = threadIdx.y; g < groups; g += 8) sum += partials[g * width + c];
  lanes[threadIdx.y][threadIdx.x] = sum;
  __syncthreads();
  if (threadIdx.y == 0 && c < width) {
    float total = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) total += lanes[l][threadIdx.x];
    dw[c] = from_float<W>(total);
  }
}

// loss[row] = weight * (logsumexp(logits[row]) - logits[row, target]); with `gradient`, logits[row]
// becomes (softmax(logits[row]) - onehot(target)) * weight.
template <typename T>
__global__ void __launch_bounds__(kThreads)
weighted_ce_kernel(T* logits, const int64_t* targets, const float* weights, float* loss, int64_t vocab, int gradient) {
  __shared__ float scratch[kThreads / 32];
  const int64_t row = blockIdx.x;
  T* lr = logits + row * vocab;
  float maximum = -INFINITY;
  for (int64_t c = threadIdx.x; c < vocab; c += kThreads) maximum = fmaxf(maximum, to_float<T>(lr[c]));
  maximum = block_max(maximum, scratch);
  float sum = 0.f;
  for (int64_t c = threadIdx.x; c < vocab; c += kThreads) sum += expf(to_float<T>(lr[c]) - maximum);
  const float lse = maximum + logf(block_sum(sum, scratch));
  const int64_t target = targets[row];
  const float weight = weights[row];
  // A target outside [0, vocab) (an ignore index on a zero-weight row) selects nothing: no read, no one-hot term.
  const bool target_ok = target >= 0 && target < vocab;
  const float selected = target_ok ? to_float<T>(lr[target]) : 0.f;
  __syncthreads();  // every thread has read the target logit before anyone overwrites it
  if (threadIdx.x == 0) loss[row] = weight * (lse - selected);
  if (gradient) {
    for (int64_t c = threadIdx.x; c < vocab; c += kThreads) {
      const float derivative = (expf(to_float<T>(lr[c]) - lse) - (target_ok && c == target ? 1.f : 0.f)) * weight;
      lr[c] = from_float<T>(derivative);
    }
  }
}

}  // namespace
}  // namespace ct

using namespace ct;

extern "C" int ct_rmsnorm_forward(const void* x, const void* w, void* y, float* rstd, int64_t rows, int64_t width,
                                  float eps, int dtype, int weight_dtype, void* stream) {
  if (rows < 0 || width <= 0) return fail(CT_ERR_ARG, "ct_rmsnorm_forward: rows=%lld width=%lld", (long long)rows, (long long)width);
  if (rows == 0) return CT_OK;
  if (!x || !w || !y || !rstd) return fail(CT_ERR_ARG, "ct_rmsnorm_forward: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  const bool vec = dtype == CT_BF16 && width % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  if (vec && weight_dtype == CT_BF16) {
    rms_forward_vec_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), rstd, width, eps);
    count_launch(false);
    return check_launch("ct_rmsnorm_forward");
  }
  if (vec && weight_dtype == CT_F32) {
    rms_forward_vec_kernel<__nv_bfloat16, float><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(w), static_cast<__nv_bfloat16*>(y), rstd, width, eps);
    count_launch(false);
    return check_launch("ct_rmsnorm_forward");
  }
#define CT_RMS_FWD(T, W) rms_forward_kernel<T, W><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x), static_cast<const W*>(w), static_cast<T*>(y), rstd, width, eps)
  if (dtype == CT_BF16 && weight_dtype == CT_BF16) CT_RMS_FWD(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == CT_BF16 && weight_dtype == CT_F32) CT_RMS_FWD(__nv_bfloat16, float);
  else if (dtype == CT_F32 && weight_dtype == CT_F32) CT_RMS_FWD(float, float);
  else if (dtype == CT_F32 && weight_dtype == CT_BF16) CT_RMS_FWD(float, __nv_bfloat16);
  else return fail(CT_ERR_ARG, "ct_rmsnorm_forward: dtype %d / %d", dtype, weight_dtype);
#undef CT_RMS_FWD
  count_launch(false);
  return check_launch("ct_rmsnorm_forward");
}

namespace {

int rms_backward_launch(const void* x, const void* w, const float* rstd, const void* go, const void* add, void* gx,
                        int64_t rows, int64_t width, int dtype, int weight_dtype, bool from_output, void* stream) {
  if (rows < 0 || width <= 0) return fail(CT_ERR_ARG, "ct_rmsnorm_backward: rows=%lld width=%lld", (long long)rows, (long long)width);
  if (rows == 0) return CT_OK;
  if (!x || !w || !rstd || !go || !gx) return fail(CT_ERR_ARG, "ct_rmsnorm_backward: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  const bool vec = dtype == CT_BF16 && width % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(go) | reinterpret_cast<uintptr_t>(gx) |
                     reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(add)) & 15) == 0;
  using bf16 = __nv_bfloat16;
#define CT_RMS_BWD_VEC(W, ADD, OUT)                                                                                   \
  rms_backward_vec_kernel<bf16, W, ADD, OUT><<<grid, kThreads, 0, s>>>(                                               \
      static_cast<const bf16*>(x), static_cast<const W*>(w), rstd, static_cast<const bf16*>(go),                      \
      static_cast<const bf16*>(add), static_cast<bf16*>(gx), width)
  if (vec && (weight_dtype == CT_BF16 || weight_dtype == CT_F32)) {
    const bool narrow = weight_dtype == CT_BF16;
    if (from_output && add) { if (narrow) CT_RMS_BWD_VEC(bf16, true, true); else CT_RMS_BWD_VEC(float, true, true); }
    else if (from_output) { if (narrow) CT_RMS_BWD_VEC(bf16, false, true); else CT_RMS_BWD_VEC(float, false, true); }
    else if (add)    { if (narrow) CT_RMS_BWD_VEC(bf16, true, false); else CT_RMS_BWD_VEC(float, true, false); }
    else             { if (narrow) CT_RMS_BWD_VEC(bf16, false, false); else CT_RMS_BWD_VEC(float, false, false); }
    count_launch(false);
    return check_launch("ct_rmsnorm_backward");
  }
#undef CT_RMS_BWD_VEC
#define CT_RMS_BWD(T, W)                                                                                              \
  do {                                                                                                                \
    if (from_output)                                                                                                  \
      rms_backward_kernel<T, W, true><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x), static_cast<const W*>(w),   \
          rstd, static_cast<const T*>(go), static_cast<const T*>(add), static_cast<T*>(gx), width);                   \
    else                                                                                                              \
      rms_backward_kernel<T, W, false><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x), static_cast<const W*>(w),  \
          rstd, static_cast<const T*>(go), static_cast<const T*>(add), static_cast<T*>(gx), width);                   \
  } while (0)
  if (dtype == CT_BF16 && weight_dtype == CT_BF16) CT_RMS_BWD(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == CT_BF16 && weight_dtype == CT_F32) CT_RMS_BWD(__nv_bfloat16, float);
  else if (dtype == CT_F32 && weight_dtype == CT_F32) CT_RMS_BWD(float, float);
  else if (dtype == CT_F32 && weight_dtype == CT_BF16) CT_RMS_BWD(float, __nv_bfloat16);
  else return fail(CT_ERR_ARG, "ct_rmsnorm_backward: dtype %d / %d", dtype, weight_dtype);
#undef CT_RMS_BWD
  count_launch(false);
  return check_launch("ct_rmsnorm_backward");
}

}  // namespace

extern "C" int ct_rmsnorm_backward_add(const void* x, const void* w, const float* rstd, const void* go, const void* add,
                                       void* gx, int64_t rows, int64_t width, int dtype, int weight_dtype,
                                       void* stream) {
  return rms_backward_launch(x, w, rstd, go, add, gx, rows, width, dtype, weight_dtype, false, stream);
}

extern "C" int ct_rmsnorm_backward(const void* x, const void* w, const float* rstd, const void* go, void* gx,
                                   int64_t rows, int64_t width, int dtype, int weight_dtype, void* stream) {
  return rms_backward_launch(x, w, rstd, go, nullptr, gx, rows, width, dtype, weight_dtype, false, stream);
}

extern "C" int ct_rmsnorm_backward_from_output(const void* y, const void* w, const float* rstd, const void* go,
                                               const void* add, void* gx, int64_t rows, int64_t width, int dtype,
                                               int weight_dtype, void* stream) {
  return rms_backward_launch(y, w, rstd, go, add, gx, rows, width, dtype, weight_dtype, true, stream);
}

extern "C" int ct_rmsnorm_weight_gradient(const void* x, const void* w, const float* rstd, const void* go, void* gx,
                                          float* partials, int64_t rows, int64_t width, int64_t rows_per_group,
                                          int dtype, int weight_dtype, void* stream) {
  if (rows < 0 || width <= 0 || rows_per_group <= 0)
    return fail(CT_ERR_ARG, "ct_rmsnorm_weight_gradient: rows=%lld width=%lld rows_per_group=%lld", (long long)rows,
                (long long)width, (long long)rows_per_group);
  if (rows == 0) return CT_OK;
  if (!x || !w || !rstd || !go || !partials) return fail(CT_ERR_ARG, "ct_rmsnorm_weight_gradient: null pointer");
  if (gx && gx == go) return fail(CT_ERR_ARG, "ct_rmsnorm_weight_gradient: gx must not alias go (go is read after gx is written)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t groups = (rows + rows_per_group - 1) / rows_per_group;
  if (groups > 0x7fffffff) return fail(CT_ERR_ARG, "ct_rmsnorm_weight_gradient: %lld groups", (long long)groups);
  // Column sums live in shared memory when the row fits (any hidden width in practice), else in the
  // global partial row itself; either way every column has exactly one owner thread.
  const size_t wanted = static_cast<size_t>(width) * sizeof(float);
  const bool in_shared = wanted <= kWeightGradSharedLimit;
  const size_t smem = in_shared ? wanted : 0;
#define CT_RMS_WG(T, W)                                                                                               \
  do {                                                                                                                \
    auto kernel = rms_weight_gradient_kernel<T, W>;                                                                   \
    if (smem > 48 * 1024 &&                                                                                           \
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) \
      return fail(CT_ERR_CUDA, "ct_rmsnorm_weight_gradient: cannot opt in to %zu bytes of shared memory", smem);      \
    kernel<<<static_cast<unsigned>(groups), kThreads, smem, s>>>(static_cast<const T*>(x), static_cast<const W*>(w), \
        rstd, static_cast<const T*>(go), static_cast<T*>(gx), partials, rows, width, rows_per_group, in_shared ? 1 : 0); \
  } while (0)
  if (dtype == CT_BF16 && weight_dtype == CT_BF16) CT_RMS_WG(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == CT_BF16 && weight_dtype == CT_F32) CT_RMS_WG(__nv_bfloat16, float);
  else if (dtype == CT_F32 && weight_dtype == CT_F32) CT_RMS_WG(float, float);
  else if (dtype == CT_F32 && weight_dtype == CT_BF16) CT_RMS_WG(float, __nv_bfloat16);
  else return fail(CT_ERR_ARG, "ct_rmsnorm_weight_gradient: dtype %d / %d", dtype, weight_dtype);
#undef CT_RMS_WG
  count_launch(false);
  return check_launch("ct_rmsnorm_weight_gradient");
}

extern "C" int ct_rmsnorm_weight_reduce(const float* partials, int64_t groups, int64_t width, void* dw, int weight_dtype,
                                        void* stream) {
  if (groups < 0 || width <= 0) return fail(CT_ERR_ARG, "ct_rmsnorm_weight_reduce: groups=%lld width=%lld", (long long)groups, (long long)width);
  if (!dw || (groups > 0 && !partials)) return fail(CT_ERR_ARG, "ct_rmsnorm_weight_reduce: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>((width + 31) / 32);
  if (weight_dtype == CT_F32)
    rms_weight_reduce_kernel<float><<<grid, dim3(32, 8), 0, s>>>(partials, groups, width, static_cast<float*>(dw));
  else if (weight_dtype == CT_BF16)
    rms_weight_reduce_kernel<__nv_bfloat16><<<grid, dim3(32, 8), 0, s>>>(partials, groups, width, static_cast<__nv_bfloat16*>(dw));
  else if (weight_dtype == CT_F16)
    rms_weight_reduce_kernel<__half><<<grid, dim3(32, 8), 0, s>>>(partials, groups, width, static_cast<__half*>(dw));
  else
    return fail(CT_ERR_ARG, "ct_rmsnorm_weight_reduce: dtype %d", weight_dtype);
  count_launch(false);
  return check_launch("ct_rmsnorm_weight_reduce");
}

extern "C" int ct_weighted_ce(void* logits, const int64_t* targets, const float* weights, float* loss, int64_t rows,
                              int64_t vocab, int gradient, int dtype, void* stream) {
  if (rows < 0 || vocab <= 0) return fail(CT_ERR_ARG, "ct_weighted_ce: rows=%lld vocab=%lld", (long long)rows, (long long)vocab);
  if (rows == 0) return CT_OK;
  if (!logits || !targets || !weights || !loss) return fail(CT_ERR_ARG, "ct_weighted_ce: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  if (dtype == CT_BF16)
    weighted_ce_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(static_cast<__nv_bfloat16*>(logits), targets, weights, loss, vocab, gradient);
  else if (dtype == CT_F32)
    weighted_ce_kernel<float><<<grid, kThreads, 0, s>>>(static_cast<float*>(logits), targets, weights, loss, vocab, gradient);
  else
    return fail(CT_ERR_ARG, "ct_weighted_ce: dtype %d", dtype);
  count_launch(false);
  return check_launch("ct_weighted_ce");
}
