// Gradient scale + global-norm clip + AdamW over a list of fp32 tensors, in two passes over the
// gradients instead of the reference's four separate multi-tensor passes (divide, norm, clip, AdamW;
// training/engine.py:97-107).
//
//   ct_grad_norm / ct_adamw_update are the two passes:
//   pass 1  partial sums of (g / divisor)^2, one per block, then one block adds the partials in index
//           order: norm = sqrt(sum), coef = min(1, max_norm / (norm + 1e-6))  (coef = 1 when max_norm <= 0)
//   pass 2  g' = g / divisor * coef;  p *= 1 - lr * wd;  m += (g' - m) * (1 - beta1);
//           v = beta2 * v + (1 - beta2) * g'^2;  p -= lr / bc1 * m / (sqrt(v) / sqrt(bc2) + eps)
//
// `divisor` lives on the device (the summed supervision weight, clamped to >= 1 by the caller), so
// the host never waits for it. A non-finite norm leaves every tensor untouched; the caller reads
// norm_out afterwards and raises. Tensors are handed over in batches of kBatch pointers passed by
// value as the kernel argument; a block walks 4096-element chunks of the batch's concatenation with
// a fixed chunk -> block assignment, so the norm is reproducible run to run.
#include "common.cuh"

namespace ct {
namespace {

constexpr int kBatch = 40;          // tensors per launch (the table travels as a kernel argument)
constexpr int kOptThreads = 256;
constexpr int kChunk = 4096;        // elements per block iteration: 256 threads x 4 float4
constexpr int kOptBlocks = 148 * 4;

struct OptBatch {
  float* grad[kBatch];
  float* param[kBatch];
  float* m[kBatch];
  float* v[kBatch];
  float decay[kBatch];
  long long size[kBatch];
  int first_chunk[kBatch + 1];      // prefix sum of ceil(size / kChunk)
  int count;
  int vec;                          // every pointer 16-byte aligned
};

__device__ __forceinline__ int tensor_of(const OptBatch& b, int chunk) {
  int lo = 0, hi = b.count - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (b.first_chunk[mid] <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float block_sum(float value, float* shared) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) shared[warp] = value;
  __syncthreads();
  float total = 0.f;
  if (threadIdx.x == 0)
    for (int w = 0; w < kOptThreads / 32; ++w) total += shared[w];
  return total;   // valid in thread 0
}

__global__ void __launch_bounds__(kOptThreads) sumsq_kernel(const __grid_constant__ OptBatch batch,
                                                            const float* __restrict__ divisor,
                                                            float* __restrict__ partials) {
  __shared__ float shared[kOptThreads / 32];
  const float d = *divisor;
  const int chunks = batch.first_chunk[batch.count];
  float acc = 0.f;
  for (int chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
    const int t = tensor_of(batch, chunk);
    const long long begin = static_cast<long long>(chunk - batch.first_chunk[t]) * kChunk;
    const long long size = batch.size[t];
    const float* g = batch.grad[t] + begin;
    const int n = static_cast<int>(size - begin < kChunk ? size - begin : kChunk);
    if (batch.vec && n == kChunk) {
      float4 q[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = reinterpret_cast<const float4*>(g)[i * kOptThreads + threadIdx.x];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = q[i].x / d, b = q[i].y / d, c = q[i].z / d, e = q[i].w / d;
        acc += a * a + b * b + c * c + e * e;
      }
    } else {
      for (int i = threadIdx.x; i < n; i += kOptThreads) {
        const float a = g[i] / d;
        acc += a * a;
      }
    }
  }
  const float total = block_sum(acc, shared);
  if (threadIdx.x == 0) partials[blockIdx.x] = total;
}

// One block: adds `count` partials in index order (each thread a strided subsequence, then a fixed tree).
__global__ void __launch_bounds__(kOptThreads) norm_kernel(const float* __restrict__ partials, int count,
                                                           float max_norm, float* __restrict__ norm_out) {
  __shared__ double shared[kOptThreads];
  double acc = 0.0;
  for (int i = threadIdx.x; i < count; i += kOptThreads) acc += static_cast<double>(partials[i]);
  shared[threadIdx.x] = acc;
  __syncthreads();
  for (int offset = kOptThreads / 2; offset > 0; offset >>= 1) {
    if (threadIdx.x < offset) shared[threadIdx.x] += shared[threadIdx.x + offset];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float norm = static_cast<float>(sqrt(shared[0]));
    float coef = 1.f;
    if (max_norm > 0.f) coef = fminf(1.f, max_norm / (norm + 1e-6f));
    norm_out[0] = norm;
    norm_out[1] = coef;
  }
}

struct Hyper {
  float lr, beta1, beta2, eps;
  float step_size;      // lr / (1 - beta1^step)
  float bc2_sqrt;       // sqrt(1 - beta2^step)
  int write_grads;
};

__device__ __forceinline__ void adamw_one(float& g, float& p, float& m, float& v, float d, float coef, float decay,
                                          const Hyper& h) {
  g = g / d * coef;
  p *= 1.f - h.lr * decay;
  m += (g - m) * (1.f - h.beta1);
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  const float denom = sqrtf(v) / h.bc2_sqrt + h.eps;
  p -= h.step_size * (m / denom);
}

__global__ void __launch_bounds__(kOptThreads) adamw_kernel(const __grid_constant__ OptBatch batch,
                                                            const float* __restrict__ divisor,
                                                            const float* __restrict__ norm, const Hyper h) {
  const float total = norm[0], coef = norm[1];
  if (!isfinite(total)) return;                 // the caller reports the non-finite norm; nothing is stepped
  const float d = *divisor;
  const int chunks = batch.first_chunk[batch.count];
  for (int chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
    const int t = tensor_of(batch, chunk);
    const long long begin = static_cast<long long>(chunk - batch.first_chunk[t]) * kChunk;
    const long long size = batch.size[t];
    float* g = batch.grad[t] + begin;
    float* p = batch.param[t] + begin;
    float* m = batch.m[t] + begin;
    float* v = batch.v[t] + begin;
    const float decay = batch.decay[t];
    const int n = static_cast<int>(size - begin < kChunk ? size - begin : kChunk);
    if (batch.vec && n == kChunk) {
#pragma unroll 2
      for (int i = 0; i < 4; ++i) {
        const int at = i * kOptThreads + threadIdx.x;
        float4 qg = reinterpret_cast<float4*>(g)[at], qp = reinterpret_cast<float4*>(p)[at];
        float4 qm = reinterpret_cast<float4*>(m)[at], qv = reinterpret_cast<float4*>(v)[at];
        adamw_one(qg.x, qp.x, qm.x, qv.x, d, coef, decay, h);
        adamw_one(qg.y, qp.y, qm.y, qv.y, d, coef, decay, h);
        adamw_one(qg.z, qp.z, qm.z, qv.z, d, coef, decay, h);
        adamw_one(qg.w, qp.w, qm.w, qv.w, d, coef, decay, h);
        reinterpret_cast<float4*>(p)[at] = qp;
        reinterpret_cast<float4*>(m)[at] = qm;
        reinterpret_cast<float4*>(v)[at] = qv;
        if (h.write_grads) reinterpret_cast<float4*>(g)[at] = qg;
      }
    } else {
      for (int i = threadIdx.x; i < n; i += kOptThreads) {
        float sg = g[i], sp = p[i], sm = m[i], sv = v[i];
        adamw_one(sg, sp, sm, sv, d, coef, decay, h);
        p[i] = sp;
        m[i] = sm;
        v[i] = sv;
        if (h.write_grads) g[i] = sg;
      }
    }
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int launches_for(int count) { return (count + kBatch - 1) / kBatch; }

}  // namespace
}  // namespace ct

using namespace ct;

extern "C" int64_t ct_grad_norm_workspace(int count) {
  if (count <= 0) return 0;
  return static_cast<int64_t>(launches_for(count)) * kOptBlocks * sizeof(float);
}

extern "C" int ct_grad_norm(int count, void* const* grads, const int64_t* sizes, const float* divisor, float max_norm,
                            float* norm_out, void* workspace, void* stream) {
  if (count < 0) return fail(CT_ERR_ARG, "ct_grad_norm: count=%d", count);
  if (!divisor || !norm_out) return fail(CT_ERR_ARG, "ct_grad_norm: null divisor or norm_out");
  if (count && (!grads || !sizes || !workspace)) return fail(CT_ERR_ARG, "ct_grad_norm: null table or workspace");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int launches = launches_for(count);
  float* partials = static_cast<float*>(workspace);
  for (int l = 0; l < launches; ++l) {
    OptBatch batch{};
    batch.count = 0;
    batch.vec = 1;
    batch.first_chunk[0] = 0;
    for (int i = l * kBatch; i < count && i < (l + 1) * kBatch; ++i) {
      if (sizes[i] < 0) return fail(CT_ERR_ARG, "ct_grad_norm: negative size at %d", i);
      if (sizes[i] == 0) continue;
      if (!grads[i]) return fail(CT_ERR_ARG, "ct_grad_norm: null tensor at %d", i);
      const int j = batch.count++;
      batch.grad[j] = static_cast<float*>(grads[i]);
      batch.size[j] = sizes[i];
      const long long chunks = (sizes[i] + kChunk - 1) / kChunk;
      if (batch.first_chunk[j] + chunks > 0x7fffffffLL) return fail(CT_ERR_UNSUPPORTED, "ct_grad_norm: tensor too large");
      batch.first_chunk[j + 1] = batch.first_chunk[j] + static_cast<int>(chunks);
      if (!aligned16(grads[i])) batch.vec = 0;
    }
    // A batch without elements still writes its partials (zeros), so the sum below reads defined values.
    sumsq_kernel<<<kOptBlocks, kOptThreads, 0, s>>>(batch, divisor, partials + static_cast<size_t>(l) * kOptBlocks);
    count_launch(false);
  }
  norm_kernel<<<1, kOptThreads, 0, s>>>(partials, launches * kOptBlocks, max_norm, norm_out);
  count_launch(false);
  return check_launch("ct_grad_norm");
}

extern "C" int ct_adamw_update(int count, void* const* grads, void* const* params, void* const* exp_avg,
                               void* const* exp_avg_sq, const int64_t* sizes, const float* weight_decay,
                               const float* divisor, const float* norm, float lr, float beta1, float beta2, float eps,
                               int64_t step, int write_grads, void* stream) {
  if (count < 0 || step < 1) return fail(CT_ERR_ARG, "ct_adamw_update: count=%d step=%lld", count, (long long)step);
  if (!divisor || !norm) return fail(CT_ERR_ARG, "ct_adamw_update: null divisor or norm");
  if (count && (!grads || !params || !exp_avg || !exp_avg_sq || !sizes || !weight_decay))
    return fail(CT_ERR_ARG, "ct_adamw_update: null table");
  if (!(beta1 >= 0.f && beta1 < 1.f && beta2 >= 0.f && beta2 < 1.f))
    return fail(CT_ERR_ARG, "ct_adamw_update: betas %g %g", beta1, beta2);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Hyper h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps;
  h.step_size = static_cast<float>(static_cast<double>(lr) / (1.0 - pow(static_cast<double>(beta1), static_cast<double>(step))));
  h.bc2_sqrt = static_cast<float>(sqrt(1.0 - pow(static_cast<double>(beta2), static_cast<double>(step))));
  h.write_grads = write_grads;
  for (int l = 0; l < launches_for(count); ++l) {
    OptBatch batch{};
    batch.count = 0;
    batch.vec = 1;
    batch.first_chunk[0] = 0;
    for (int i = l * kBatch; i < count && i < (l + 1) * kBatch; ++i) {
      if (sizes[i] < 0) return fail(CT_ERR_ARG, "ct_adamw_update: negative size at %d", i);
      if (sizes[i] == 0) continue;
      if (!grads[i] || !params[i] || !exp_avg[i] || !exp_avg_sq[i])
        return fail(CT_ERR_ARG, "ct_adamw_update: null tensor at %d", i);
      const int j = batch.count++;
      batch.grad[j] = static_cast<float*>(grads[i]);
      batch.param[j] = static_cast<float*>(params[i]);
      batch.m[j] = static_cast<float*>(exp_avg[i]);
      batch.v[j] = static_cast<float*>(exp_avg_sq[i]);
      batch.decay[j] = weight_decay[i];
      batch.size[j] = sizes[i];
      const long long chunks = (sizes[i] + kChunk - 1) / kChunk;
      if (batch.first_chunk[j] + chunks > 0x7fffffffLL) return fail(CT_ERR_UNSUPPORTED, "ct_adamw_update: tensor too large");
      batch.first_chunk[j + 1] = batch.first_chunk[j] + static_cast<int>(chunks);
      if (!(aligned16(grads[i]) && aligned16(params[i]) && aligned16(exp_avg[i]) && aligned16(exp_avg_sq[i])))
        batch.vec = 0;
    }
    if (batch.count == 0) continue;
    adamw_kernel<<<kOptBlocks, kOptThreads, 0, s>>>(batch, divisor, norm, h);
    count_launch(false);
  }
  return check_launch("ct_adamw_update");
}
