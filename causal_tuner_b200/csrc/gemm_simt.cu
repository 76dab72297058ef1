// Shape-generic SIMT matrix product: any M, N, K, any element strides, fp32 or
// 16-bit operands, fp32 accumulation. It serves the shapes the tcgen05 kernel
// cannot take (fp32 compute dtype, leading dimensions that break the 16-byte
// TMA stride rule such as rank 3/5/7 adapters or 68-wide rows, unaligned views)
// so that every call still runs on the GPU. Correctness first: 64x64 output tile
// per CTA, 16-deep shared-memory slices, 4x4 register tile per thread.
#include "common.cuh"

namespace ct {
namespace {

constexpr int TM = 64, TN = 64, TK = 16, kThreads = 256;

struct SimtParams {
  GemmArgs g;
};

template <typename InT>
__device__ __forceinline__ float fetch(const void* base, int64_t index) {
  return to_float<InT>(static_cast<const InT*>(base)[index]);
}

template <typename InT>
__global__ void __launch_bounds__(kThreads) gemm_simt_kernel(const SimtParams p) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const GemmArgs& g = p.g;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * TM, n0 = static_cast<int64_t>(blockIdx.x) * TN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int s = 0; s < g.nseg; ++s) {
    const Segment& seg = g.seg[s];
    const bool a_k_contig = seg.a_cs == 1, b_k_contig = seg.b_rs == 1;
    for (int64_t k0 = 0; k0 < seg.k; k0 += TK) {
#pragma unroll
      for (int j = 0; j < (TM * TK) / kThreads; ++j) {
        const int idx = threadIdx.x + kThreads * j;
        const int mm = a_k_contig ? idx / TK : idx % TM, kk = a_k_contig ? idx % TK : idx / TM;
        const int64_t m = m0 + mm, k = k0 + kk;
        As[kk][mm] = (m < g.M && k < seg.k) ? fetch<InT>(seg.a, m * seg.a_rs + k * seg.a_cs) : 0.0f;
      }
#pragma unroll
      for (int j = 0; j < (TN * TK) / kThreads; ++j) {
        const int idx = threadIdx.x + kThreads * j;
        const int nn = b_k_contig ? idx / TK : idx % TN, kk = b_k_contig ? idx % TK : idx / TN;
        const int64_t n = n0 + nn, k = k0 + kk;
        Bs[kk][nn] = (n < g.N && k < seg.k) ? fetch<InT>(seg.b, k * seg.b_rs + n * seg.b_cs) : 0.0f;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < TK; ++kk) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      if (g.beta) v += load_as_float(g.out, m * g.ldo + n, g.out_dtype);
      if (g.bias) v += load_as_float(g.bias, n, g.in_dtype);
      if (g.residual)
        v = __fadd_rn(round_dtype(v, g.out_dtype), load_as_float(g.residual, m * g.ld_res + n, g.out_dtype));
      store_from_float(g.out, m * g.ldo + n, g.out_dtype, v);
    }
  }
}

}  // namespace

int gemm_simt(const GemmArgs& g, cudaStream_t stream) {
  if (g.M == 0 || g.N == 0) return CT_OK;
  if (g.split_k > 1) return fail(CT_ERR_UNSUPPORTED, "gemm_simt: split contraction is a tcgen05 feature");
  const int64_t gx = (g.N + TN - 1) / TN, gy = (g.M + TM - 1) / TM;
  if (gy > 65535) {
    // Walk row bands so that gridDim.y stays within its limit.
    const int64_t band = 65535LL * TM;
    for (int64_t start = 0; start < g.M; start += band) {
      GemmArgs part = g;
      part.M = (g.M - start < band) ? g.M - start : band;
      for (int s = 0; s < g.nseg; ++s)
        part.seg[s].a = static_cast<const char*>(g.seg[s].a) + start * g.seg[s].a_rs * dtype_size(g.in_dtype);
      part.out = static_cast<char*>(g.out) + start * g.ldo * dtype_size(g.out_dtype);
      if (g.residual)
        part.residual = static_cast<const char*>(g.residual) + start * g.ld_res * dtype_size(g.out_dtype);
      const int rc = gemm_simt(part, stream);
      if (rc != CT_OK) return rc;
    }
    return CT_OK;
  }
  SimtParams p{g};
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  if (g.in_dtype == CT_F32) gemm_simt_kernel<float><<<grid, kThreads, 0, stream>>>(p);
  else if (g.in_dtype == CT_BF16) gemm_simt_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(p);
  else if (g.in_dtype == CT_F16) gemm_simt_kernel<__half><<<grid, kThreads, 0, stream>>>(p);
  else return fail(CT_ERR_ARG, "gemm_simt: dtype %d", g.in_dtype);
  count_launch(false);
  return check_launch("gemm_simt");
}

}  // namespace ct
