// Internal declarations shared by the kernels of libct_b200.so.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ct_b200.h"

namespace ct {

// ---- error text + launch accounting (api.cu) --------------------------------
int fail(int code, const char* fmt, ...);
void count_launch(bool tcgen05);
int check_launch(const char* what);
// Per-device int the kernels raise when a bounded wait gives up.
int* device_error_flag();
// Optional per-launch timing of the tcgen05 GEMM (CUDA events on the launching stream).
bool timing_enabled();
void timing_begin(cudaStream_t stream);
void timing_end(cudaStream_t stream, double flops, long long m, long long n, long long k);

// ---- programmatic dependent launch ---------------------------------------------
// A kernel launched through launch_dependent() may be scheduled while the previous kernel of the
// stream is still running: its prologue overlaps that kernel's tail, and grid_dependency_wait()
// then blocks until the previous kernel has completed and its writes are visible. Only kernels
// that call grid_dependency_wait() before their first access to global memory may be launched
// this way. CT_B200_PDL=0 in the environment turns the attribute off (plain stream order).
bool dependent_launch_enabled();

__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled() ? 1 : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// ---- dtype helpers ------------------------------------------------------------
__host__ __device__ inline int dtype_size(int dtype) { return dtype == CT_F32 ? 4 : 2; }

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

// Round an fp32 value to T and widen it back.
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_float<T>(from_float<T>(v)); }

__device__ __forceinline__ float load_as_float(const void* p, int64_t i, int dtype) {
  if (dtype == CT_F32) return static_cast<const float*>(p)[i];
  if (dtype == CT_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void* p, int64_t i, int dtype, float v) {
  if (dtype == CT_F32) static_cast<float*>(p)[i] = v;
  else if (dtype == CT_BF16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(p)[i] = __float2half_rn(v);
}

__device__ __forceinline__ float round_dtype(float v, int dtype) {
  if (dtype == CT_F32) return v;
  if (dtype == CT_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return __half2float(__float2half_rn(v));
}

// ---- SwiGLU, one element (kernels/mlp_cuda.py:10-25 of the reference) -----------------
// h = round(silu(g)) * u; backward: d_gate = round(grad * u) * sigmoid'(g)-term, d_up = grad * round(silu(g)).
// Shared by the stand-alone kernel and the GEMM epilogue that applies it to accumulator tiles, which have to
// agree bit for bit: every product and the one fused multiply-add are spelled out, so the compiler has no
// contraction of its own to decide.
template <typename T>
__device__ __forceinline__ void swiglu_element(float g, float u, float grad, bool backward, bool reconstruct,
                                               float& h, float& dg, float& du) {
  // 16-bit activations: the exponential and the reciprocal come from the special-function unit
  // (relative error about 2^-21, far below the 8 or 11 mantissa bits the results are rounded to);
  // the kernels are bound by instruction issue, not by HBM, with the full-precision forms.
  float sig;
  if constexpr (sizeof(T) == 2) sig = __fdividef(1.0f, __fadd_rn(1.0f, __expf(-g)));
  else sig = 1.0f / (1.0f + expf(-g));
  const float activated = round_to<T>(__fmul_rn(g, sig));
  if (backward) {
    const float product_grad = round_to<T>(__fmul_rn(grad, u));
    dg = __fmul_rn(product_grad, __fmul_rn(sig, __fmaf_rn(g, __fsub_rn(1.0f, sig), 1.0f)));
    du = __fmul_rn(grad, activated);
  }
  if (reconstruct) h = __fmul_rn(activated, u);
}

// ---- GEMM description shared by the SIMT and tcgen05 kernels ------------------
// D[M, N] = (beta ? D : 0) + sum over segments s of A_s[M, k_s] * B_s[k_s, N] + bias[N]
// then (optionally)  D = round(D) + residual, rounded again.
// Element (m, k) of A_s is at a[m * a_rs + k * a_cs]; element (k, n) of B_s at
// b[k * b_rs + n * b_cs]. One stride of each pair is 1.
constexpr int kMaxSegments = 6;

struct Segment {
  const void* a;
  int64_t a_rs, a_cs;
  const void* b;
  int64_t b_rs, b_cs;
  int64_t k;
};

struct GemmArgs {
  int64_t M, N;
  int nseg;
  Segment seg[kMaxSegments];
  int in_dtype;        // CT_BF16 / CT_F32 (SIMT only) for every A_s and B_s
  void* out;
  int64_t ldo;
  int out_dtype;
  int beta;            // 1: accumulate onto the existing `out`
  const void* bias;    // [N] in in_dtype, or null
  const void* residual;  // [M, N] in out_dtype, or null
  int64_t ld_res;
  int split_k;         // >1: slice s writes fp32 partials to out + s*M*ldo (tcgen05, 1 segment)
};

int gemm_simt(const GemmArgs& g, cudaStream_t stream);
// Returns CT_ERR_UNSUPPORTED (without launching) when a TMA rule is not met.
int gemm_tcgen05(const GemmArgs& g, cudaStream_t stream);
bool gemm_tcgen05_supported(const GemmArgs& g);
// Several independent products (at most 6) in ONE launch of the CTA-pair kernel; each must be supported.
int gemm_tcgen05_group(const GemmArgs* problems, int count, cudaStream_t stream);
int gemm_dispatch(const GemmArgs& g, int path, cudaStream_t stream);
// out[T, N] = x[T, K] . dequant(W)^T with the NF4 decode of W[N, K] inside the tcgen05 kernel (bf16, blocks of 64).
bool gemm_tcgen05_nf4_supported(const void* x, int64_t ldx, const void* packed, const void* absmax, const void* code,
                                const void* out, int64_t ldo, int64_t T, int64_t K, int64_t N);
int gemm_tcgen05_nf4(const void* x, int64_t ldx, const uint8_t* packed, const float* absmax, const float* code,
                     void* out, int64_t ldo, int64_t T, int64_t K, int64_t N, cudaStream_t stream);
// SwiGLU MLP in the tcgen05 kernel (bf16). `w_pair` is the gate and up weights interleaved in 128-row blocks
// ([2 N, K]); xa_* are the low-rank inputs x . a^T, b_* the [N, r] adapter outputs.
struct GatedArgs {
  const void* x; int64_t ldx;
  const void* w_pair; int64_t ldw;
  const void* xa_gate; const void* xa_up; int64_t ld_xa;
  const void* b_gate; const void* b_up;
  int64_t T, K, N, r_gate, r_up;
  void* h;            // [T, N]: silu(gate) * up
  void* gate;         // forward: gate(x) or null; backward: d_gate
  void* up;           // forward: up(x) or null; backward: d_up
  const void* dh;     // null = forward; else the gradient of h (may be the same buffer as h)
  int64_t ld_out;     // leading dimension of h, gate, up and dh
};
bool gemm_tcgen05_gated_supported(const GatedArgs& a);
int gemm_tcgen05_gated(const GatedArgs& a, cudaStream_t stream);
struct GatedGradientArgs {
  const void* dg; const void* du; int64_t ld_signal;
  const void* w_pair; int64_t ldw;
  const void* low_gate; const void* low_up; int64_t ld_low;
  const void* a_gate; const void* a_up;      // [r, K] row-major
  int64_t T, K, N, r_gate, r_up;
  void* dx; int64_t ld_dx;
  int add;
};
int gemm_tcgen05_gated_input_gradient(const GatedGradientArgs& a, cudaStream_t stream);
struct GatedDownArgs {
  const void* dy; int64_t ld_dy;           // [T, N]: gradient of the following projection's output
  const void* w; int64_t ldw;              // [N, K]: that projection's base weight (K = width of the SwiGLU)
  const void* a;                           // [r, K]
  const void* low; int64_t ld_low;         // [T, r] = dy . b
  const void* gate; const void* up; int64_t ld_saved;    // [T, K], kept by the forward pass
  void* d_gate; void* d_up; void* hidden; int64_t ld_out;  // [T, K] outputs
  int64_t T, K, N, r;
};
int gemm_tcgen05_gated_down_gradient(const GatedDownArgs& a, cudaStream_t stream);
// Launches one thread that waits `limit_us` on a barrier nothing completes and reports it (gemm_tc.cu).
int bounded_wait_selftest(int64_t limit_us, cudaStream_t stream);

// out[i] = (add ? out[i] : 0) + partial[0][i] + partial[1][i] + ... in that order.
int reduce_partials(const float* partials, int slices, int64_t rows, int64_t cols, int64_t ld_partial,
                    float* out, int64_t ld_out, int add, cudaStream_t stream);

}  // namespace ct
