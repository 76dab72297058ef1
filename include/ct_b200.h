/*
 * C ABI of libct_b200.so: the B200 (sm_100a) kernels behind causal-tuner's
 * fused projection / SwiGLU-MLP operator layer.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer on the
 *     current CUDA device unless a comment says otherwise;
 *   - the caller owns every buffer (inputs, outputs and workspaces);
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *     kernels are enqueued on it and the call returns without synchronising;
 *   - the return value is CT_OK (0) or a negative CT_ERR_* code; nothing is
 *     thrown across the boundary;
 *   - matrices are row-major with an explicit leading dimension in ELEMENTS;
 *   - `dtype` arguments take the CT_F32 / CT_BF16 / CT_F16 codes below;
 *   - there is no CPU fallback: without a CUDA device every compute entry
 *     point returns CT_ERR_CUDA.
 *
 * Each declaration cites the reference function (path inside the
 * causal-tuner project : line) whose arithmetic it replaces.
 */
#ifndef CT_B200_H
#define CT_B200_H

#include <stdint.h>

#if defined(__GNUC__)
#define CT_API __attribute__((visibility("default")))
#else
#define CT_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum { CT_F32 = 0, CT_BF16 = 1, CT_F16 = 2 };

enum {
  CT_OK = 0,
  CT_ERR_ARG = -1,          /* null pointer, negative size, unknown dtype */
  CT_ERR_UNSUPPORTED = -2,  /* shape/alignment the requested path cannot take */
  CT_ERR_CUDA = -3,         /* a CUDA runtime/driver call failed */
  CT_ERR_DEVICE = -4        /* a kernel reported a bounded-wait timeout */
};

/* GEMM path selection. AUTO picks the tcgen05 kernel when every operand meets
 * the TMA rules (bf16, 16-byte aligned base, leading dimension a multiple of
 * 8 elements) and falls back to the shape-generic SIMT kernel otherwise. Both
 * run on the GPU. */
enum { CT_PATH_AUTO = 0, CT_PATH_SIMT = 1, CT_PATH_TCGEN05 = 2 };

/* ---- library state ------------------------------------------------------ */

/* ABI version of this header. */
CT_API int ct_abi_version(void);
/* Kernels launched by this library in this process so far (all devices). */
CT_API int64_t ct_launch_count(void);
/* Kernels among those that were the tcgen05 GEMM. */
CT_API int64_t ct_tcgen05_launch_count(void);
/* Synchronises `stream`, then returns CT_OK, or CT_ERR_DEVICE when a kernel on
 * the current device gave up on a bounded wait since the last call (the flag is
 * cleared), or CT_ERR_CUDA with the sticky CUDA error. */
CT_API int ct_check_device(void* stream);
/* Per-launch timing of the tcgen05 GEMM, for roofline reports. While enabled,
 * every launch is bracketed by CUDA events recorded on the launching stream.
 * ct_timing_enable(on) clears what was recorded and switches recording on/off;
 * ct_timing_collect waits for the recorded launches and returns their summed
 * device time (ms), their summed algorithmic work (2*M*N*K FLOP per launch, true
 * sizes, no padding) and their number, then clears the record. No counterpart in
 * the reference (it times whole steps only, train.py:219-223). */
CT_API int ct_timing_enable(int on);
CT_API int ct_timing_collect(double* total_ms, double* total_flops, int64_t* launches);
/* Self-test of the failure path, no counterpart in the reference: enqueues one thread that waits
 * `limit_us` microseconds (1 .. 100000) on an mbarrier that nothing ever completes, using the
 * GEMM's bounded wait; it gives up, raises the per-device error flag and returns. The next
 * ct_check_device on that device then returns CT_ERR_DEVICE and clears the flag; the context
 * stays usable. Nothing faults, traps or spins without a limit. */
CT_API int ct_selftest_bounded_wait(int64_t limit_us, void* stream);
/* Text of the most recent CT_ERR_* on the calling thread (static storage). */
CT_API const char* ct_last_error(void);

/* ---- NF4 decode ---------------------------------------------------------
 * Replaces kernels/nf4_cuda.py:32-43 (dequantize_nf4) and its Triton kernel
 * kernels/nf4_cuda.py:9-29.
 *   out[blocksize*g + 2j]   = code[packed[..] >> 4] * s_g
 *   out[blocksize*g + 2j+1] = code[packed[..] & 15] * s_g
 * s_g = absmax[g] (fp32) when nested == 0, else
 * s_g = code2[absmax_u8[g]] * absmax2[g / blocksize2] + offset[0], the multiply
 * and the add rounded separately. The fp32 product is rounded to `state_dtype`
 * and then to `out_dtype`. `n` elements, (n+1)/2 packed bytes. `blocksize`
 * must be even. When nested != 0 `absmax` points at uint8 values. */
CT_API int ct_nf4_decode(const uint8_t* packed, const void* absmax, const float* code,
                  const float* code2, const float* absmax2, const float* offset,
                  void* out, int64_t n, int blocksize, int blocksize2, int nested,
                  int state_dtype, int out_dtype, void* stream);

/* The same decode with the output written in runs: element e goes to out[(e / chunk) * pitch + e % chunk].
 * With chunk = 128 * K and pitch = 256 * K two [N, K] weights decode into one [2 N, K] buffer of interleaved
 * 128-row blocks (the second with `out` advanced by 128 * K elements): the B operand of ct_gated_forward.
 * `chunk` and `pitch` are multiples of 8 elements, pitch >= chunk. */
CT_API int ct_nf4_decode_chunks(const uint8_t* packed, const void* absmax, const float* code,
                  const float* code2, const float* absmax2, const float* offset,
                  void* out, int64_t n, int blocksize, int blocksize2, int nested,
                  int state_dtype, int out_dtype, int64_t chunk, int64_t pitch, void* stream);

/* The same decode written TRANSPOSED: W[rows, cols] (packed row-major) -> out[cols, rows] (bf16, leading dimension
 * ld_out), through 64 x 64 shared-memory tiles so that both the packed reads and the transposed writes are whole
 * sectors. For the backward pass: dx = dy @ W contracts over the rows of W, and with this storage W is the K-major
 * operand of that GEMM (pass it to ct_input_gradient with strides (1, ld_out)). Same values as ct_nf4_decode.
 * rows and cols multiples of 64, blocksize a multiple of 16, bf16 output; else CT_ERR_UNSUPPORTED. */
CT_API int ct_nf4_decode_transposed(const uint8_t* packed, const void* absmax, const float* code,
                  const float* code2, const float* absmax2, const float* offset, void* out,
                  int64_t rows, int64_t cols, int64_t ld_out, int blocksize, int blocksize2,
                  int nested, int state_dtype, int out_dtype, void* stream);

/* ---- NF4 encode ---------------------------------------------------------
 * Replaces the bitsandbytes quantiser the reference calls when it installs a frozen base
 * weight (modeling/lora.py:41-56, `Params4bit(..., quant_type="nf4", compress_statistics=True)`).
 * ct_nf4_encode: for each block g of `blocksize` consecutive elements of weight[n] (`dtype`):
 *   absmax[g] = max |w|;  index(w) = number of midpoints (code[i] + code[i+1]) / 2 strictly
 *   below w / max(absmax[g], FLT_MIN);  packed[j] = index(w[2j]) << 4 | index(w[2j+1]);
 *   elements past n count as 0. (n+1)/2 packed bytes, ceil(n / blocksize) absmax values.
 *   `blocksize` is a power of two from 8 to 256 (CT_ERR_UNSUPPORTED otherwise).
 * ct_nf4_nest: nested statistics of `blocks` absmax values:
 *   offset[0] = mean(absmax) (fp64 accumulation in a fixed order, rounded to fp32);
 *   absmax2[h] = max |absmax - offset| over group h of `blocksize2` values;
 *   quantised[g] = number of midpoints of the 256-entry table `code2` strictly below
 *   (absmax[g] - offset) / max(absmax2[h], FLT_MIN).
 * ct_nf4_decode inverts both. All pointers are device memory. */
CT_API int ct_nf4_encode(const void* weight, int64_t n, int dtype, int blocksize, const float* code,
                         uint8_t* packed, float* absmax, void* stream);
CT_API int ct_nf4_nest(const float* absmax, int64_t blocks, int blocksize2, const float* code2,
                       uint8_t* quantised, float* absmax2, float* offset, void* stream);

/* ---- dtype cast ---------------------------------------------------------
 * Replaces the per-call `a.to(dtype)`, `b.to(dtype)`, `bias.to(dtype)` casts of
 * kernels/linear.py:70-71 and kernels/mlp_cuda.py:62. src[rows, cols] (ld_src)
 * -> dst[rows, cols] (ld_dst), round-to-nearest-even. */
CT_API int ct_cast(const void* src, int src_dtype, int64_t ld_src, void* dst, int dst_dtype,
            int64_t ld_dst, int64_t rows, int64_t cols, void* stream);
/* The same casts for `count` contiguous tensors in one launch (all the adapters an operator
 * needs in the compute dtype). `src`, `dst` and `sizes` (elements) are HOST arrays. */
CT_API int ct_cast_many(int count, const void* const* src, void* const* dst, const int64_t* sizes,
                        int src_dtype, int dst_dtype, void* stream);

/* ---- generic matrix product --------------------------------------------
 * Replaces kernels/linear.py:16-24 (accumulate) and the bare torch.mm calls at
 * kernels/linear.py:83,124,125 and kernels/mlp_cuda.py:134,139.
 *   C[m, n] = (add ? C[m, n] : 0) + sum_k A(m, k) * B(k, n)
 * A(m, k) = A[m * a_rs + k * a_cs], B(k, n) = B[k * b_rs + n * b_cs] (element
 * strides, one of each pair must be 1). fp32 accumulation; `in_dtype` is the
 * type of A and B, `out_dtype` that of C. With add == 0, C is never read. */
CT_API int ct_matmul(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs,
              int64_t b_cs, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
              int in_dtype, int out_dtype, int add, int path, void* stream);

/* ---- base product with the NF4 decode inside the GEMM -------------------------------
 * Replaces `materialize` + the base product of kernels/linear.py:29 (`dequantize_nf4`, kernels/nf4_cuda.py:32-43,
 * then torch.mm) for callers that do not want the dense weight to exist:
 *   out[T, N] = round(x[T, K] @ W^T),  W[n, k] = round(code[nibble(n, k)] * absmax[(n * K + k) / 64])
 * with the decode arithmetic of ct_nf4_decode (fp32 product rounded once to bf16; bit-identical values).
 * Four extra warps per CTA turn 128-bit loads of packed codes into the swizzled shared-memory B tiles that the
 * tcgen05 MMAs read; x tiles arrive by TMA. The result is bit-identical to ct_nf4_decode followed by ct_matmul.
 * Every row tile of x decodes the weight again, so this form pays for small T only (a few hundred tokens);
 * the training path decodes once per call instead (see ct_nf4_decode). bf16, `blocksize` 64, fp32 absmax
 * (not nested), K a multiple of 64, rows of x and the packed codes 16-byte aligned; anything else returns
 * CT_ERR_UNSUPPORTED and the caller decodes first. */
CT_API int ct_matmul_nf4(const void* x, int64_t ldx, const uint8_t* packed, const float* absmax,
                         const float* code, void* out, int64_t ld_out, int64_t T, int64_t K, int64_t N,
                         int blocksize, int dtype, void* stream);

/* ---- fused projection forward --------------------------------------------
 * Replaces kernels/linear.py:27-33 (forward_linear) plus the in-place residual
 * add of kernels/linear.py:90-91.
 *   xa  = round(x @ a^T)                                   [T, r]
 *   out = round(round(x @ w^T + xa @ b^T + bias) + residual)   [T, N]
 * x[T,K] (ldx), w[N,K] dense (ldw), a[r,K], b[N,r] contiguous, bias[N] or NULL,
 * residual[T,N] (ld_res) or NULL; all of `dtype` (CT_BF16 or CT_F32). The
 * low-rank term enters the same accumulator as the base product (one GEMM over
 * the concatenated contraction [x | xa] . [w | b]^T), so `out` is rounded once
 * where the reference rounds after the base product and again after the
 * low-rank update. r may be 0 (a, b, xa ignored). With r > 0 and a == NULL, `xa`
 * is an INPUT that already holds round(x @ a^T) - projections that share x compute
 * their low-rank inputs in one stacked product (ct_matmul with the a matrices
 * stacked row-wise) and pass column slices of the result (ld_xa = total rank). */
CT_API int ct_forward_linear(const void* x, int64_t ldx, const void* w, int64_t ldw,
                      const void* a, const void* b, const void* bias,
                      const void* residual, int64_t ld_res, void* out, int64_t ld_out,
                      void* xa, int64_t ld_xa, int64_t T, int64_t K, int64_t N,
                      int64_t r, int dtype, int path, void* stream);

/* ---- fused input gradient ---------------------------------------------------
 * Replaces kernels/linear.py:36-39 (input_gradient).
 *   low = round(dy @ b)                                        [T, r]
 *   dx  = round((add ? dx : 0) + dy @ w + low @ a)             [T, K]
 * dy[T,N] (ld_dy), a[r,K], b[N,r] contiguous. Element (n, k) of w[N,K] is at w[n * w_rs + k * w_cs] (element
 * strides, one of them 1): (ld, 1) for the row-major weight, (1, ld) for a weight that was decoded transposed
 * (ct_nf4_decode_transposed) - the contraction of this product runs over n, so the transposed storage is the
 * K-major operand the tensor core reads fastest; the values are the same either way. `w` may be NULL:
 * then only `low` is written (kernels/linear.py:124). `b` may be NULL with r > 0:
 * then `low` is an INPUT that already holds round(dy @ b) (a caller that computed it
 * while the base weight was still being decoded on another stream). */
CT_API int ct_input_gradient(const void* dy, int64_t ld_dy, const void* w, int64_t w_rs, int64_t w_cs,
                      const void* a, const void* b, void* dx, int64_t ld_dx,
                      void* low, int64_t ld_low, int64_t T, int64_t K, int64_t N,
                      int64_t r, int add, int dtype, int path, void* stream);

/* ---- fused input gradient of a projection group ---------------------------------
 * Replaces the per-projection accumulation `add=index > 0` of kernels/linear.py:122 for the
 * projections that share one input (q/k/v, gate/up): `count` (1..3) projections,
 *   low_i = round(dy_i @ b_i)                                             [T, r_i]
 *   dx    = round((add ? dx : 0) + sum_i (dy_i @ w_i + low_i @ a_i))      [T, K]
 * in ONE GEMM over the concatenated contraction [dy_0 | low_0 | dy_1 | low_1 | ...], so dx is
 * written (and rounded) once instead of being re-read and re-rounded per projection. Arrays of
 * `count` device pointers / sizes live in HOST memory. dy_i[T, N_i], w_i[N_i, K] with element strides
 * (w_rs[i], w_cs[i]) as in ct_input_gradient, a_i[r_i, K], b_i[N_i, r_i] contiguous. */
CT_API int ct_input_gradient_group(int count, const void* const* dy, const int64_t* ld_dy,
                                   const void* const* w, const int64_t* w_rs, const int64_t* w_cs,
                                   const void* const* a,
                                   const void* const* b, const int64_t* N, const int64_t* r, void* dx,
                                   int64_t ld_dx, void* const* low, const int64_t* ld_low, int64_t T,
                                   int64_t K, int add, int dtype, int path, void* stream);

/* ---- LoRA parameter gradients ----------------------------------------------
 * Replaces kernels/linear.py:42-44 (parameter_gradients).
 *   da[r, K] = (add ? da : 0) + low^T @ x     fp32
 *   db[N, r] = (add ? db : 0) + dy^T  @ xa    fp32
 * Deterministic: the contraction over T is split into a fixed number of
 * slices whose fp32 partial sums are added in slice order (no atomics).
 * `workspace` must hold ct_parameter_gradients_workspace(...) bytes (may be
 * NULL when that is 0). */
CT_API int64_t ct_parameter_gradients_workspace(int64_t T, int64_t K, int64_t N, int64_t r,
                                         int dtype, int path);
CT_API int ct_parameter_gradients(const void* x, int64_t ldx, const void* dy, int64_t ld_dy,
                           const void* low, int64_t ld_low, const void* xa,
                           int64_t ld_xa, float* da, float* db, int64_t T, int64_t K,
                           int64_t N, int64_t r, int add, int dtype, void* workspace,
                           int path, void* stream);

/* ---- token-contracted fp32 accumulation ------------------------------------
 * Replaces kernels/linear.py:16-24 (accumulate) as parameter_gradients uses it
 * (kernels/linear.py:42-44, `accumulate(da, low.T, x)`):
 *   out[rows, cols] = (add ? out : 0) + left^T @ right     fp32, out contiguous
 * left[T, rows] (ld_left), right[T, cols] (ld_right) of `dtype`. Same fixed-order
 * slicing of the contraction over T as ct_parameter_gradients, which is this call
 * twice; with the low matrices of several projections stacked column-wise in
 * `left`, one call yields their stacked dA. `workspace` holds
 * ct_accumulate_workspace(...) bytes (NULL when that is 0). */
CT_API int64_t ct_accumulate_workspace(int64_t rows, int64_t cols, int64_t T, int dtype, int path);
CT_API int ct_accumulate(const void* left, int64_t ld_left, const void* right, int64_t ld_right,
                         float* out, int64_t rows, int64_t cols, int64_t T, int add, int dtype,
                         void* workspace, int path, void* stream);

/* ---- several token-contracted accumulations in one launch -------------------------
 * `count` independent products out_i[rows_i, cols_i] = (add_i ? out_i : 0) + left_i^T @ right_i over the same T
 * tokens - the dA and dB of the projections of one operator (kernels/linear.py:42-44 called once per
 * projection at kernels/linear.py:126 and kernels/mlp_cuda.py:135-141). Same arithmetic as `count` calls of
 * ct_accumulate; with 2 to 6 products whose operands meet the tensor-core rules they run as ONE persistent
 * launch that walks the concatenated tile lists, so that products with fewer tiles than the machine has
 * CTA pairs share its waves instead of each ending in a partial one. One slice count for the whole group
 * (a function of the shapes alone; fp32 partial planes summed in slice order), so results are reproducible.
 * The pointer tables, `ld_*`, `rows`, `cols` and `add` are HOST arrays of length `count`; `workspace` holds
 * ct_token_gradients_group_workspace(...) bytes (NULL when that is 0). */
CT_API int64_t ct_token_gradients_group_workspace(int count, const int64_t* rows, const int64_t* cols,
                                                  int64_t T, int dtype, int path);
CT_API int ct_token_gradients_group(int count, const void* const* left, const int64_t* ld_left,
                                    const void* const* right, const int64_t* ld_right, float* const* out,
                                    const int64_t* rows, const int64_t* cols, int64_t T, const int* add,
                                    int dtype, void* workspace, int path, void* stream);

/* ---- LoRA parameter gradients for callers that must not allocate ---------------
 * No counterpart in the reference (its gradients go through torch's caching
 * allocator, kernels/linear.py:102). Same arithmetic, same fixed summation order
 * and bit-identical results as ct_parameter_gradients, but the slice scratch is
 * a fixed array inside the library image instead of a caller-provided workspace,
 * and the call performs no cudaMalloc / cudaFree (nor any allocating library
 * routine). It is meant for hosts that cannot allocate device memory at this
 * point: a runtime that handed the whole GPU to its own memory pool at start-up
 * (a raw cudaMalloc would then fail), or a step loop that cannot accept the
 * device-wide synchronisation a cudaMalloc or cudaFree implies.
 *   - Capacity: ct_parameter_gradients_noalloc_capacity() bytes (16 MiB, e.g. the
 *     four slices of a rank-256 gradient over 4096 columns). A problem whose
 *     ct_parameter_gradients_workspace(...) exceeds it is refused with
 *     CT_ERR_UNSUPPORTED and nothing is launched.
 *   - The FIRST call on a device is a set-up call: it resolves the array's device
 *     address (cudaGetSymbolAddress), and because CUDA loads code lazily it is also
 *     the moment the driver places the library's image - the 16 MiB array and the
 *     GEMM kernels - on that device, which takes device memory once and can fail with
 *     CT_ERR_CUDA if none is left. Make one warm-up call per device at start-up
 *     (any small problem; r = 0 resolves the addresses and launches nothing), before
 *     the host's pool takes the rest of the memory and before any stream capture.
 *     From then on the device holds the array until the process exits and later
 *     calls change neither free nor allocated device memory.
 *   - All calls share the one array and it keeps the previous call's partial
 *     sums; nothing in it needs clearing (every slice is fully overwritten before
 *     it is read), but two calls whose kernels overlap on the GPU (different
 *     streams, or several host threads) race on it. Keep calls on one stream or
 *     order them with events. */
CT_API int64_t ct_parameter_gradients_noalloc_capacity(void);
CT_API int ct_parameter_gradients_noalloc(const void* x, int64_t ldx, const void* dy,
                                   int64_t ld_dy, const void* low, int64_t ld_low,
                                   const void* xa, int64_t ld_xa, float* da, float* db,
                                   int64_t T, int64_t K, int64_t N, int64_t r, int add,
                                   int dtype, int path, void* stream);

/* ---- SwiGLU activation ------------------------------------------------------
 * Replaces kernels/mlp_cuda.py:10-35 (_activation / activation) and the
 * separate-output backward of kernels/mlp_cuda.py:45-51.
 * forward (grad == NULL):  out = round_d(g * sigmoid(g)) * u
 * backward (grad != NULL): dg = round_d(grad * u) * sigmoid(g) * (1 + g * (1 - sigmoid(g)))
 *                          du = grad * round_d(g * sigmoid(g))
 *   and, when `reconstruct`, h = round_d(g * sigmoid(g)) * u is written to `out`.
 * round_d rounds to `dtype`. `dg`/`du`/`out` may alias `gate`/`up`/`grad`
 * element for element (the in-place use of kernels/mlp_cuda.py:133). */
CT_API int ct_swiglu(const void* gate, const void* up, const void* grad, void* out, void* dg,
              void* du, int64_t n, int dtype, int reconstruct, void* stream);

/* ---- gate / up projections with the SwiGLU inside the GEMM ---------------------------------
 * Replaces, in one launch each, the gate and up projections plus the activation between them and the down
 * projection: kernels/mlp_cuda.py:69-73 (forward: two forward_linear calls, then `activation`) and
 * kernels/mlp_cuda.py:118-133 (backward without cached activations: the same two projections recomputed,
 * then `activation(gate, up, hidden_grad)` in place).
 * `w_pair` [2 N, K] holds both base weights, interleaved in 128-row blocks: rows [256 t, 256 t + 128) are
 * rows [128 t, 128 t + 128) of the gate weight, the next 128 rows the same rows of the up weight
 * (ct_nf4_decode_chunks writes that layout). A tile of the tcgen05 kernel then accumulates 128 columns of
 * gate(x) and the same 128 columns of up(x) side by side - base product over `w_pair`, the two low-rank terms
 * xa_gate @ b_gate^T and xa_up @ b_up^T by MMAs of half the width into their half of the accumulator - and
 * the epilogue rounds both to bf16 as stored projection outputs would be and applies ct_swiglu's arithmetic:
 *   ct_gated_forward:  h = round(silu(gate)) * up; `gate` / `up` (NULL allowed) receive the two projections
 *                      for callers that keep them for the backward pass.
 *   ct_gated_backward: with `dh` = gradient of h: (d_gate, d_up, h) as ct_swiglu's in-place backward, written
 *                      to (`d_gate`, `d_up`, `h`); gate and up exist in the accumulator only. `h` may be `dh`.
 * Results are bit-identical to ct_forward_linear x 2 + ct_swiglu. xa_* are [T, r_*] with leading dimension
 * ld_xa, b_* are [N, r_*] contiguous, h / gate / up / dh are [T, N] with leading dimension ld_out. bf16 only,
 * N a multiple of 128, rows 16-byte aligned; anything else returns CT_ERR_UNSUPPORTED (nothing launched).
 * ct_gated_input_gradient: dx[T, K] = (add ? dx : 0) + d_gate @ W_gate + low_gate @ a_gate + d_up @ W_up +
 *   low_up @ a_up with the two base weights read from `w_pair` (kernels/mlp_cuda.py:136-138 in one GEMM);
 *   low_* = d_* @ b_* are inputs. */
CT_API int ct_gated_forward(const void* x, int64_t ldx, const void* w_pair, int64_t ldw, const void* xa_gate,
                            const void* xa_up, int64_t ld_xa, const void* b_gate, const void* b_up, void* h,
                            void* gate, void* up, int64_t ld_out, int64_t T, int64_t K, int64_t N,
                            int64_t r_gate, int64_t r_up, int dtype, void* stream);
CT_API int ct_gated_backward(const void* x, int64_t ldx, const void* w_pair, int64_t ldw, const void* xa_gate,
                             const void* xa_up, int64_t ld_xa, const void* b_gate, const void* b_up,
                             const void* dh, void* h, void* d_gate, void* d_up, int64_t ld_out, int64_t T,
                             int64_t K, int64_t N, int64_t r_gate, int64_t r_up, int dtype, void* stream);
CT_API int ct_gated_input_gradient(const void* d_gate, const void* d_up, int64_t ld_signal, const void* w_pair,
                                   int64_t ldw, const void* low_gate, const void* low_up, int64_t ld_low,
                                   const void* a_gate, const void* a_up, void* dx, int64_t ld_dx, int64_t T,
                                   int64_t K, int64_t N, int64_t r_gate, int64_t r_up, int add, int dtype,
                                   void* stream);

/* ct_input_gradient_swiglu: the backward pass of an MLP that kept gate(x) and up(x) (kernels/mlp_cuda.py:122-133
 * with cached activations: `input_gradient` of the down projection, then `activation(gate, up, hidden_grad)`),
 * in one launch. dh = dy @ w + low @ a ([T, K], K = width of the SwiGLU, w [N, K], a [r, K], low = dy @ b [T, r]) is
 * accumulated in TMEM, rounded to bf16 as the stored gradient would be and never written: the epilogue reads
 * `gate` and `up` ([T, K], leading dimension ld_saved; requested one 32-column chunk ahead of their use) and writes
 *   d_gate, d_up, hidden  =  ct_swiglu's in-place backward of (gate, up, dh)
 * ([T, K], leading dimension ld_out; none may alias gate or up, which stay intact for a repeated backward
 * pass). Bit-identical to ct_input_gradient followed by ct_swiglu. bf16, K a multiple of 32, rows 16-byte
 * aligned; anything else returns CT_ERR_UNSUPPORTED (nothing launched). */
CT_API int ct_input_gradient_swiglu(const void* dy, int64_t ld_dy, const void* w, int64_t ldw, const void* a,
                                    const void* low, int64_t ld_low, const void* gate, const void* up,
                                    int64_t ld_saved, void* d_gate, void* d_up, void* hidden, int64_t ld_out,
                                    int64_t T, int64_t K, int64_t N, int64_t r, int dtype, void* stream);

/* ---- adjacent-pair partial RoPE ---------------------------------------------
 * Replaces kernels/core_cuda.py:146-164 (_rope: forward, or inverse into a
 * private tile, kernels/core_cuda.py:203-208) and kernels/core_cuda.py:167-199
 * (in-place rotation of freshly produced q and k). x[rows, heads*head_dim],
 * cos/sin[rows, half]; pairs (2c, 2c+1), c < half, of every head rotate; each
 * product is rounded to `dtype` before the add (kernels/core_cuda.py:134-142).
 * y may alias x. */
CT_API int ct_rope(const void* x, const void* cosine, const void* sine, void* y, int64_t rows,
            int heads, int head_dim, int half, int inverse, int dtype, void* stream);

/* ---- rotary position table --------------------------------------------------
 * Replaces kernels/core_cuda.py:11-27 (_position_values, position_values):
 *   cosine[t, c] = round(cos(float(positions[t]) * inverse[c])), sine likewise, c < half,
 * the product in fp32 and cos / sin with full-range argument reduction (long logical
 * positions), rounded to `dtype`. positions int64[count], inverse fp32[half]. */
CT_API int ct_position_values(const int64_t* positions, const float* inverse, void* cosine,
                              void* sine, int64_t count, int half, int dtype, void* stream);

/* ---- elementwise add ---------------------------------------------------------
 * Replaces `outputs[0].add_(residual)` (kernels/linear.py:90-91) and
 * `output.add_(residual)` (kernels/mlp_cuda.py:79-80): y = round(y + r). */
CT_API int ct_add_inplace(void* y, const void* r, int64_t n, int dtype, void* stream);

/* ---- RMSNorm ---------------------------------------------------------------------
 * Replaces kernels/core_cuda.py:30-40 (_rms_forward) and the input-gradient branch of
 * kernels/core_cuda.py:43-82 (_rms_gradient_row / _rms_backward with a frozen weight).
 *   rstd[row] = rsqrt(mean(x[row]^2) + eps)
 *   y  = round(x * rstd) * round(w)
 *   gx = rstd * (g - x * rstd^2 * mean(g * x)),  g = round(go * round(w))
 * round() rounds to `dtype` (the activation dtype); `w` has `weight_dtype`. x, y, go, gx are
 * [rows, width] contiguous; gx may alias go (the reference's reuse of a private upstream
 * gradient, kernels/core_cuda.py:113-115). */
CT_API int ct_rmsnorm_forward(const void* x, const void* w, void* y, float* rstd, int64_t rows,
                              int64_t width, float eps, int dtype, int weight_dtype, void* stream);
CT_API int ct_rmsnorm_backward(const void* x, const void* w, const float* rstd, const void* go,
                               void* gx, int64_t rows, int64_t width, int dtype, int weight_dtype,
                               void* stream);
/* The same input gradient plus the gradient that reaches x along the residual path it also
 * feeds (modeling/model.py:153-155 of the reference, where autograd adds the two):
 *   gx = round(round(rms gradient) + add), `add` [rows, width] in `dtype`, read only.
 * add == NULL is ct_rmsnorm_backward. */
CT_API int ct_rmsnorm_backward_add(const void* x, const void* w, const float* rstd, const void* go,
                                   const void* add, void* gx, int64_t rows, int64_t width, int dtype,
                                   int weight_dtype, void* stream);

/* Output-reconstruction mode of a frozen pre-norm (kernels/core_cuda.py:56-59, FROM_OUTPUT): the
 * backward pass is given the norm's OUTPUT y instead of its input (the caller keeps y anyway as the
 * input of the projection that follows, so x need not be retained):
 *   n = y / round(w);  gx = rstd * (g - n * mean(g * n)),  g = round(go * round(w))
 * Only meaningful where no weight is near zero; the caller decides (modeling/model.py:46-58 of the
 * reference allows 1/256 <= |w| <= 256 in bf16). gx may alias go; `add` (may be NULL) is the
 * residual-path gradient of ct_rmsnorm_backward_add. */
CT_API int ct_rmsnorm_backward_from_output(const void* y, const void* w, const float* rstd,
                                           const void* go, const void* add, void* gx, int64_t rows,
                                           int64_t width, int dtype, int weight_dtype, void* stream);
/* Trainable norm weight (kernels/core_cuda.py:60-91, _rms_gradient_row with WEIGHT_GRAD, _rms_backward,
 * _rms_weight_reduce): group `i` of `rows_per_group` consecutive rows writes
 *   partials[i, c] = sum over its rows of go[row, c] * round(x[row, c] * rstd[row])      fp32
 * (rows added in order) and, when gx != NULL, the input gradient of ct_rmsnorm_backward for those rows
 * (gx must not alias go here). partials is [ceil(rows / rows_per_group), width] fp32.
 * ct_rmsnorm_weight_reduce then writes dw[c] = sum over groups of partials[group, c] (fixed order) in
 * `weight_dtype`; groups == 0 gives zeros. */
CT_API int ct_rmsnorm_weight_gradient(const void* x, const void* w, const float* rstd, const void* go,
                                      void* gx, float* partials, int64_t rows, int64_t width,
                                      int64_t rows_per_group, int dtype, int weight_dtype, void* stream);
CT_API int ct_rmsnorm_weight_reduce(const float* partials, int64_t groups, int64_t width, void* dw,
                                    int weight_dtype, void* stream);

/* ---- weighted cross-entropy over a tile of logits -------------------------------
 * Replaces kernels/loss_cuda.py:12-72 (_statistics, _finish, weighted_ce).
 *   loss[row] = weights[row] * (logsumexp(logits[row]) - logits[row, targets[row]])
 * and, when `gradient` != 0, logits[row] is overwritten by
 *   (softmax(logits[row]) - onehot(targets[row])) * weights[row].
 * logits[rows, vocab] contiguous in `dtype`, targets int64, weights and loss fp32. */
CT_API int ct_weighted_ce(void* logits, const int64_t* targets, const float* weights, float* loss,
                          int64_t rows, int64_t vocab, int gradient, int dtype, void* stream);

/* ---- gradient scale + global-norm clip + AdamW --------------------------------
 * Replace the tail of Trainer.update (training/engine.py:97-107): `_foreach_div_(grads,
 * denominator)`, `clip_grad_norm_(parameters, max_norm)` and the fused `AdamW.step()`
 * (training/engine.py:10-16), as two passes over `count` fp32 tensors on one device.
 * ct_grad_norm:
 *   norm = || g / *divisor ||_2 over all tensors, coef = min(1, max_norm / (norm + 1e-6))
 *          (coef = 1 when max_norm <= 0); norm_out[0] = norm, norm_out[1] = coef.
 *   The sum runs in a fixed order, so the value is reproducible run to run.
 * ct_adamw_update, with `norm` = the two floats above:
 *   g' = g / *divisor * coef;  p *= 1 - lr * weight_decay[i];  m += (g' - m) * (1 - beta1);
 *   v = beta2 * v + (1 - beta2) * g'^2;
 *   p -= lr / (1 - beta1^step) * m / (sqrt(v) / sqrt(1 - beta2^step) + eps)
 *   and g' is written back over g when `write_grads` != 0 (what the reference leaves in .grad).
 *   If norm[0] is not finite no tensor is modified; the caller reads it and raises
 *   (error_if_nonfinite=True in the reference).
 * The pointer tables, `sizes` (elements) and `weight_decay` are HOST arrays of length `count`;
 * `divisor` (1 float), `norm_out` / `norm` (2 floats) and `workspace`
 * (ct_grad_norm_workspace(count) bytes) are device memory. `step` counts from 1. */
CT_API int64_t ct_grad_norm_workspace(int count);
CT_API int ct_grad_norm(int count, void* const* grads, const int64_t* sizes, const float* divisor,
                        float max_norm, float* norm_out, void* workspace, void* stream);
CT_API int ct_adamw_update(int count, void* const* grads, void* const* params, void* const* exp_avg,
                           void* const* exp_avg_sq, const int64_t* sizes, const float* weight_decay,
                           const float* divisor, const float* norm, float lr, float beta1, float beta2,
                           float eps, int64_t step, int write_grads, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CT_B200_H */
