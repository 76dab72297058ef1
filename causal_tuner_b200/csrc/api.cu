// extern "C" surface of libct_b200.so: argument checking, the mapping of each
// reference operator onto GEMM segments, and the library state (error text,
// launch counters, per-device error flag).
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace ct {

namespace {
thread_local char g_error_text[512] = "";
std::atomic<int64_t> g_launches{0}, g_tc_launches{0};
constexpr int kMaxDevices = 64;
// Per-device error flag (device memory, or a device symbol when the no-allocation entry point came
// first). Installed on first use under g_device_mutex, so that two host threads that make their first
// calls on a device at the same moment agree on one flag.
int* g_error_flags[kMaxDevices] = {};
std::mutex g_device_mutex;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error_text, sizeof(g_error_text), fmt, args);
  va_end(args);
  return code;
}

void count_launch(bool tcgen05) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (tcgen05) g_tc_launches.fetch_add(1, std::memory_order_relaxed);
}

int check_launch(const char* what) {
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(CT_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
  return CT_OK;
}

// ---- per-launch timing -------------------------------------------------------------
namespace {
struct TimedLaunch {
  cudaEvent_t start, stop;
  double flops;
  long long m, n, k;
};
std::mutex g_timing_mutex;
std::vector<TimedLaunch> g_timed;
std::vector<cudaEvent_t> g_event_pool;
std::atomic<int> g_timing_on{0};
cudaEvent_t g_pending_start = nullptr;

cudaEvent_t take_event() {
  if (!g_event_pool.empty()) {
    cudaEvent_t e = g_event_pool.back();
    g_event_pool.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
  return e;
}
}  // namespace

bool timing_enabled() { return g_timing_on.load(std::memory_order_relaxed) != 0; }

void timing_begin(cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  g_pending_start = take_event();
  if (g_pending_start) cudaEventRecord(g_pending_start, stream);
}

void timing_end(cudaStream_t stream, double flops, long long m, long long n, long long k) {
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  if (!g_pending_start) return;
  cudaEvent_t stop = take_event();
  if (!stop) return;
  cudaEventRecord(stop, stream);
  g_timed.push_back({g_pending_start, stop, flops, m, n, k});
  g_pending_start = nullptr;
}

bool dependent_launch_enabled() {
  static const bool enabled = [] {
    const char* text = getenv("CT_B200_PDL");
    return !(text && text[0] == '0');
  }();
  return enabled;
}

int* device_error_flag() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (!g_error_flags[dev]) {
    int* flag = nullptr;
    if (cudaMalloc(&flag, sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMemset(flag, 0, sizeof(int)) != cudaSuccess) return nullptr;
    g_error_flags[dev] = flag;
  }
  return g_error_flags[dev];
}

namespace {

bool known_dtype(int d) { return d == CT_F32 || d == CT_BF16 || d == CT_F16; }

Segment segment(const void* a, int64_t a_rs, int64_t a_cs, const void* b, int64_t b_rs, int64_t b_cs, int64_t k) {
  Segment s;
  s.a = a; s.a_rs = a_rs; s.a_cs = a_cs;
  s.b = b; s.b_rs = b_rs; s.b_cs = b_cs;
  s.k = k;
  return s;
}

GemmArgs blank(int64_t M, int64_t N, int in_dtype, void* out, int64_t ldo, int out_dtype) {
  GemmArgs g;
  g.M = M; g.N = N; g.nseg = 0; g.in_dtype = in_dtype;
  g.out = out; g.ldo = ldo; g.out_dtype = out_dtype;
  g.beta = 0; g.bias = nullptr; g.residual = nullptr; g.ld_res = 0; g.split_k = 1;
  return g;
}

// Contraction slices for the token-contracted LoRA gradients. A function of the
// shapes alone (148 is the B200 SM count), so a given problem is always summed in
// the same order.
int gradient_splits(int64_t rows, int64_t cols, int64_t T) {
  // Output tiles are 256 x 256 on 74 CTA pairs from 256 rows up, 128 x 256 on 148 CTAs below.
  const bool pairs = rows >= 256;
  const int64_t tiles = ((rows + (pairs ? 255 : 127)) / (pairs ? 256 : 128)) * ((cols + 255) / 256);
  const int64_t k_blocks = (T + 63) / 64;
  const int64_t slots = pairs ? 74 : 148;
  if (tiles <= 0 || tiles >= slots) return 1;
  // Cost of s slices in k-block times: rounds of resident tiles, each (k_blocks / s) long plus a fixed
  // fill + epilogue share, plus the ordered sum of s partial planes. Smallest cost wins, fewest
  // slices on a tie; at least 8 k-blocks per slice.
  int64_t best = 1, best_cost = -1;
  for (int64_t s = 1; s <= 16 && s * 8 <= (k_blocks > 8 ? k_blocks : 8); ++s) {
    const int64_t rounds = (tiles * s + slots - 1) / slots;
    const int64_t cost = rounds * ((k_blocks + s - 1) / s + 16) + (s > 1 ? 4 * s : 0);
    if (best_cost < 0 || cost < best_cost) {
      best = s;
      best_cost = cost;
    }
  }
  return static_cast<int>(best);
}

// out[rows, cols] (fp32) (+)= A^T . B over T rows; A is [T, rows], B is [T, cols].
int token_contraction(const void* a, int64_t lda, const void* b, int64_t ldb, float* out, int64_t rows, int64_t cols,
                      int64_t T, int add, int dtype, void* workspace, int path, cudaStream_t stream) {
  GemmArgs g = blank(rows, cols, dtype, out, cols, CT_F32);
  g.nseg = 1;
  g.seg[0] = segment(a, 1, lda, b, ldb, 1, T);
  g.beta = add;
  const bool tc = path != CT_PATH_SIMT && gemm_tcgen05_supported(g);
  const int splits = tc ? gradient_splits(rows, cols, T) : 1;
  if (splits <= 1) return gemm_dispatch(g, path, stream);
  if (!workspace) return fail(CT_ERR_ARG, "parameter gradients: workspace is null but %d slices are needed", splits);
  g.out = workspace;
  g.beta = 0;
  g.split_k = splits;
  int rc = gemm_tcgen05(g, stream);
  if (rc != CT_OK) return rc;
  return reduce_partials(static_cast<const float*>(workspace), splits, rows, cols, cols, out, cols, add, stream);
}

}  // namespace
}  // namespace ct

using namespace ct;

extern "C" int ct_abi_version(void) { return 1; }
extern "C" int64_t ct_launch_count(void) { return g_launches.load(); }
extern "C" int64_t ct_tcgen05_launch_count(void) { return g_tc_launches.load(); }
extern "C" const char* ct_last_error(void) { return g_error_text; }

extern "C" int ct_timing_enable(int on) {
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  for (auto& t : g_timed) {
    g_event_pool.push_back(t.start);
    g_event_pool.push_back(t.stop);
  }
  g_timed.clear();
  g_timing_on.store(on ? 1 : 0);
  return CT_OK;
}

extern "C" int ct_timing_collect(double* total_ms, double* total_flops, int64_t* launches) {
  if (!total_ms || !total_flops || !launches) return fail(CT_ERR_ARG, "ct_timing_collect: null pointer");
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  double ms = 0, flops = 0;
  int64_t count = 0;
  // CT_B200_TIMING_LOG=<file>: append one "M,N,K,ms" line per recorded launch (shape studies).
  const char* log_path = getenv("CT_B200_TIMING_LOG");
  FILE* shape_log = log_path ? fopen(log_path, "a") : nullptr;
  for (auto& t : g_timed) {
    cudaError_t err = cudaEventSynchronize(t.stop);
    float one = 0;
    if (err == cudaSuccess) err = cudaEventElapsedTime(&one, t.start, t.stop);
    if (err != cudaSuccess) return fail(CT_ERR_CUDA, "ct_timing_collect: %s", cudaGetErrorString(err));
    ms += one;
    flops += t.flops;
    ++count;
    if (shape_log) fprintf(shape_log, "%lld,%lld,%lld,%.6f\n", t.m, t.n, t.k, one);
    g_event_pool.push_back(t.start);
    g_event_pool.push_back(t.stop);
  }
  g_timed.clear();
  if (shape_log) fclose(shape_log);
  *total_ms = ms;
  *total_flops = flops;
  *launches = count;
  return CT_OK;
}

extern "C" int ct_check_device(void* stream) {
  cudaError_t err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(CT_ERR_CUDA, "ct_check_device: %s", cudaGetErrorString(err));
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(CT_ERR_CUDA, "ct_check_device: no current device");
  int* flag = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_device_mutex);
    flag = g_error_flags[dev];
  }
  if (!flag) return CT_OK;
  int value = 0;
  err = cudaMemcpy(&value, flag, sizeof(int), cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) return fail(CT_ERR_CUDA, "ct_check_device: %s", cudaGetErrorString(err));
  if (value == 0) return CT_OK;
  cudaMemset(flag, 0, sizeof(int));
  static const char* roles[] = {"", "TMA producer waiting for a free stage", "MMA issuer waiting for a free accumulator",
                                "MMA issuer waiting for a filled stage", "epilogue waiting for a finished accumulator",
                                "the self-test's wait on a barrier that nothing completes"};
  return fail(CT_ERR_DEVICE, "a tcgen05 GEMM CTA gave up on a bounded wait: %s", value >= 1 && value <= 5 ? roles[value] : "?");
}

extern "C" int ct_selftest_bounded_wait(int64_t limit_us, void* stream) {
  return bounded_wait_selftest(limit_us, static_cast<cudaStream_t>(stream));
}

extern "C" int ct_matmul(const void* A, int64_t a_rs, int64_t a_cs, const void* B, int64_t b_rs, int64_t b_cs, void* C,
                         int64_t ldc, int64_t M, int64_t N, int64_t K, int in_dtype, int out_dtype, int add, int path,
                         void* stream) {
  if (M < 0 || N < 0 || K < 0) return fail(CT_ERR_ARG, "ct_matmul: negative size");
  if (M == 0 || N == 0) return CT_OK;
  if (!C || (K > 0 && (!A || !B))) return fail(CT_ERR_ARG, "ct_matmul: null pointer");
  if (!known_dtype(in_dtype) || !known_dtype(out_dtype)) return fail(CT_ERR_ARG, "ct_matmul: dtype");
  GemmArgs g = blank(M, N, in_dtype, C, ldc, out_dtype);
  g.nseg = 1;
  g.seg[0] = segment(A, a_rs, a_cs, B, b_rs, b_cs, K);
  g.beta = add;
  return gemm_dispatch(g, path, static_cast<cudaStream_t>(stream));
}

extern "C" int ct_matmul_nf4(const void* x, int64_t ldx, const uint8_t* packed, const float* absmax, const float* code,
                             void* out, int64_t ld_out, int64_t T, int64_t K, int64_t N, int blocksize, int dtype,
                             void* stream) {
  if (T < 0 || K < 0 || N < 0) return fail(CT_ERR_ARG, "ct_matmul_nf4: negative size");
  if (T == 0 || N == 0) return CT_OK;
  if (!x || !packed || !absmax || !code || !out) return fail(CT_ERR_ARG, "ct_matmul_nf4: null pointer");
  if (dtype != CT_BF16 || blocksize != 64)
    return fail(CT_ERR_UNSUPPORTED, "ct_matmul_nf4: bf16 activations and 64-element blocks with fp32 absmax only");
  return gemm_tcgen05_nf4(x, ldx, packed, absmax, code, out, ld_out, T, K, N, static_cast<cudaStream_t>(stream));
}

namespace {
int gated(const char* what, const void* x, int64_t ldx, const void* w_pair, int64_t ldw, const void* xa_gate,
          const void* xa_up, int64_t ld_xa, const void* b_gate, const void* b_up, const void* dh, void* h, void* gate,
          void* up, int64_t ld_out, int64_t T, int64_t K, int64_t N, int64_t r_gate, int64_t r_up, int dtype,
          void* stream) {
  if (T < 0 || K <= 0 || N < 0 || r_gate <= 0 || r_up <= 0) return fail(CT_ERR_ARG, "%s: sizes", what);
  if (T == 0 || N == 0) return CT_OK;
  if (!x || !w_pair || !xa_gate || !xa_up || !b_gate || !b_up || !h) return fail(CT_ERR_ARG, "%s: null pointer", what);
  if (dtype != CT_BF16) return fail(CT_ERR_UNSUPPORTED, "%s: bf16 only", what);
  GatedArgs a;
  a.x = x; a.ldx = ldx; a.w_pair = w_pair; a.ldw = ldw;
  a.xa_gate = xa_gate; a.xa_up = xa_up; a.ld_xa = ld_xa; a.b_gate = b_gate; a.b_up = b_up;
  a.T = T; a.K = K; a.N = N; a.r_gate = r_gate; a.r_up = r_up;
  a.h = h; a.gate = gate; a.up = up; a.dh = dh; a.ld_out = ld_out;
  return gemm_tcgen05_gated(a, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" int ct_gated_forward(const void* x, int64_t ldx, const void* w_pair, int64_t ldw, const void* xa_gate,
                                const void* xa_up, int64_t ld_xa, const void* b_gate, const void* b_up, void* h,
                                void* gate, void* up, int64_t ld_out, int64_t T, int64_t K, int64_t N, int64_t r_gate,
                                int64_t r_up, int dtype, void* stream) {
  return gated("ct_gated_forward", x, ldx, w_pair, ldw, xa_gate, xa_up, ld_xa, b_gate, b_up, nullptr, h, gate, up,
               ld_out, T, K, N, r_gate, r_up, dtype, stream);
}

extern "C" int ct_gated_backward(const void* x, int64_t ldx, const void* w_pair, int64_t ldw, const void* xa_gate,
                                 const void* xa_up, int64_t ld_xa, const void* b_gate, const void* b_up, const void* dh,
                                 void* h, void* d_gate, void* d_up, int64_t ld_out, int64_t T, int64_t K, int64_t N,
                                 int64_t r_gate, int64_t r_up, int dtype, void* stream) {
  if (T > 0 && N > 0 && (!dh || !d_gate || !d_up)) return fail(CT_ERR_ARG, "ct_gated_backward: null pointer");
  return gated("ct_gated_backward", x, ldx, w_pair, ldw, xa_gate, xa_up, ld_xa, b_gate, b_up, dh, h, d_gate, d_up,
               ld_out, T, K, N, r_gate, r_up, dtype, stream);
}

extern "C" int ct_gated_input_gradient(const void* d_gate, const void* d_up, int64_t ld_signal, const void* w_pair,
                                       int64_t ldw, const void* low_gate, const void* low_up, int64_t ld_low,
                                       const void* a_gate, const void* a_up, void* dx, int64_t ld_dx, int64_t T,
                                       int64_t K, int64_t N, int64_t r_gate, int64_t r_up, int add, int dtype,
                                       void* stream) {
  if (T < 0 || K < 0 || N <= 0 || r_gate <= 0 || r_up <= 0) return fail(CT_ERR_ARG, "ct_gated_input_gradient: sizes");
  if (T == 0 || K == 0) return CT_OK;
  if (!d_gate || !d_up || !w_pair || !low_gate || !low_up || !a_gate || !a_up || !dx)
    return fail(CT_ERR_ARG, "ct_gated_input_gradient: null pointer");
  if (dtype != CT_BF16) return fail(CT_ERR_UNSUPPORTED, "ct_gated_input_gradient: bf16 only");
  GatedGradientArgs a;
  a.dg = d_gate; a.du = d_up; a.ld_signal = ld_signal; a.w_pair = w_pair; a.ldw = ldw;
  a.low_gate = low_gate; a.low_up = low_up; a.ld_low = ld_low; a.a_gate = a_gate; a.a_up = a_up;
  a.T = T; a.K = K; a.N = N; a.r_gate = r_gate; a.r_up = r_up;
  a.dx = dx; a.ld_dx = ld_dx; a.add = add;
  return gemm_tcgen05_gated_input_gradient(a, static_cast<cudaStream_t>(stream));
}

extern "C" int ct_input_gradient_swiglu(const void* dy, int64_t ld_dy, const void* w, int64_t ldw, const void* a,
                                        const void* low, int64_t ld_low, const void* gate, const void* up,
                                        int64_t ld_saved, void* d_gate, void* d_up, void* hidden, int64_t ld_out,
                                        int64_t T, int64_t K, int64_t N, int64_t r, int dtype, void* stream) {
  if (T < 0 || K < 0 || N <= 0 || r < 0) return fail(CT_ERR_ARG, "ct_input_gradient_swiglu: sizes");
  if (T == 0 || K == 0) return CT_OK;
  if (!dy || !w || (r > 0 && (!a || !low)) || !gate || !up || !d_gate || !d_up || !hidden)
    return fail(CT_ERR_ARG, "ct_input_gradient_swiglu: null pointer");
  if (dtype != CT_BF16) return fail(CT_ERR_UNSUPPORTED, "ct_input_gradient_swiglu: bf16 only");
  GatedDownArgs args;
  args.dy = dy; args.ld_dy = ld_dy; args.w = w; args.ldw = ldw; args.a = a; args.low = low; args.ld_low = ld_low;
  args.gate = gate; args.up = up; args.ld_saved = ld_saved;
  args.d_gate = d_gate; args.d_up = d_up; args.hidden = hidden; args.ld_out = ld_out;
  args.T = T; args.K = K; args.N = N; args.r = r;
  return gemm_tcgen05_gated_down_gradient(args, static_cast<cudaStream_t>(stream));
}

extern "C" int ct_forward_linear(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* a, const void* b,
                                 const void* bias, const void* residual, int64_t ld_res, void* out, int64_t ld_out,
                                 void* xa, int64_t ld_xa, int64_t T, int64_t K, int64_t N, int64_t r, int dtype,
                                 int path, void* stream) {
  if (T < 0 || K < 0 || N < 0 || r < 0) return fail(CT_ERR_ARG, "ct_forward_linear: negative size");
  if (T == 0 || N == 0) return CT_OK;
  if (!out || (K > 0 && (!x || !w)) || (r > 0 && (!b || !xa))) return fail(CT_ERR_ARG, "ct_forward_linear: null pointer");
  if (!known_dtype(dtype)) return fail(CT_ERR_ARG, "ct_forward_linear: dtype %d", dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (r > 0 && a) {   // a == NULL: xa already holds x . a^T (computed for several projections at once)
    GemmArgs low = blank(T, r, dtype, xa, ld_xa, dtype);
    low.nseg = 1;
    low.seg[0] = segment(x, ldx, 1, a, 1, K, K);
    const int rc = gemm_dispatch(low, path, s);
    if (rc != CT_OK) return rc;
  }
  GemmArgs g = blank(T, N, dtype, out, ld_out, dtype);
  g.seg[g.nseg++] = segment(x, ldx, 1, w, 1, ldw, K);
  if (r > 0) g.seg[g.nseg++] = segment(xa, ld_xa, 1, b, 1, r, r);
  g.bias = bias;
  g.residual = residual;
  g.ld_res = ld_res;
  return gemm_dispatch(g, path, s);
}

extern "C" int ct_input_gradient(const void* dy, int64_t ld_dy, const void* w, int64_t w_rs, int64_t w_cs,
                                 const void* a, const void* b, void* dx, int64_t ld_dx, void* low, int64_t ld_low,
                                 int64_t T, int64_t K, int64_t N, int64_t r, int add, int dtype, int path,
                                 void* stream) {
  if (T < 0 || K < 0 || N < 0 || r < 0) return fail(CT_ERR_ARG, "ct_input_gradient: negative size");
  if (T == 0) return CT_OK;
  if ((N > 0 && !dy) || (r > 0 && !low) || (w && (!dx || (r > 0 && !a))))
    return fail(CT_ERR_ARG, "ct_input_gradient: null pointer");
  if (!known_dtype(dtype)) return fail(CT_ERR_ARG, "ct_input_gradient: dtype %d", dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (r > 0 && b) {   // b == NULL: low already holds dy . b (computed while the base weight was still decoding)
    GemmArgs g = blank(T, r, dtype, low, ld_low, dtype);
    g.nseg = 1;
    g.seg[0] = segment(dy, ld_dy, 1, b, r, 1, N);
    const int rc = gemm_dispatch(g, path, s);
    if (rc != CT_OK) return rc;
  }
  if (!w || K == 0) return CT_OK;
  GemmArgs g = blank(T, K, dtype, dx, ld_dx, dtype);
  g.seg[g.nseg++] = segment(dy, ld_dy, 1, w, w_rs, w_cs, N);
  if (r > 0) g.seg[g.nseg++] = segment(low, ld_low, 1, a, K, 1, r);
  g.beta = add;
  return gemm_dispatch(g, path, s);
}

extern "C" int ct_input_gradient_group(int count, const void* const* dy, const int64_t* ld_dy, const void* const* w,
                                       const int64_t* w_rs, const int64_t* w_cs, const void* const* a,
                                       const void* const* b,
                                       const int64_t* N, const int64_t* r, void* dx, int64_t ld_dx, void* const* low,
                                       const int64_t* ld_low, int64_t T, int64_t K, int add, int dtype, int path,
                                       void* stream) {
  if (count < 1 || 2 * count > kMaxSegments) return fail(CT_ERR_ARG, "ct_input_gradient_group: count %d", count);
  if (T < 0 || K < 0) return fail(CT_ERR_ARG, "ct_input_gradient_group: negative size");
  if (T == 0 || K == 0) return CT_OK;
  if (!dy || !ld_dy || !w || !w_rs || !w_cs || !a || !b || !N || !r || !dx || !low || !ld_low)
    return fail(CT_ERR_ARG, "ct_input_gradient_group: null pointer");
  if (!known_dtype(dtype)) return fail(CT_ERR_ARG, "ct_input_gradient_group: dtype %d", dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < count; ++i) {
    if (N[i] <= 0 || r[i] <= 0 || !dy[i] || !w[i] || !a[i] || !b[i] || !low[i])
      return fail(CT_ERR_ARG, "ct_input_gradient_group: projection %d is incomplete", i);
    GemmArgs g = blank(T, r[i], dtype, low[i], ld_low[i], dtype);
    g.nseg = 1;
    g.seg[0] = segment(dy[i], ld_dy[i], 1, b[i], r[i], 1, N[i]);
    const int rc = gemm_dispatch(g, path, s);
    if (rc != CT_OK) return rc;
  }
  GemmArgs g = blank(T, K, dtype, dx, ld_dx, dtype);
  for (int i = 0; i < count; ++i) {
    g.seg[g.nseg++] = segment(dy[i], ld_dy[i], 1, w[i], w_rs[i], w_cs[i], N[i]);
    g.seg[g.nseg++] = segment(low[i], ld_low[i], 1, a[i], K, 1, r[i]);
  }
  g.beta = add;
  return gemm_dispatch(g, path, s);
}

extern "C" int64_t ct_parameter_gradients_workspace(int64_t T, int64_t K, int64_t N, int64_t r, int dtype, int path) {
  if (dtype != CT_BF16 || path == CT_PATH_SIMT || T <= 0 || r <= 0) return 0;
  const int sa = gradient_splits(r, K, T), sb = gradient_splits(N, r, T);
  const int64_t need_a = sa > 1 ? sa * r * K * 4 : 0, need_b = sb > 1 ? sb * N * r * 4 : 0;
  return need_a > need_b ? need_a : need_b;
}

extern "C" int ct_parameter_gradients(const void* x, int64_t ldx, const void* dy, int64_t ld_dy, const void* low,
                                      int64_t ld_low, const void* xa, int64_t ld_xa, float* da, float* db, int64_t T,
                                      int64_t K, int64_t N, int64_t r, int add, int dtype, void* workspace, int path,
                                      void* stream) {
  if (T < 0 || K < 0 || N < 0 || r < 0) return fail(CT_ERR_ARG, "ct_parameter_gradients: negative size");
  if (r == 0) return CT_OK;
  if (!da || !db || (T > 0 && (!x || !dy || !low || !xa))) return fail(CT_ERR_ARG, "ct_parameter_gradients: null pointer");
  if (!known_dtype(dtype)) return fail(CT_ERR_ARG, "ct_parameter_gradients: dtype %d", dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = token_contraction(low, ld_low, x, ldx, da, r, K, T, add, dtype, workspace, path, s);
  if (rc != CT_OK) return rc;
  return token_contraction(dy, ld_dy, xa, ld_xa, db, N, r, T, add, dtype, workspace, path, s);
}

extern "C" int64_t ct_accumulate_workspace(int64_t rows, int64_t cols, int64_t T, int dtype, int path) {
  if (dtype != CT_BF16 || path == CT_PATH_SIMT || T <= 0 || rows <= 0 || cols <= 0) return 0;
  const int splits = gradient_splits(rows, cols, T);
  return splits > 1 ? static_cast<int64_t>(splits) * rows * cols * static_cast<int64_t>(sizeof(float)) : 0;
}

extern "C" int ct_accumulate(const void* left, int64_t ld_left, const void* right, int64_t ld_right, float* out,
                             int64_t rows, int64_t cols, int64_t T, int add, int dtype, void* workspace, int path,
                             void* stream) {
  if (rows < 0 || cols < 0 || T < 0) return fail(CT_ERR_ARG, "ct_accumulate: negative size");
  if (rows == 0 || cols == 0) return CT_OK;
  if (!out || (T > 0 && (!left || !right))) return fail(CT_ERR_ARG, "ct_accumulate: null pointer");
  if (!known_dtype(dtype)) return fail(CT_ERR_ARG, "ct_accumulate: dtype %d", dtype);
  return token_contraction(left, ld_left, right, ld_right, out, rows, cols, T, add, dtype, workspace, path,
                           static_cast<cudaStream_t>(stream));
}

// ---- several token contractions in one launch ---------------------------------------------------
namespace {
constexpr int kMaxTokenGroup = 6;

// One slice count for the whole group (every product contracts over the same T): the cheapest of 1..16 by the
// cost model of gradient_splits applied to the group's tile total. A function of the shapes alone.
int group_splits(int count, const int64_t* rows, const int64_t* cols, int64_t T) {
  int64_t tiles = 0;
  for (int i = 0; i < count; ++i) tiles += ((rows[i] + 255) / 256) * ((cols[i] + 255) / 256);
  const int64_t k_blocks = (T + 63) / 64, slots = 74;
  if (tiles <= 0) return 1;
  int64_t best = 1, best_cost = -1;
  for (int64_t s = 1; s <= 16 && s * 8 <= (k_blocks > 8 ? k_blocks : 8); ++s) {
    const int64_t rounds = (tiles * s + slots - 1) / slots;
    const int64_t cost = rounds * ((k_blocks + s - 1) / s + 16) + (s > 1 ? 4 * s : 0);
    if (best_cost < 0 || cost < best_cost) {
      best = s;
      best_cost = cost;
    }
  }
  return static_cast<int>(best);
}

bool group_on_tensor_cores(int count, const void* const* left, const int64_t* ld_left, const void* const* right,
                           const int64_t* ld_right, float* const* out, const int64_t* rows, const int64_t* cols,
                           int64_t T, int dtype, int path) {
  if (path == CT_PATH_SIMT || dtype != CT_BF16 || count < 2 || count > kMaxTokenGroup) return false;
  for (int i = 0; i < count; ++i) {
    GemmArgs g = blank(rows[i], cols[i], dtype, out[i], cols[i], CT_F32);
    g.nseg = 1;
    g.seg[0] = segment(left[i], 1, ld_left[i], right[i], ld_right[i], 1, T);
    if (!gemm_tcgen05_supported(g)) return false;
  }
  return true;
}
}  // namespace

extern "C" int64_t ct_token_gradients_group_workspace(int count, const int64_t* rows, const int64_t* cols, int64_t T,
                                                      int dtype, int path) {
  if (count < 1 || !rows || !cols || T <= 0 || dtype != CT_BF16 || path == CT_PATH_SIMT) return 0;
  int64_t bytes = 0, single = 0;
  const int s = count >= 2 && count <= kMaxTokenGroup ? group_splits(count, rows, cols, T) : 1;
  for (int i = 0; i < count; ++i) {
    bytes += static_cast<int64_t>(s) * rows[i] * cols[i] * 4;
    const int64_t alone = ct_accumulate_workspace(rows[i], cols[i], T, dtype, path);   // the one-by-one route
    single = alone > single ? alone : single;
  }
  if (s <= 1) bytes = 0;
  return bytes > single ? bytes : single;
}

extern "C" int ct_token_gradients_group(int count, const void* const* left, const int64_t* ld_left,
                                        const void* const* right, const int64_t* ld_right, float* const* out,
                                        const int64_t* rows, const int64_t* cols, int64_t T, const int* add, int dtype,
                                        void* workspace, int path, void* stream) {
  if (count < 1) return fail(CT_ERR_ARG, "ct_token_gradients_group: count %d", count);
  if (!left || !ld_left || !right || !ld_right || !out || !rows || !cols || !add)
    return fail(CT_ERR_ARG, "ct_token_gradients_group: null pointer");
  if (T < 0) return fail(CT_ERR_ARG, "ct_token_gradients_group: negative size");
  if (!known_dtype(dtype)) return fail(CT_ERR_ARG, "ct_token_gradients_group: dtype %d", dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < count; ++i) {
    if (rows[i] < 0 || cols[i] < 0) return fail(CT_ERR_ARG, "ct_token_gradients_group: negative size");
    if (rows[i] > 0 && cols[i] > 0 && (!out[i] || (T > 0 && (!left[i] || !right[i]))))
      return fail(CT_ERR_ARG, "ct_token_gradients_group: null pointer in problem %d", i);
  }
  bool grouped = T > 0 && group_on_tensor_cores(count, left, ld_left, right, ld_right, out, rows, cols, T, dtype, path);
  for (int i = 0; grouped && i < count; ++i) grouped = rows[i] > 0 && cols[i] > 0;
  if (!grouped) {   // one by one: odd shapes, fp32 operands, the SIMT path, a single product
    for (int i = 0; i < count; ++i) {
      if (rows[i] == 0 || cols[i] == 0) continue;
      const int rc = token_contraction(left[i], ld_left[i], right[i], ld_right[i], out[i], rows[i], cols[i], T, add[i],
                                       dtype, workspace, path, s);
      if (rc != CT_OK) return rc;
    }
    return CT_OK;
  }
  const int splits = group_splits(count, rows, cols, T);
  if (splits > 1 && !workspace)
    return fail(CT_ERR_ARG, "ct_token_gradients_group: workspace is null but %d slices are needed", splits);
  GemmArgs problems[kMaxTokenGroup];
  float* planes[kMaxTokenGroup];
  float* cursor = static_cast<float*>(workspace);
  for (int i = 0; i < count; ++i) {
    GemmArgs& g = problems[i];
    g = blank(rows[i], cols[i], dtype, out[i], cols[i], CT_F32);
    g.nseg = 1;
    g.seg[0] = segment(left[i], 1, ld_left[i], right[i], ld_right[i], 1, T);
    g.beta = add[i];
    planes[i] = nullptr;
    if (splits > 1) {
      planes[i] = cursor;
      cursor += static_cast<int64_t>(splits) * rows[i] * cols[i];
      g.out = planes[i];
      g.beta = 0;
      g.split_k = splits;
    }
  }
  int rc = gemm_tcgen05_group(problems, count, s);
  if (rc != CT_OK) return rc;
  for (int i = 0; splits > 1 && i < count; ++i) {
    rc = reduce_partials(planes[i], splits, rows[i], cols[i], cols[i], out[i], cols[i], add[i], s);
    if (rc != CT_OK) return rc;
  }
  return CT_OK;
}

// ---- parameter gradients without any allocation ----------------------------------------------
// Slice-partial scratch that lives in the library image itself. Every GPU on which this entry point
// has been called holds these bytes until the process exits. In HOST code the array's name is only a stand-in for
// the symbol; the device address comes from cudaGetSymbolAddress, once per device.
namespace {
constexpr int64_t kNoAllocScratchBytes = 16ll << 20;  // e.g. 4 slices of a 256 x 4096 fp32 gradient
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
static __device__ int g_noalloc_error_flag;
void* g_noalloc_scratch_address[kMaxDevices] = {};

// First use on a device: resolve the device addresses of the two symbols above. The call itself asks for no
// memory, but CUDA loads a module's image lazily: the module that holds these symbols (and with it the
// 16 MiB array) reaches the device here, on the first call, and the GEMM's module on its first launch.
// A host that must not allocate later makes one warm-up call per device at start-up.
int noalloc_setup(void** scratch) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(CT_ERR_CUDA, "ct_parameter_gradients_noalloc: no current device");
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (!g_noalloc_scratch_address[dev]) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_noalloc_scratch);
    if (err != cudaSuccess || !address)
      return fail(CT_ERR_CUDA, "ct_parameter_gradients_noalloc: cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(err));
    if (!g_error_flags[dev]) {
      // The GEMM reports bounded-wait timeouts through a per-device int that the other entry points
      // allocate on first use; here it is a static symbol instead, so this path never allocates.
      void* flag = nullptr;
      err = cudaGetSymbolAddress(&flag, g_noalloc_error_flag);
      if (err != cudaSuccess || !flag)
        return fail(CT_ERR_CUDA, "ct_parameter_gradients_noalloc: cudaGetSymbolAddress(flag): %s", cudaGetErrorString(err));
      g_error_flags[dev] = static_cast<int*>(flag);
    }
    g_noalloc_scratch_address[dev] = address;
  }
  *scratch = g_noalloc_scratch_address[dev];
  return CT_OK;
}
}  // namespace

extern "C" int64_t ct_parameter_gradients_noalloc_capacity(void) { return kNoAllocScratchBytes; }

extern "C" int ct_parameter_gradients_noalloc(const void* x, int64_t ldx, const void* dy, int64_t ld_dy,
                                              const void* low, int64_t ld_low, const void* xa, int64_t ld_xa,
                                              float* da, float* db, int64_t T, int64_t K, int64_t N, int64_t r,
                                              int add, int dtype, int path, void* stream) {
  const int64_t need = ct_parameter_gradients_workspace(T, K, N, r, dtype, path);
  if (need > kNoAllocScratchBytes)
    return fail(CT_ERR_UNSUPPORTED,
                "ct_parameter_gradients_noalloc: this problem needs %lld bytes of slice scratch, the built-in "
                "array holds %lld; use ct_parameter_gradients with a caller-provided workspace",
                (long long)need, (long long)kNoAllocScratchBytes);
  void* scratch = nullptr;
  const int rc = noalloc_setup(&scratch);
  if (rc != CT_OK) return rc;
  // Nothing in the scratch has to start at zero: every slice plane is written in full by the GEMM
  // (one store per element) before the ordered reduction reads it.
  return ct_parameter_gradients(x, ldx, dy, ld_dy, low, ld_low, xa, ld_xa, da, db, T, K, N, r, add, dtype, scratch,
                                path, stream);
}
