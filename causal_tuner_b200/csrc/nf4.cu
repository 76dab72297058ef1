// NF4 decode: packed 4-bit codes + per-block absmax -> dense bf16/fp16/fp32.
//
// HBM-bound: 0.5 B of codes + 4/blocksize B of absmax read and 2 B (bf16) or
// 4 B (fp32) written per element. Per step each thread takes one 32-bit load of
// packed codes (8 elements), looks every nibble up in a shared-memory copy of
// the 16-entry code table, scales with one fp32 multiply per element and writes
// one 16-byte vector of bf16: a warp reads 128 contiguous bytes and writes 512
// contiguous bytes per step, so every sector is written whole. The table is
// stored once per lane (entry i of lane l at word 32*i + l), so the
// data-dependent look-ups of a warp always fall into 32 different banks.
//
// Arithmetic follows the reference Triton kernel (kernels/nf4_cuda.py:9-29):
// high nibble first, fp32 product, nested scale = code2[u8] * absmax2 + offset
// with the multiply and the add rounded separately, product rounded to the
// quant state's dtype and then to the output dtype.
#include "common.cuh"

namespace ct {
namespace {

constexpr int kThreads = 256;
constexpr int kGroup = 8;  // elements per thread per step: 4 packed bytes in, 16 bytes of bf16 out
constexpr int kSteps = 8;  // steps per thread

struct Nf4Params {
  const uint8_t* packed;
  const void* absmax;
  const float* code;
  const float* code2;
  const float* absmax2;
  const float* offset;
  void* out;
  int64_t n;
  int blocksize;
  int blocksize2;
  int nested;
  int state_dtype;
  int vector_ok;  // packed is 4-byte aligned and out 16-byte aligned
  int block_shift;   // log2(blocksize) when it is a power of two, else -1
  int block2_shift;  // the same for blocksize2
  // Chunked output (chunk > 0): element e is written to out[(e / chunk) * pitch + e % chunk], i.e. runs of
  // `chunk` elements land `pitch` elements apart - two weights decoded into one buffer of interleaved row blocks.
  int64_t chunk;
  int64_t pitch;
};

__device__ __forceinline__ int64_t place(const Nf4Params& p, int64_t element) {
  if (p.chunk <= 0) return element;
  const int64_t run = element / p.chunk;
  return run * p.pitch + (element - run * p.chunk);
}

__device__ __forceinline__ int64_t block_of(const Nf4Params& p, int64_t element) {
  return p.block_shift >= 0 ? element >> p.block_shift : element / p.blocksize;
}

// Rounding to the quant state's dtype before the output rounding. STATE = CT_F32 means none is
// needed: the state is fp32, or it has the output type (rounding twice to one type changes nothing).
template <int STATE>
__device__ __forceinline__ float round_state(float v) {
  if constexpr (STATE == CT_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  else if constexpr (STATE == CT_F16) return __half2float(__float2half_rn(v));
  else return v;
}

__device__ __forceinline__ float block_scale(const Nf4Params& p, int64_t group) {
  if (!p.nested) return __ldg(static_cast<const float*>(p.absmax) + group);
  const uint8_t q = __ldg(static_cast<const uint8_t*>(p.absmax) + group);
  const float decoded = __ldg(p.code2 + q);
  const float maximum = __ldg(p.absmax2 + (p.block2_shift >= 0 ? group >> p.block2_shift : group / p.blocksize2));
  return __fadd_rn(__fmul_rn(decoded, maximum), __ldg(p.offset));
}

template <typename OutT>
__device__ __forceinline__ void store_group(OutT* out, const float (&v)[kGroup]);

template <>
__device__ __forceinline__ void store_group<__nv_bfloat16>(__nv_bfloat16* out, const float (&v)[kGroup]) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&pair);
  }
  *reinterpret_cast<uint4*>(out) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <>
__device__ __forceinline__ void store_group<__half>(__half* out, const float (&v)[kGroup]) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __half2 pair = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&pair);
  }
  *reinterpret_cast<uint4*>(out) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <>
__device__ __forceinline__ void store_group<float>(float* out, const float (&v)[kGroup]) {
  float4* dst = reinterpret_cast<float4*>(out);
  dst[0] = make_float4(v[0], v[1], v[2], v[3]);
  dst[1] = make_float4(v[4], v[5], v[6], v[7]);
}

template <typename OutT, int STATE>
__global__ void __launch_bounds__(kThreads) nf4_decode_kernel(const Nf4Params p) {
  __shared__ float lut[16 * 32];
  lut[threadIdx.x] = __ldg(p.code + (threadIdx.x >> 5));
  lut[threadIdx.x + kThreads] = __ldg(p.code + ((threadIdx.x + kThreads) >> 5));
  __syncthreads();
  const float* mine = lut + (threadIdx.x & 31);
  OutT* out = static_cast<OutT*>(p.out);
  const bool vector = p.vector_ok && p.blocksize % kGroup == 0;
  const int64_t block_first = static_cast<int64_t>(blockIdx.x) * kSteps * kThreads * kGroup;

  if (vector && block_first + static_cast<int64_t>(kSteps) * kThreads * kGroup <= p.n) {
    // Whole block in range: issue every load of the thread before the first use, so that four
    // independent 4-byte reads (plus their scales) are in flight per thread.
    uint32_t word[kSteps];
    float scale[kSteps];
#pragma unroll
    for (int step = 0; step < kSteps; ++step) {
      const int64_t first = block_first + (static_cast<int64_t>(step) * kThreads + threadIdx.x) * kGroup;
      word[step] = __ldg(reinterpret_cast<const uint32_t*>(p.packed + first / 2));
      scale[step] = block_scale(p, block_of(p, first));
    }
#pragma unroll
    for (int step = 0; step < kSteps; ++step) {
      const int64_t first = block_first + (static_cast<int64_t>(step) * kThreads + threadIdx.x) * kGroup;
      float v[kGroup];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (word[step] >> (8 * b)) & 255u;
        v[2 * b] = round_state<STATE>(__fmul_rn(mine[(byte >> 4) * 32], scale[step]));
        v[2 * b + 1] = round_state<STATE>(__fmul_rn(mine[(byte & 15u) * 32], scale[step]));
      }
      store_group<OutT>(out + place(p, first), v);
    }
    return;
  }

#pragma unroll 1
  for (int step = 0; step < kSteps; ++step) {
    const int64_t group = (static_cast<int64_t>(blockIdx.x) * kSteps + step) * kThreads + threadIdx.x;
    const int64_t first = group * kGroup;
    if (first >= p.n) return;
    if (vector && first + kGroup <= p.n) {
      const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(p.packed + first / 2));
      const float scale = block_scale(p, block_of(p, first));
      float v[kGroup];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (word >> (8 * b)) & 255u;
        v[2 * b] = round_state<STATE>(__fmul_rn(mine[(byte >> 4) * 32], scale));
        v[2 * b + 1] = round_state<STATE>(__fmul_rn(mine[(byte & 15u) * 32], scale));
      }
      store_group<OutT>(out + place(p, first), v);
      continue;
    }
    // Ragged tail, unaligned buffers or block sizes that are not multiples of 8:
    // one packed byte at a time, element stores guarded by n.
    const int64_t last = (first + kGroup < p.n) ? first + kGroup : p.n;
    for (int64_t e = first; e < last; e += 2) {
      const uint8_t byte = __ldg(p.packed + e / 2);
      const float high = mine[(byte >> 4) * 32], low = mine[(byte & 15) * 32];
      const float scale = block_scale(p, block_of(p, e));
      out[place(p, e)] = from_float<OutT>(round_state<STATE>(__fmul_rn(high, scale)));
      if (e + 1 < p.n) out[place(p, e + 1)] = from_float<OutT>(round_state<STATE>(__fmul_rn(low, scale)));
    }
  }
}

// The same decode with the result written TRANSPOSED: W[rows, cols] (packed row-major) -> out[cols, rows] (bf16,
// leading dimension ld_out). One CTA takes a 64 x 64 tile: thread t decodes 16 consecutive elements of tile row
// t / 4 (one 8-byte load of codes, one scale: the 16 lie in one absmax block), parks them in a shared-memory tile
// indexed [column][row], and after the barrier writes 32 contiguous bytes of a transposed row - four threads
// cover the 128 bytes a tile contributes to it, so every sector is written whole. rows and cols are multiples of 64.
// The input gradient dx = dy . W contracts over the rows of W: with this layout W is a K-major operand of that
// GEMM, which the tensor core reads faster than the MN-major 64 x 64 boxes of the row-major weight.
constexpr int kTile = 64;
constexpr int kTilePitch = kTile + 8;   // bf16 elements per tile row: 144 bytes, 16-byte aligned

template <int STATE>
__global__ void __launch_bounds__(kThreads) nf4_decode_transposed_kernel(const Nf4Params p, int64_t rows, int64_t cols,
                                                                         int64_t ld_out) {
  __shared__ float lut[16 * 32];
  __shared__ __align__(16) __nv_bfloat16 tile[kTile * kTilePitch];
  lut[threadIdx.x] = __ldg(p.code + (threadIdx.x >> 5));
  lut[threadIdx.x + kThreads] = __ldg(p.code + ((threadIdx.x + kThreads) >> 5));
  __syncthreads();
  const float* mine = lut + (threadIdx.x & 31);
  const int64_t col0 = static_cast<int64_t>(blockIdx.x) * kTile, row0 = static_cast<int64_t>(blockIdx.y) * kTile;
  {
    const int r = threadIdx.x >> 2, quarter = threadIdx.x & 3;
    const int64_t first = (row0 + r) * cols + col0 + quarter * 16;
    const uint2 codes = __ldg(reinterpret_cast<const uint2*>(p.packed + first / 2));
    const float scale = block_scale(p, block_of(p, first));
    const uint32_t words[2] = {codes.x, codes.y};
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const uint32_t byte = (words[b >> 2] >> (8 * (b & 3))) & 255u;
      const float high = round_state<STATE>(__fmul_rn(mine[(byte >> 4) * 32], scale));
      const float low = round_state<STATE>(__fmul_rn(mine[(byte & 15u) * 32], scale));
      tile[(quarter * 16 + 2 * b) * kTilePitch + r] = __float2bfloat16_rn(high);
      tile[(quarter * 16 + 2 * b + 1) * kTilePitch + r] = __float2bfloat16_rn(low);
    }
  }
  __syncthreads();
  {
    const int c = threadIdx.x >> 2, quarter = threadIdx.x & 3;
    const uint4* source = reinterpret_cast<const uint4*>(tile + c * kTilePitch + quarter * 16);
    uint4* target = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + (col0 + c) * ld_out + row0 + quarter * 16);
    target[0] = source[0];
    target[1] = source[1];
  }
}

}  // namespace
}  // namespace ct

namespace ct {
namespace {
int decode(const uint8_t* packed, const void* absmax, const float* code, const float* code2, const float* absmax2,
           const float* offset, void* out, int64_t n, int blocksize, int blocksize2, int nested, int state_dtype,
           int out_dtype, int64_t chunk, int64_t pitch, void* stream);
}
}  // namespace ct

extern "C" int ct_nf4_decode(const uint8_t* packed, const void* absmax, const float* code,
                             const float* code2, const float* absmax2, const float* offset,
                             void* out, int64_t n, int blocksize, int blocksize2, int nested,
                             int state_dtype, int out_dtype, void* stream) {
  return ct::decode(packed, absmax, code, code2, absmax2, offset, out, n, blocksize, blocksize2, nested, state_dtype,
                    out_dtype, 0, 0, stream);
}

extern "C" int ct_nf4_decode_chunks(const uint8_t* packed, const void* absmax, const float* code,
                                    const float* code2, const float* absmax2, const float* offset,
                                    void* out, int64_t n, int blocksize, int blocksize2, int nested,
                                    int state_dtype, int out_dtype, int64_t chunk, int64_t pitch, void* stream) {
  if (chunk <= 0 || chunk % 8 != 0 || pitch < chunk || pitch % 8 != 0)
    return ct::fail(CT_ERR_ARG, "ct_nf4_decode_chunks: chunk=%lld pitch=%lld (multiples of 8, pitch >= chunk)",
                    (long long)chunk, (long long)pitch);
  return ct::decode(packed, absmax, code, code2, absmax2, offset, out, n, blocksize, blocksize2, nested, state_dtype,
                    out_dtype, chunk, pitch, stream);
}

extern "C" int ct_nf4_decode_transposed(const uint8_t* packed, const void* absmax, const float* code,
                                        const float* code2, const float* absmax2, const float* offset, void* out,
                                        int64_t rows, int64_t cols, int64_t ld_out, int blocksize, int blocksize2,
                                        int nested, int state_dtype, int out_dtype, void* stream) {
  using namespace ct;
  if (rows < 0 || cols < 0 || blocksize <= 0) return fail(CT_ERR_ARG, "ct_nf4_decode_transposed: sizes");
  if (rows == 0 || cols == 0) return CT_OK;
  if (!packed || !absmax || !code || !out) return fail(CT_ERR_ARG, "ct_nf4_decode_transposed: null pointer");
  if (nested && (!code2 || !absmax2 || !offset || blocksize2 <= 0))
    return fail(CT_ERR_ARG, "ct_nf4_decode_transposed: nested statistics missing");
  if (out_dtype != CT_BF16 || state_dtype < CT_F32 || state_dtype > CT_F16 || rows % kTile || cols % kTile ||
      blocksize % 16 || ld_out < rows || ld_out % 8 || (reinterpret_cast<uintptr_t>(packed) & 7) ||
      (reinterpret_cast<uintptr_t>(out) & 15) || rows / kTile > 65535)
    return fail(CT_ERR_UNSUPPORTED, "ct_nf4_decode_transposed: bf16 output, rows and columns in multiples of 64, block size a multiple of 16, aligned buffers");
  auto log2_of = [](int value) {
    if (value <= 0 || (value & (value - 1))) return -1;
    int shift = 0;
    while ((1 << shift) < value) ++shift;
    return shift;
  };
  const int inner2 = blocksize2 > 0 ? blocksize2 : 1;
  Nf4Params p{packed, absmax, code, code2, absmax2, offset, out, rows * cols, blocksize, inner2, nested, state_dtype,
              1, log2_of(blocksize), log2_of(inner2), 0, 0};
  const dim3 grid(static_cast<unsigned>(cols / kTile), static_cast<unsigned>(rows / kTile));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int state = (state_dtype == CT_F32 || state_dtype == out_dtype) ? CT_F32 : state_dtype;
  if (state == CT_F16) nf4_decode_transposed_kernel<CT_F16><<<grid, kThreads, 0, s>>>(p, rows, cols, ld_out);
  else nf4_decode_transposed_kernel<CT_F32><<<grid, kThreads, 0, s>>>(p, rows, cols, ld_out);
  count_launch(false);
  return check_launch("ct_nf4_decode_transposed");
}

namespace ct {
namespace {
int decode(const uint8_t* packed, const void* absmax, const float* code, const float* code2, const float* absmax2,
           const float* offset, void* out, int64_t n, int blocksize, int blocksize2, int nested, int state_dtype,
           int out_dtype, int64_t chunk, int64_t pitch, void* stream) {
  if (n < 0 || blocksize <= 0 || (blocksize & 1)) return fail(CT_ERR_ARG, "ct_nf4_decode: n=%lld blocksize=%d", (long long)n, blocksize);
  if (n == 0) return CT_OK;
  if (!packed || !absmax || !code || !out) return fail(CT_ERR_ARG, "ct_nf4_decode: null pointer");
  if (nested && (!code2 || !absmax2 || !offset || blocksize2 <= 0)) return fail(CT_ERR_ARG, "ct_nf4_decode: nested statistics missing");
  if (state_dtype < CT_F32 || state_dtype > CT_F16 || out_dtype < CT_F32 || out_dtype > CT_F16)
    return fail(CT_ERR_ARG, "ct_nf4_decode: dtype");
  auto log2_of = [](int value) {
    if (value <= 0 || (value & (value - 1))) return -1;
    int shift = 0;
    while ((1 << shift) < value) ++shift;
    return shift;
  };
  const int inner2 = blocksize2 > 0 ? blocksize2 : 1;
  Nf4Params p{packed, absmax, code, code2, absmax2, offset, out, n, blocksize, inner2, nested, state_dtype,
              (reinterpret_cast<uintptr_t>(packed) & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
              log2_of(blocksize), log2_of(inner2), chunk, pitch};
  const int64_t per_block = static_cast<int64_t>(kThreads) * kSteps * kGroup;
  const unsigned blocks = static_cast<unsigned>((n + per_block - 1) / per_block);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The state rounding is a separate step only when it changes something.
  const int state = (state_dtype == CT_F32 || state_dtype == out_dtype) ? CT_F32 : state_dtype;
#define CT_NF4_LAUNCH(OutT)                                                                    \
  do {                                                                                         \
    if (state == CT_BF16) nf4_decode_kernel<OutT, CT_BF16><<<blocks, kThreads, 0, s>>>(p);     \
    else if (state == CT_F16) nf4_decode_kernel<OutT, CT_F16><<<blocks, kThreads, 0, s>>>(p);  \
    else nf4_decode_kernel<OutT, CT_F32><<<blocks, kThreads, 0, s>>>(p);                       \
  } while (0)
  if (out_dtype == CT_BF16) CT_NF4_LAUNCH(__nv_bfloat16);
  else if (out_dtype == CT_F16) CT_NF4_LAUNCH(__half);
  else CT_NF4_LAUNCH(float);
#undef CT_NF4_LAUNCH
  count_launch(false);
  return check_launch("ct_nf4_decode");
}
}  // namespace
}  // namespace ct
