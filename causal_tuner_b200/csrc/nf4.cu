// NF4 decode: packed 4-bit codes + per-block absmax -> dense bf16/fp16/fp32.
//
// HBM-bound: 0.5 B of codes + 4/blocksize B of absmax read and 2 B (bf16) or
// 4 B (fp32) written per element. Each thread takes one 128-bit load of packed
// codes (32 elements, half of a 64-element block), looks both nibbles of every
// byte up in a 256-entry shared-memory table of (high, low) code pairs, scales
// with one fp32 multiply per element and writes 64 contiguous bytes of bf16.
// A warp therefore reads 512 contiguous bytes and writes 2 KB contiguous bytes.
//
// Arithmetic follows the reference Triton kernel (kernels/nf4_cuda.py:9-29):
// high nibble first, fp32 product, nested scale = code2[u8] * absmax2 + offset
// with the multiply and the add rounded separately, product rounded to the
// quant state's dtype and then to the output dtype.
#include "common.cuh"

namespace ct {
namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 32;  // elements per thread (16 packed bytes)

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
  int vector_ok;  // packed and out are 16-byte aligned
};

__device__ __forceinline__ float block_scale(const Nf4Params& p, int64_t group) {
  if (!p.nested) return __ldg(static_cast<const float*>(p.absmax) + group);
  const uint8_t q = __ldg(static_cast<const uint8_t*>(p.absmax) + group);
  const float decoded = __ldg(p.code2 + q);
  const float maximum = __ldg(p.absmax2 + group / p.blocksize2);
  return __fadd_rn(__fmul_rn(decoded, maximum), __ldg(p.offset));
}

template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* out, const float (&v)[kChunk]);

template <>
__device__ __forceinline__ void store_chunk<__nv_bfloat16>(__nv_bfloat16* out, const float (&v)[kChunk]) {
  uint4* dst = reinterpret_cast<uint4*>(out);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 pair = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&pair);
    }
    dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

template <>
__device__ __forceinline__ void store_chunk<__half>(__half* out, const float (&v)[kChunk]) {
  uint4* dst = reinterpret_cast<uint4*>(out);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 pair = __floats2half2_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&pair);
    }
    dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

template <>
__device__ __forceinline__ void store_chunk<float>(float* out, const float (&v)[kChunk]) {
  float4* dst = reinterpret_cast<float4*>(out);
#pragma unroll
  for (int q = 0; q < 8; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
}

template <typename OutT>
__global__ void __launch_bounds__(kThreads) nf4_decode_kernel(const Nf4Params p) {
  __shared__ float2 lut[256];
  {
    const int b = threadIdx.x;
    lut[b] = make_float2(__ldg(p.code + (b >> 4)), __ldg(p.code + (b & 15)));
  }
  __syncthreads();

  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t first = chunk * kChunk;
  if (first >= p.n) return;
  OutT* out = static_cast<OutT*>(p.out);

  if (p.vector_ok && first + kChunk <= p.n && p.blocksize % kChunk == 0) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p.packed + first / 2));
    const float scale = block_scale(p, first / p.blocksize);
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[kChunk];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float2 pair = lut[(words[w] >> (8 * b)) & 255u];
        v[8 * w + 2 * b] = round_dtype(__fmul_rn(pair.x, scale), p.state_dtype);
        v[8 * w + 2 * b + 1] = round_dtype(__fmul_rn(pair.y, scale), p.state_dtype);
      }
    }
    store_chunk<OutT>(out + first, v);
    return;
  }

  // Ragged tail, unaligned buffers or block sizes that are not multiples of 32:
  // one packed byte at a time, element stores guarded by n.
  const int64_t last = (first + kChunk < p.n) ? first + kChunk : p.n;
  for (int64_t e = first; e < last; e += 2) {
    const uint8_t byte = __ldg(p.packed + e / 2);
    const float2 pair = lut[byte];
    const float scale = block_scale(p, e / p.blocksize);
    out[e] = from_float<OutT>(round_dtype(__fmul_rn(pair.x, scale), p.state_dtype));
    if (e + 1 < p.n) out[e + 1] = from_float<OutT>(round_dtype(__fmul_rn(pair.y, scale), p.state_dtype));
  }
}

}  // namespace
}  // namespace ct

extern "C" int ct_nf4_decode(const uint8_t* packed, const void* absmax, const float* code,
                             const float* code2, const float* absmax2, const float* offset,
                             void* out, int64_t n, int blocksize, int blocksize2, int nested,
                             int state_dtype, int out_dtype, void* stream) {
  using namespace ct;
  if (n < 0 || blocksize <= 0 || (blocksize & 1)) return fail(CT_ERR_ARG, "ct_nf4_decode: n=%lld blocksize=%d", (long long)n, blocksize);
  if (n == 0) return CT_OK;
  if (!packed || !absmax || !code || !out) return fail(CT_ERR_ARG, "ct_nf4_decode: null pointer");
  if (nested && (!code2 || !absmax2 || !offset || blocksize2 <= 0)) return fail(CT_ERR_ARG, "ct_nf4_decode: nested statistics missing");
  if (state_dtype < CT_F32 || state_dtype > CT_F16 || out_dtype < CT_F32 || out_dtype > CT_F16)
    return fail(CT_ERR_ARG, "ct_nf4_decode: dtype");
  Nf4Params p{packed, absmax, code, code2, absmax2, offset, out, n, blocksize, blocksize2 > 0 ? blocksize2 : 1,
              nested, state_dtype,
              ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(out)) & 15) == 0};
  const int64_t chunks = (n + kChunk - 1) / kChunk;
  const unsigned blocks = static_cast<unsigned>((chunks + kThreads - 1) / kThreads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == CT_BF16) nf4_decode_kernel<__nv_bfloat16><<<blocks, kThreads, 0, s>>>(p);
  else if (out_dtype == CT_F16) nf4_decode_kernel<__half><<<blocks, kThreads, 0, s>>>(p);
  else nf4_decode_kernel<float><<<blocks, kThreads, 0, s>>>(p);
  count_launch(false);
  return check_launch("ct_nf4_decode");
}
