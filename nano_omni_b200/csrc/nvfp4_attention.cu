// Exact expansion of NVFP4 operands (e2m1 nibbles + one ue4m3 scale per 16 elements) to bf16.
//
// A product e2m1 x ue4m3 has at most five significant bits, so the bf16 result is exact: the dequantisation of the
// reference's ref_programs (src/nano_omni/kernels/attention/dense_nvfp4.py:638-676) as a utility for tests and for
// callers that want to attend on quantised operands with another kernel.  The attention kernels themselves
// (fa_fwd_nvfp4.cu) consume the packed operands directly.
//
// Operand layouts are those written by nob200_nvfp4_prepare: Q, K packed u8 [heads, P, 64] with
// scales [heads, P, 8]; V packed u8 [heads, 128, Pk/2] (channel-major, groups of 16 along tokens) with
// scales [heads, 128, Pk/16]; scales stored in 512-byte atoms of 128 rows x 4 groups.
#include "common.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

__device__ __forceinline__ size_t sf_offset(int r, int g, int groups) {
  return (static_cast<size_t>(r >> 7) * (groups >> 2) + (g >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (g & 3);
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}
__device__ __forceinline__ float e2m1_to_float(uint32_t code) {
  // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
  const uint32_t m = code & 7u;
  const float mag = m < 2 ? 0.5f * m : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
  return (code & 8u) ? -mag : mag;
}

// rows orientation: one thread per (row, group of 16): 8 packed bytes -> 16 bf16 (32 bytes)
__global__ void __launch_bounds__(256)
nvfp4_expand_rows_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                         __nv_bfloat16* __restrict__ out, int num_tokens, int heads, int padded, float multiplier) {
  const long long item = blockIdx.x * 256ll + threadIdx.x;  // (head, token, group)
  const long long total = static_cast<long long>(heads) * num_tokens * 8;
  if (item >= total) return;
  const int g = static_cast<int>(item & 7);
  const long long ht = item >> 3;
  const int token = static_cast<int>(ht % num_tokens), head = static_cast<int>(ht / num_tokens);
  const float sf = e4m3_to_float(scales[static_cast<size_t>(head) * padded * 8 + sf_offset(token, g, 8)]) * multiplier;
  const uint2 raw = *reinterpret_cast<const uint2*>(packed + (static_cast<size_t>(head) * padded + token) * 64 + g * 8);
  const uint32_t w[2] = {raw.x, raw.y};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = e2m1_to_float((w[i >> 2] >> (8 * (i & 3))) & 15u) * sf;
    const float b = e2m1_to_float((w[i >> 2] >> (8 * (i & 3) + 4)) & 15u) * sf;
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    o[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + (static_cast<size_t>(token) * heads + head) * 128 + g * 16);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// transposed orientation (V): CTA per (64 tokens, head); tile through shared memory
__global__ void __launch_bounds__(256)
nvfp4_expand_transposed_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                               __nv_bfloat16* __restrict__ out, int num_tokens, int heads, int padded,
                               float multiplier) {
  __shared__ __nv_bfloat16 tile[64][128 + 2];
  const int block = blockIdx.x, head = blockIdx.y;
  const int groups = padded / 16;
  // thread (channel c, 16-token group tg): 128 x 4 items, two per thread
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int item = k * 256 + threadIdx.x;
    const int c = item & 127, tg = item >> 7;
    const int g = block * 4 + tg;
    const float sf = e4m3_to_float(scales[static_cast<size_t>(head) * 128 * groups + sf_offset(c, g, groups)]) * multiplier;
    const uint2 raw = *reinterpret_cast<const uint2*>(packed + (static_cast<size_t>(head) * 128 + c) * (padded / 2) +
                                                      block * 32 + tg * 8);
    const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t code = (w[i >> 3] >> (4 * (i & 7))) & 15u;
      tile[tg * 16 + i][c] = __float2bfloat16_rn(e2m1_to_float(code) * sf);
    }
  }
  __syncthreads();
  // 64 tokens x 128 channels -> rows of 256 B; 16 lanes x 16 B per row
  const int lane16 = threadIdx.x & 15;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int t = p * 16 + (threadIdx.x >> 4);
    const int token = block * 64 + t;
    if (token < num_tokens) {
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        o[i] = *reinterpret_cast<const uint32_t*>(&tile[t][lane16 * 8 + 2 * i]);
      *reinterpret_cast<uint4*>(out + (static_cast<size_t>(token) * heads + head) * 128 + lane16 * 8) =
          make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace
}  // namespace nob200

using namespace nob200;

extern "C" int nob200_nvfp4_expand(int num_tokens, const void* quantized, const void* scales, void* output, int heads,
                                   int transpose, void* stream) {
  return nob200_nvfp4_expand_scaled(num_tokens, quantized, scales, output, heads, transpose, 1.0f, stream);
}

extern "C" int nob200_nvfp4_expand_scaled(int num_tokens, const void* quantized, const void* scales, void* output,
                                          int heads, int transpose, float multiplier, void* stream) {
  NOB_REQUIRE(num_tokens > 0 && heads > 0, "nvfp4_expand: sizes must be positive");
  NOB_REQUIRE(quantized && scales && output, "nvfp4_expand: NULL tensor");
  NOB_REQUIRE(heads <= 65535, "nvfp4_expand: heads exceed the grid limit");
  const int padded = (num_tokens + 127) / 128 * 128;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!transpose) {
    const long long total = static_cast<long long>(heads) * num_tokens * 8;
    nvfp4_expand_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
        static_cast<const uint8_t*>(quantized), static_cast<const uint8_t*>(scales),
        static_cast<__nv_bfloat16*>(output), num_tokens, heads, padded, multiplier);
  } else {
    nvfp4_expand_transposed_kernel<<<dim3((num_tokens + 63) / 64, heads), 256, 0, s>>>(
        static_cast<const uint8_t*>(quantized), static_cast<const uint8_t*>(scales),
        static_cast<__nv_bfloat16*>(output), num_tokens, heads, padded, multiplier);
  }
  return check_launch("nvfp4_expand");
}
