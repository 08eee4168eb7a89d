// Quantisers that feed the int8-fp8 and nvfp4 attention kernels, plus the
// per-channel statistics they need.  All are HBM-bound CUDA-core kernels built
// around 16-byte loads; none uses fast-math, because their outputs are compared
// byte for byte with IEEE fp32 arithmetic (divide, round-half-even).
//
// Reference programs replaced here:
//   token_group_mean          src/nano_omni/kernels/normalization/token_group_mean.py:51-116
//   int8_fp8_quantize_qk      src/nano_omni/kernels/attention/int8_fp8/quantize_qk.py:18-68
//   int8_fp8_value_scale      src/nano_omni/kernels/attention/int8_fp8/value_scale.py:18-55
//   int8_fp8_quantize_value   src/nano_omni/kernels/attention/int8_fp8/quantize_value.py:20-65
//   nvfp4_prepare             src/nano_omni/kernels/attention/nvfp4_prepare.py:37-113
#include <cuda_fp4.h>

#include <mutex>

#include "common.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

constexpr float kInvSqrt128 = 0.08838834764831845f;

struct Vec8 {
  float v[8];
};

__device__ __forceinline__ Vec8 load8_bf16(const __nv_bfloat16* p) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  Vec8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    r.v[2 * i] = __uint_as_float(w[i] << 16);
    r.v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
  return r;
}

// Normalised 128-point Walsh-Hadamard transform (Sylvester order) of a row that
// is spread over 16 consecutive lanes, 8 consecutive channels per lane.  The
// butterfly network (strides 1,2,4 in registers, then 8..64 across lanes) fixes
// the order of every fp32 add, so any implementation of the same network is
// bit-identical; the result is multiplied by fl(1/sqrt(128)) at the end.
__device__ __forceinline__ void hadamard128(Vec8& x, int lane16) {
#pragma unroll
  for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & h) == 0) {
        const float a = x.v[i], b = x.v[i + h];
        x.v[i] = a + b;
        x.v[i + h] = a - b;
      }
    }
  }
#pragma unroll
  for (int m = 1; m < 16; m <<= 1) {
    const bool upper = (lane16 & m) != 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, x.v[i], m);
      x.v[i] = upper ? (other - x.v[i]) : (x.v[i] + other);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) x.v[i] *= kInvSqrt128;
}

__device__ __forceinline__ float vec_absmax(const Vec8& x) {
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(x.v[i]));
  return m;
}

// ------------------------------------------------------- rotation of bf16 rows
// The transform of the quantisers applied to rows of 128 bf16 (it is its own inverse): brings an attention output
// computed on rotated V back to the original channels.  16 lanes per row, 16 rows per CTA round; in place allowed.
__global__ void __launch_bounds__(256)
hadamard_rows_kernel(const __nv_bfloat16* src, __nv_bfloat16* dst, long long rows, int heads, int total_heads,
                     int head_offset) {  // row r = (token, head) -> tensor row token * total_heads + head_offset + head
  const int lane16 = threadIdx.x & 15;
  const long long stride = static_cast<long long>(gridDim.x) * 16;
  for (long long base = static_cast<long long>(blockIdx.x) * 16; base < rows; base += stride) {
    const long long row = base + (threadIdx.x >> 4);
    const bool live = row < rows;
    const long long r = live ? row : 0;
    const long long at = ((r / heads) * total_heads + head_offset + (r % heads)) * 128 + 8 * lane16;
    Vec8 x = load8_bf16(src + at);
    hadamard128(x, lane16);
    if (live) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(x.v[2 * i], x.v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&v);
      }
      *reinterpret_cast<uint4*>(dst + at) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// ------------------------------------------------------------ column mean
// Canonical summation order (the CPU restatement uses the same): tokens of a
// group are cut into chunks of 128; each chunk is summed sequentially in token
// order starting from the first token; chunk sums are then added sequentially
// in chunk order; the total is divided (IEEE) by the group's divisor.
constexpr int kMeanChunk = 128;

__global__ void __launch_bounds__(128)
mean_chunk_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ dst, int num_tokens, int columns,
                  int tokens_per_block, int chunks_per_group, int include_padding, int direct) {
  const int col = (blockIdx.x * 128 + threadIdx.x) * 4;
  if (col >= columns) return;
  const int chunk_id = blockIdx.y;  // group * chunks_per_group + chunk
  const int group = chunk_id / chunks_per_group, chunk = chunk_id % chunks_per_group;
  const int group_begin = group * tokens_per_block;
  const int begin = group_begin + chunk * kMeanChunk;
  int end = min(begin + kMeanChunk, group_begin + tokens_per_block);
  end = min(end, num_tokens);
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  const __nv_bfloat16* p = in + static_cast<size_t>(begin) * columns + col;
#pragma unroll 8
  for (int t = begin; t < end; ++t, p += columns) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    a0 += __uint_as_float(raw.x << 16);
    a1 += __uint_as_float(raw.x & 0xffff0000u);
    a2 += __uint_as_float(raw.y << 16);
    a3 += __uint_as_float(raw.y & 0xffff0000u);
  }
  if (direct) {
    const int valid = min(tokens_per_block, num_tokens - group_begin);
    const float div = static_cast<float>(include_padding ? tokens_per_block : valid);
    a0 /= div, a1 /= div, a2 /= div, a3 /= div;
  }
  *reinterpret_cast<float4*>(dst + static_cast<size_t>(chunk_id) * columns + col) = make_float4(a0, a1, a2, a3);
}

// One CTA per (32 columns, group).  The chunk sums of a column are added by ONE thread in chunk order (the canonical
// order), but they are fetched by the whole CTA, 256 chunks at a time with every load in flight at once, through
// shared memory: a thread fetching its own column's sums one after the other pays an L2 round trip per handful.
constexpr int kFinishChunks = 256;

__global__ void __launch_bounds__(256)
mean_finish_kernel(const float* __restrict__ partial, float* __restrict__ out, int num_tokens, int columns,
                   int tokens_per_block, int chunks_per_group, int include_padding) {
  __shared__ float tile[kFinishChunks][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  const int group = blockIdx.y;
  const int group_begin = group * tokens_per_block;
  const int valid = min(tokens_per_block, num_tokens - group_begin);
  const int used = (valid + kMeanChunk - 1) / kMeanChunk;
  const float* p = partial + static_cast<size_t>(group) * chunks_per_group * columns + min(col, columns - 1);
  float acc = 0.f;
  for (int c0 = 0; c0 < used; c0 += kFinishChunks) {
    const int m = min(kFinishChunks, used - c0);
    float v[kFinishChunks / 8];
#pragma unroll
    for (int k = 0; k < kFinishChunks / 8; ++k) {
      const int r = warp + 8 * k;
      v[k] = r < m ? p[static_cast<size_t>(c0 + r) * columns] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < kFinishChunks / 8; ++k) tile[warp + 8 * k][lane] = v[k];
    __syncthreads();
    if (warp == 0) {
      int r = 0;
      if (c0 == 0) acc = tile[0][lane], r = 1;
      for (; r < m; ++r) acc += tile[r][lane];
    }
    __syncthreads();
  }
  if (warp == 0 && col < columns) {
    const float div = static_cast<float>(include_padding ? tokens_per_block : valid);
    out[static_cast<size_t>(group) * columns + col] = acc / div;
  }
}

// ------------------------------------------------------- int8 Q/K quantiser
// One CTA per (token block, head).  A row of 128 channels is held by 16 lanes.  The block's rows stay in registers as
// the 16-byte pieces they were loaded as and are converted twice (once for the maximum, once for the codes): half the
// registers of holding them as fp32, so five CTAs fit an SM and enough loads are in flight to keep HBM busy.
template <int TPB, bool HADAMARD>
__global__ void __launch_bounds__(TPB >= 64 ? 256 : 128, (TPB == 128 || HADAMARD) ? 1 : (TPB == 64 ? 5 : 10))
quantize_qk_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ mean,
                   int8_t* __restrict__ quantized, float* __restrict__ scales, int num_tokens, int heads,
                   int num_blocks, int center) {
  constexpr int kThreads = TPB >= 64 ? 256 : 128;
  constexpr int kRowsPerPass = kThreads / 16;
  constexpr int kPasses = TPB / kRowsPerPass;
  const int head = blockIdx.x, block = blockIdx.y;  // heads fastest: CTAs in flight read whole rows of the source
  const int lane16 = threadIdx.x & 15, row_in_pass = threadIdx.x >> 4;
  const int columns = heads * 128;
  const int ch = head * 128 + lane16 * 8;

  uint4 raw[kPasses];
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const int token = block * TPB + p * kRowsPerPass + row_in_pass;
    raw[p] = token < num_tokens ? __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(token) * columns + ch))
                                : make_uint4(0u, 0u, 0u, 0u);
  }
  Vec8 mu;
#pragma unroll
  for (int i = 0; i < 8; ++i) mu.v[i] = 0.f;
  if (center) {
    const float4 m0 = *reinterpret_cast<const float4*>(mean + ch);
    const float4 m1 = *reinterpret_cast<const float4*>(mean + ch + 4);
    mu.v[0] = m0.x, mu.v[1] = m0.y, mu.v[2] = m0.z, mu.v[3] = m0.w;
    mu.v[4] = m1.x, mu.v[5] = m1.y, mu.v[6] = m1.z, mu.v[7] = m1.w;
  }
  // row p of this thread as fp32, centred and rotated (rows past the end are zero, as the padding requires)
  auto row_values = [&](int p) {
    const uint32_t w[4] = {raw[p].x, raw[p].y, raw[p].z, raw[p].w};
    Vec8 x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x.v[2 * i] = __uint_as_float(w[i] << 16);
      x.v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
    const int token = block * TPB + p * kRowsPerPass + row_in_pass;
    if (center && token < num_tokens) {
#pragma unroll
      for (int i = 0; i < 8; ++i) x.v[i] -= mu.v[i];
    }
    if (HADAMARD) hadamard128(x, lane16);
    return x;
  };
  float amax = 0.f;
#pragma unroll
  for (int p = 0; p < kPasses; ++p) amax = fmaxf(amax, vec_absmax(row_values(p)));
  __shared__ float warp_max[kThreads / 32];
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) amax = fmaxf(amax, warp_max[w]);
  const float scale = fmaxf(amax / 127.0f, 1e-10f);
  const float inv_scale = __frcp_rn(scale);
  if (threadIdx.x == 0) scales[static_cast<size_t>(head) * num_blocks + block] = scale;
  int8_t* dst_base = quantized + (static_cast<size_t>(head) * num_blocks * TPB + static_cast<size_t>(block) * TPB) * 128;
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const int r = p * kRowsPerPass + row_in_pass;
    const Vec8 xp = row_values(p);
    // The result must be rint(RN(x / scale)).  x * RN(1/scale) is within 2.6e-5 of RN(x / scale) for
    // |x / scale| <= 128, so both round to the same integer unless the product lies within 4e-5 of a
    // half-integer; only then (about one element in 10^4) the IEEE division is done.  Rounding and the
    // conversion to an integer are one addition: 2^23 * 1.5 + a, rounded to nearest even by the adder, holds
    // rint(a) in its low mantissa bits (two's complement in the low byte once clamped to [-128, 127]).
    constexpr float kRound = 12582912.0f;
    uint32_t bits[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = xp.v[i] * inv_scale;
      float t = a + kRound;
      const float q = t - kRound;
      if (0.5f - fabsf(a - q) < 4e-5f) t = rintf(__fdiv_rn(xp.v[i], scale)) + kRound;
      bits[i] = __float_as_uint(fminf(fmaxf(t, kRound - 128.f), kRound + 127.f));
    }
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h)
      w[h] = __byte_perm(__byte_perm(bits[4 * h], bits[4 * h + 1], 0x0040), __byte_perm(bits[4 * h + 2], bits[4 * h + 3], 0x0040), 0x5410);
    *reinterpret_cast<uint2*>(dst_base + r * 128 + lane16 * 8) = make_uint2(w[0], w[1]);
  }
}

// ------------------------------------------------------------- V statistics
// amax[c] over all tokens, accumulated with atomicMax on the (non-negative) bit
// pattern, then turned into max(amax / 2.25, 1e-10) in place.
constexpr int kVScaleTokens = 256;

__global__ void __launch_bounds__(256)
value_amax_kernel(const __nv_bfloat16* __restrict__ src, uint32_t* __restrict__ amax_bits, int num_tokens,
                  int columns) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = (blockIdx.x * 32 + lane) * 8;
  const int begin = blockIdx.y * kVScaleTokens;
  const int end = min(begin + kVScaleTokens, num_tokens);
  __shared__ uint32_t part[8][32][8];
  uint32_t m[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < columns) {
#pragma unroll 4
    for (int t = begin + warp; t < end; t += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(t) * columns + col);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // |bf16| as fp32 bit patterns; integer max == float max for non-negative values
        m[2 * i] = max(m[2 * i], (w[i] << 16) & 0x7fffffffu);
        m[2 * i + 1] = max(m[2 * i + 1], w[i] & 0x7fff0000u);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[warp][lane][i] = m[i];
  __syncthreads();
  if (warp == 0 && col < columns) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t v = part[0][lane][i];
#pragma unroll
      for (int w = 1; w < 8; ++w) v = max(v, part[w][lane][i]);
      atomicMax(amax_bits + col + i, v);
    }
  }
}

__global__ void value_scale_finish_kernel(float* __restrict__ scales, int columns) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < columns) scales[c] = fmaxf(scales[c] / 2.25f, 1e-10f);
}

// ------------------------------------------------------------ V -> fp8 e4m3
// One CTA per (64-token block, head): scale, round to e4m3, transpose to channel-major, and place
// token s of each group of 16 at position ((s&7)>>1)*4 + (s>>3)*2 + (s&1)  (inverse of
// [0,1,8,9,2,3,10,11,4,5,12,13,6,7,14,15]).  A thread owns 8 channels of the four tokens that share
// one 32-bit output word, so shared memory is written in words, not bytes.
// The byte must equal e4m3(RN(x / scale)).  x * RN(1/scale) is within 1.8e-7 (relative) of RN(x / scale);
// if the product moved by +-4e-7 (relative) rounds to the same byte on both sides, that byte is the
// answer; otherwise (about one element in 10^5) the IEEE division is done.
__device__ __forceinline__ uint32_t e4m3_of_quotient(float x, float scale, float inv_scale) {
  const float a = x * inv_scale;
  const uint32_t pair = __nv_cvt_float2_to_fp8x2(make_float2(a * (1.0f + 4e-7f), a * (1.0f - 4e-7f)), __NV_SATFINITE,
                                                 __NV_E4M3);
  if ((pair & 0xffu) == (pair >> 8)) return pair & 0xffu;
  return __nv_cvt_float_to_fp8(__fdiv_rn(x, scale), __NV_SATFINITE, __NV_E4M3);
}

__global__ void __launch_bounds__(256)
quantize_value_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ scale,
                      uint8_t* __restrict__ out, int num_tokens, int heads, int padded_tokens) {
  // [channel][word of four stored positions]; the word index is XORed with the channel's group of 8 so
  // that the 16 channel groups of a warp hit 16 different banks
  __shared__ __align__(16) uint32_t tile[128][16];
  const int head = blockIdx.x, block = blockIdx.y;  // heads fastest: CTAs in flight read whole rows of the source
  const int columns = heads * 128;
  const int lane16 = threadIdx.x & 15, word = threadIdx.x >> 4;  // 16 channel groups x 16 output words
  const int ch = lane16 * 8;
  float sc[8], inv[8];
  {
    const float4 s0 = *reinterpret_cast<const float4*>(scale + head * 128 + ch);
    const float4 s1 = *reinterpret_cast<const float4*>(scale + head * 128 + ch + 4);
    sc[0] = s0.x, sc[1] = s0.y, sc[2] = s0.z, sc[3] = s0.w;
    sc[4] = s1.x, sc[5] = s1.y, sc[6] = s1.z, sc[7] = s1.w;
#pragma unroll
    for (int i = 0; i < 8; ++i) inv[i] = __frcp_rn(sc[i]);
  }
  // stored positions 4*word .. 4*word+3 hold source tokens 16*(word/4) + {2w', 2w'+1, 8+2w', 9+2w'}, w' = word%4
  const int base_token = block * 64 + 16 * (word >> 2) + 2 * (word & 3);
  uint32_t packed[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  uint4 loaded[4];  // all four loads are issued before the first conversion
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int token = base_token + (b & 1) + 8 * (b >> 1);
    loaded[b] = token < num_tokens
                 ? __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(token) * columns + head * 128 + ch))
                 : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const uint32_t w[4] = {loaded[b].x, loaded[b].y, loaded[b].z, loaded[b].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      packed[2 * i] |= e4m3_of_quotient(__uint_as_float(w[i] << 16), sc[2 * i], inv[2 * i]) << (8 * b);
      packed[2 * i + 1] |= e4m3_of_quotient(__uint_as_float(w[i] & 0xffff0000u), sc[2 * i + 1], inv[2 * i + 1]) << (8 * b);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) tile[ch + i][word ^ lane16] = packed[i];
  __syncthreads();
  // 128 channels x 64 bytes: 512 16-byte pieces
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int piece = k * 256 + threadIdx.x;
    const int c = piece >> 2, part = piece & 3;
    const int key = (c >> 3) & 15;  // logical word w sits at w ^ key: same aligned group of four, permuted inside
    const uint4 raw = *reinterpret_cast<const uint4*>(&tile[c][4 * (part ^ (key >> 2))]);
    const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
    uint4 v;
    const int k2 = key & 3;
    v.x = k2 == 0 ? r[0] : k2 == 1 ? r[1] : k2 == 2 ? r[2] : r[3];
    v.y = k2 == 0 ? r[1] : k2 == 1 ? r[0] : k2 == 2 ? r[3] : r[2];
    v.z = k2 == 0 ? r[2] : k2 == 1 ? r[3] : k2 == 2 ? r[0] : r[1];
    v.w = k2 == 0 ? r[3] : k2 == 1 ? r[2] : k2 == 2 ? r[1] : r[0];
    *reinterpret_cast<uint4*>(out + (static_cast<size_t>(head) * 128 + c) * padded_tokens + block * 64 + part * 16) = v;
  }
}

// ---------------------------------------------------------------- NVFP4
// Two e2m1 codes (round to nearest, ties to the even code, saturating at 6, sign kept for zeros):
// `lo` in bits 0-3, `hi` in bits 4-7.  One cvt.rn.satfinite.e2m1x2.f32.
__device__ __forceinline__ uint32_t e2m1_pair(float lo, float hi) {
  return __nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}
// Block scale and the factor that multiplies (or divides) the 16 values.
// global_scale == 0: sf = e4m3(min(amax/6, 448)), y = x * (1/sf)   (attention prepare)
// global_scale  > 0: bs = amax/(G*6) kept in fp32 for y = x / (bs*G); stored e4m3(bs)
struct Fp4Scale {
  uint8_t byte;
  float factor;
  bool divide;
};
__device__ __forceinline__ Fp4Scale fp4_scale(float amax, float global_scale) {
  Fp4Scale r;
  if (global_scale > 0.f) {
    const float bs = amax / (global_scale * 6.0f);
    r.byte = __nv_cvt_float_to_fp8(bs, __NV_SATFINITE, __NV_E4M3);
    r.factor = (bs == 0.f ? 1.0f : bs) * global_scale;
    r.divide = true;
  } else {
    r.byte = __nv_cvt_float_to_fp8(fminf(amax / 6.0f, 448.0f), __NV_SATFINITE, __NV_E4M3);
    const float sf = e4m3_to_float(r.byte);
    r.factor = (sf == 0.f) ? 0.f : 1.0f / sf;
    r.divide = false;
  }
  return r;
}
__device__ __forceinline__ float fp4_apply(float x, const Fp4Scale& s) { return s.divide ? x / s.factor : x * s.factor; }

// Byte offset of the scale of (row r, 16-group g) inside one head's scale plane
// with `groups` 16-groups per row: 512-byte atoms of 128 rows x 4 groups,
// atoms ordered row-block major, then group-block; inside an atom
// (r%32)*16 + ((r%128)/32)*4 + g%4.
__device__ __forceinline__ size_t sf_offset(int r, int g, int groups) {
  return (static_cast<size_t>(r >> 7) * (groups >> 2) + (g >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (g & 3);
}

// Q/K orientation: rows are tokens (padded to 128), 8 groups of 16 channels.
__global__ void __launch_bounds__(256)
nvfp4_prepare_rows_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ mean,
                          uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, int num_tokens, int heads,
                          int padded_tokens, int hadamard, float global_scale) {
  constexpr int kRows = 4;  // rows per thread: their loads are all in flight before the first is used
  const int head = blockIdx.x;  // heads fastest: CTAs in flight read whole rows of the source
  const int lane16 = threadIdx.x & 15;
  const int first_row = blockIdx.y * (16 * kRows) + (threadIdx.x >> 4);
  const int columns = heads * 128;
  const int ch = lane16 * 8;
  uint4 loaded[kRows];
#pragma unroll
  for (int p = 0; p < kRows; ++p) {
    const int row = first_row + 16 * p;
    loaded[p] = row < num_tokens
                    ? __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(row) * columns + head * 128 + ch))
                    : make_uint4(0u, 0u, 0u, 0u);
  }
  float mu[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (mean) {
    const float4 m0 = *reinterpret_cast<const float4*>(mean + head * 128 + ch);
    const float4 m1 = *reinterpret_cast<const float4*>(mean + head * 128 + ch + 4);
    mu[0] = m0.x, mu[1] = m0.y, mu[2] = m0.z, mu[3] = m0.w;
    mu[4] = m1.x, mu[5] = m1.y, mu[6] = m1.z, mu[7] = m1.w;
  }
  uint8_t* head_packed = packed + static_cast<size_t>(head) * padded_tokens * 64;
  uint8_t* head_sf = scales + static_cast<size_t>(head) * padded_tokens * 8;
#pragma unroll
  for (int p = 0; p < kRows; ++p) {
    const int row = first_row + 16 * p;  // < padded_tokens: the grid covers exactly the padded rows (a multiple of 128)
    const uint32_t w[4] = {loaded[p].x, loaded[p].y, loaded[p].z, loaded[p].w};
    Vec8 x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x.v[2 * i] = __uint_as_float(w[i] << 16);
      x.v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
    if (row < num_tokens) {
#pragma unroll
      for (int i = 0; i < 8; ++i) x.v[i] -= mu[i];
    }
    if (hadamard) hadamard128(x, lane16);
    float amax = vec_absmax(x);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const Fp4Scale s = fp4_scale(amax, global_scale);
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; i += 2) word |= e2m1_pair(fp4_apply(x.v[i], s), fp4_apply(x.v[i + 1], s)) << (4 * i);
    *reinterpret_cast<uint32_t*>(head_packed + static_cast<size_t>(row) * 64 + lane16 * 4) = word;
    if ((lane16 & 1) == 0) head_sf[sf_offset(row, lane16 >> 1, 8)] = s.byte;
  }
}

// V orientation: rows are the 128 channels, groups of 16 run along tokens.
// One CTA per (64-token block, head); the tile is transposed through shared memory.
template <bool HADAMARD>
__global__ void __launch_bounds__(256)
nvfp4_prepare_transposed_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ mean,
                                uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, int num_tokens, int heads,
                                int padded_tokens, float global_scale) {
  // 64 tokens x 128 channels pass through shared memory to change hands from (token, 8 channels) to (channel, 16
  // tokens).  Without the rotation the tile holds the bf16 pieces as loaded (16-byte stores, 2-byte loads, no bank
  // conflicts either way) and the mean is subtracted after the transposition; with it, rows must be centred and
  // rotated first and the tile holds fp32.
  using Cell = std::conditional_t<HADAMARD, float, __nv_bfloat16>;
  constexpr int kPitch = HADAMARD ? 129 : 128;
  __shared__ __align__(16) Cell tile[64][kPitch];
  const int head = blockIdx.x, block = blockIdx.y;  // heads fastest: CTAs in flight read whole rows of the source
  const int columns = heads * 128;
  const int lane16 = threadIdx.x & 15;
  const int ch = lane16 * 8;
  uint4 loaded[4];  // all four loads are issued before the first use
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int token = block * 64 + p * 16 + (threadIdx.x >> 4);
    loaded[p] = token < num_tokens
                    ? __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(token) * columns + head * 128 + ch))
                    : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int t = p * 16 + (threadIdx.x >> 4);
    if constexpr (HADAMARD) {
      const uint32_t w[4] = {loaded[p].x, loaded[p].y, loaded[p].z, loaded[p].w};
      Vec8 x;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x.v[2 * i] = __uint_as_float(w[i] << 16);
        x.v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
      if (mean && block * 64 + t < num_tokens) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x.v[i] -= mean[head * 128 + ch + i];
      }
      hadamard128(x, lane16);
#pragma unroll
      for (int i = 0; i < 8; ++i) tile[t][ch + i] = x.v[i];
    } else {
      *reinterpret_cast<uint4*>(&tile[t][ch]) = loaded[p];
    }
  }
  __syncthreads();
  const int groups = padded_tokens / 16;
  uint8_t* head_packed = packed + static_cast<size_t>(head) * 128 * (padded_tokens / 2);
  uint8_t* head_sf = scales + static_cast<size_t>(head) * 128 * groups;
  // one item per thread: (channel, pair of 16-token groups)
  const int c = threadIdx.x & 127, pair = threadIdx.x >> 7;
  const float mu = (!HADAMARD && mean) ? mean[head * 128 + c] : 0.f;
  uint32_t words[4];
  uint8_t sf[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int t0 = (pair * 2 + g) * 16;
    float v[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if constexpr (HADAMARD) {
        v[i] = tile[t0 + i][c];
      } else {
        v[i] = __bfloat162float(tile[t0 + i][c]);
        if (block * 64 + t0 + i < num_tokens) v[i] -= mu;  // rows past the end stay zero
      }
      amax = fmaxf(amax, fabsf(v[i]));
    }
    const Fp4Scale s = fp4_scale(amax, global_scale);
    sf[g] = s.byte;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      lo |= e2m1_pair(fp4_apply(v[i], s), fp4_apply(v[i + 1], s)) << (4 * i);
      hi |= e2m1_pair(fp4_apply(v[8 + i], s), fp4_apply(v[9 + i], s)) << (4 * i);
    }
    words[2 * g] = lo;
    words[2 * g + 1] = hi;
  }
  *reinterpret_cast<uint4*>(head_packed + static_cast<size_t>(c) * (padded_tokens / 2) + block * 32 + pair * 16) =
      make_uint4(words[0], words[1], words[2], words[3]);
  const int g0 = block * 4 + pair * 2;
  *reinterpret_cast<uint16_t*>(head_sf + sf_offset(c, g0, groups)) =
      static_cast<uint16_t>(sf[0]) | (static_cast<uint16_t>(sf[1]) << 8);
}

}  // namespace
}  // namespace nob200

using namespace nob200;

extern "C" size_t nob200_token_group_mean_workspace_bytes(int num_tokens, int columns, int tokens_per_block) {
  if (num_tokens <= 0 || columns <= 0 || tokens_per_block <= 0) return 0;
  const size_t chunks_per_group = (static_cast<size_t>(tokens_per_block) + kMeanChunk - 1) / kMeanChunk;
  if (chunks_per_group <= 1) return 0;
  const size_t groups = (static_cast<size_t>(num_tokens) + tokens_per_block - 1) / tokens_per_block;
  return groups * chunks_per_group * columns * sizeof(float);
}

extern "C" int nob200_token_group_mean(int num_tokens, const void* input, void* output, int columns,
                                       int tokens_per_block, int include_padding, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  NOB_REQUIRE(num_tokens > 0 && columns > 0 && tokens_per_block > 0, "token_group_mean: sizes must be positive");
  NOB_REQUIRE(columns % 4 == 0, "token_group_mean: columns (%d) must be a multiple of 4", columns);
  NOB_REQUIRE(input && output, "token_group_mean: NULL tensor");
  // a group never spans more than the tokens that exist
  const int eff_tpb = tokens_per_block;
  const int groups = (num_tokens + eff_tpb - 1) / eff_tpb;
  const int chunks_per_group = (eff_tpb + kMeanChunk - 1) / kMeanChunk;
  const size_t need = nob200_token_group_mean_workspace_bytes(num_tokens, columns, tokens_per_block);
  NOB_REQUIRE(need == 0 || (workspace && workspace_bytes >= need),
              "token_group_mean: workspace of %zu B required, %zu B given", need, workspace_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int col_blocks = (columns / 4 + 127) / 128;
  // Only chunks that hold at least one token are launched per group; the grid's y
  // covers groups*chunks_per_group and empty chunks write zeros that are never read.
  const long long total_chunks = static_cast<long long>(groups) * chunks_per_group;
  NOB_REQUIRE(total_chunks <= 65535, "token_group_mean: %lld chunks exceed the grid limit", total_chunks);
  if (chunks_per_group == 1) {
    mean_chunk_kernel<<<dim3(col_blocks, (unsigned)total_chunks), 128, 0, s>>>(
        static_cast<const __nv_bfloat16*>(input), static_cast<float*>(output), num_tokens, columns, eff_tpb, 1,
        include_padding, 1);
    return check_launch("token_group_mean");
  }
  mean_chunk_kernel<<<dim3(col_blocks, (unsigned)total_chunks), 128, 0, s>>>(
      static_cast<const __nv_bfloat16*>(input), static_cast<float*>(workspace), num_tokens, columns, eff_tpb,
      chunks_per_group, include_padding, 0);
  int rc = check_launch("token_group_mean(partial)");
  if (rc) return rc;
  mean_finish_kernel<<<dim3((columns + 31) / 32, groups), 256, 0, s>>>(
      static_cast<const float*>(workspace), static_cast<float*>(output), num_tokens, columns, eff_tpb,
      chunks_per_group, include_padding);
  return check_launch("token_group_mean(finish)");
}

extern "C" int nob200_int8_fp8_quantize_qk(int num_tokens, const void* source, const void* statistics,
                                           void* quantized, void* scales, int heads, int tokens_per_block, int center,
                                           int hadamard, void* stream) {
  NOB_REQUIRE(num_tokens > 0 && heads > 0, "int8_fp8_quantize_qk: sizes must be positive");
  NOB_REQUIRE(tokens_per_block == 32 || tokens_per_block == 64 || tokens_per_block == 128,
              "int8_fp8_quantize_qk: tokens_per_block must be 32, 64 or 128 (got %d)", tokens_per_block);
  NOB_REQUIRE(source && quantized && scales, "int8_fp8_quantize_qk: NULL tensor");
  NOB_REQUIRE(!center || statistics, "int8_fp8_quantize_qk: centring needs the statistics tensor");
  const int num_blocks = (num_tokens + tokens_per_block - 1) / tokens_per_block;
  NOB_REQUIRE(num_blocks <= 65535, "int8_fp8_quantize_qk: %d token blocks exceed the grid limit", num_blocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(heads, num_blocks);
  const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(source);
  const float* mean = static_cast<const float*>(statistics);
  int8_t* q = static_cast<int8_t*>(quantized);
  float* sc = static_cast<float*>(scales);
  auto launch = [&](auto tokens_tag, auto hadamard_tag) {
    constexpr int kTokens = decltype(tokens_tag)::value;
    quantize_qk_kernel<kTokens, decltype(hadamard_tag)::value>
        <<<grid, kTokens >= 64 ? 256 : 128, 0, s>>>(src, mean, q, sc, num_tokens, heads, num_blocks, center);
  };
  auto by_rotation = [&](auto tokens_tag) {
    if (hadamard)
      launch(tokens_tag, std::true_type{});
    else
      launch(tokens_tag, std::false_type{});
  };
  if (tokens_per_block == 32)
    by_rotation(std::integral_constant<int, 32>{});
  else if (tokens_per_block == 64)
    by_rotation(std::integral_constant<int, 64>{});
  else
    by_rotation(std::integral_constant<int, 128>{});
  return check_launch("int8_fp8_quantize_qk");
}

extern "C" int nob200_int8_fp8_value_scale(int num_tokens, const void* source, void* scales, int heads,
                                           void* stream) {
  NOB_REQUIRE(num_tokens > 0 && heads > 0, "int8_fp8_value_scale: sizes must be positive");
  NOB_REQUIRE(source && scales, "int8_fp8_value_scale: NULL tensor");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int columns = heads * 128;
  cudaError_t err = cudaMemsetAsync(scales, 0, static_cast<size_t>(columns) * sizeof(float), s);
  if (err != cudaSuccess) return fail(kCudaError, "int8_fp8_value_scale: %s", cudaGetErrorString(err));
  const int token_blocks = (num_tokens + kVScaleTokens - 1) / kVScaleTokens;
  NOB_REQUIRE(token_blocks <= 65535, "int8_fp8_value_scale: too many tokens");
  value_amax_kernel<<<dim3((columns + 255) / 256, token_blocks), 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(source), static_cast<uint32_t*>(scales), num_tokens, columns);
  int rc = check_launch("int8_fp8_value_scale(amax)");
  if (rc) return rc;
  value_scale_finish_kernel<<<(columns + 255) / 256, 256, 0, s>>>(static_cast<float*>(scales), columns);
  return check_launch("int8_fp8_value_scale(finish)");
}

extern "C" int nob200_int8_fp8_quantize_value(int num_tokens, const void* source, const void* scale, void* output,
                                              int heads, void* stream) {
  NOB_REQUIRE(num_tokens > 0 && heads > 0, "int8_fp8_quantize_value: sizes must be positive");
  NOB_REQUIRE(source && scale && output, "int8_fp8_quantize_value: NULL tensor");
  const int blocks = (num_tokens + 63) / 64;
  NOB_REQUIRE(blocks <= 65535, "int8_fp8_quantize_value: %d token blocks exceed the grid limit", blocks);
  quantize_value_kernel<<<dim3(heads, blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(source), static_cast<const float*>(scale), static_cast<uint8_t*>(output),
      num_tokens, heads, blocks * 64);
  return check_launch("int8_fp8_quantize_value");
}

extern "C" int nob200_nvfp4_prepare(int num_tokens, const void* source, const void* mean, void* quantized,
                                    void* scales, int heads, int transpose, int hadamard, float global_scale,
                                    void* stream) {
  NOB_REQUIRE(num_tokens > 0 && heads > 0, "nvfp4_prepare: sizes must be positive");
  NOB_REQUIRE(source && quantized && scales, "nvfp4_prepare: NULL tensor");
  NOB_REQUIRE(num_tokens <= 65535 * 16, "nvfp4_prepare: %d tokens exceed the grid limit", num_tokens);
  NOB_REQUIRE(global_scale >= 0.f, "nvfp4_prepare: global_scale must be >= 0 (0 selects per-block scales only)");
  const int padded = (num_tokens + 127) / 128 * 128;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!transpose) {
    nvfp4_prepare_rows_kernel<<<dim3(heads, padded / 64), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(source), static_cast<const float*>(mean), static_cast<uint8_t*>(quantized),
        static_cast<uint8_t*>(scales), num_tokens, heads, padded, hadamard, global_scale);
  } else {
    if (hadamard)
      nvfp4_prepare_transposed_kernel<true><<<dim3(heads, padded / 64), 256, 0, s>>>(
          static_cast<const __nv_bfloat16*>(source), static_cast<const float*>(mean), static_cast<uint8_t*>(quantized),
          static_cast<uint8_t*>(scales), num_tokens, heads, padded, global_scale);
    else
      nvfp4_prepare_transposed_kernel<false><<<dim3(heads, padded / 64), 256, 0, s>>>(
          static_cast<const __nv_bfloat16*>(source), static_cast<const float*>(mean), static_cast<uint8_t*>(quantized),
          static_cast<uint8_t*>(scales), num_tokens, heads, padded, global_scale);
  }
  return check_launch("nvfp4_prepare");
}

// ------------------------------------------------- column mean, no allocation
// Scratch for nob200_token_group_mean_static: a fixed array in device memory that
// every GPU loading this library holds until the process exits.  In host code the
// array's name is only a handle; the address a kernel may use comes from
// cudaGetSymbolAddress, queried once per device with that device current.
static __device__ __align__(256) unsigned char g_static_mean_scratch[NOB200_STATIC_MEAN_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;

int static_mean_scratch_ptr(float** out) {
  static std::mutex mutex;
  static float* per_device[kMaxDevices] = {};
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return fail(kCudaError, "token_group_mean_static: cudaGetDevice: %s", cudaGetErrorString(err));
  if (device < 0 || device >= kMaxDevices)
    return fail(kUnsupported, "token_group_mean_static: device index %d is outside [0, %d)", device, kMaxDevices);
  std::lock_guard<std::mutex> lock(mutex);
  if (!per_device[device]) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_static_mean_scratch);
    if (err != cudaSuccess || !address)
      return fail(kCudaError, "token_group_mean_static: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
    per_device[device] = static_cast<float*>(address);
  }
  *out = per_device[device];
  return kOk;
}

}  // namespace

extern "C" int nob200_token_group_mean_static(int num_tokens, const void* input, void* output, int columns,
                                              int tokens_per_block, int include_padding, void* stream) {
  NOB_REQUIRE(num_tokens > 0 && columns > 0 && tokens_per_block > 0,
              "token_group_mean_static: sizes must be positive");
  NOB_REQUIRE(columns % 4 == 0, "token_group_mean_static: columns (%d) must be a multiple of 4", columns);
  NOB_REQUIRE(input && output, "token_group_mean_static: NULL tensor");
  const size_t need = nob200_token_group_mean_workspace_bytes(num_tokens, columns, tokens_per_block);
  NOB_REQUIRE(need <= static_cast<size_t>(NOB200_STATIC_MEAN_SCRATCH_BYTES),
              "token_group_mean_static: this shape needs %zu B of scratch but the built-in scratch holds %zu B; "
              "use nob200_token_group_mean with a caller-provided workspace",
              need, static_cast<size_t>(NOB200_STATIC_MEAN_SCRATCH_BYTES));
  const int groups = (num_tokens + tokens_per_block - 1) / tokens_per_block;
  const int chunks_per_group = (tokens_per_block + kMeanChunk - 1) / kMeanChunk;
  const long long total_chunks = static_cast<long long>(groups) * chunks_per_group;
  NOB_REQUIRE(total_chunks <= 65535, "token_group_mean_static: %lld chunks exceed the grid limit", total_chunks);
  float* scratch = nullptr;
  int rc = static_mean_scratch_ptr(&scratch);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int col_blocks = (columns / 4 + 127) / 128;
  if (chunks_per_group == 1) {
    mean_chunk_kernel<<<dim3(col_blocks, (unsigned)total_chunks), 128, 0, s>>>(
        static_cast<const __nv_bfloat16*>(input), static_cast<float*>(output), num_tokens, columns, tokens_per_block,
        1, include_padding, 1);
    return check_launch("token_group_mean_static");
  }
  // Every chunk sum that the second kernel reads is written by the first, so the
  // scratch needs no clearing although it still holds the previous call's sums.
  mean_chunk_kernel<<<dim3(col_blocks, (unsigned)total_chunks), 128, 0, s>>>(
      static_cast<const __nv_bfloat16*>(input), scratch, num_tokens, columns, tokens_per_block, chunks_per_group,
      include_padding, 0);
  rc = check_launch("token_group_mean_static(partial)");
  if (rc) return rc;
  mean_finish_kernel<<<dim3((columns + 31) / 32, groups), 256, 0, s>>>(
      scratch, static_cast<float*>(output), num_tokens, columns, tokens_per_block, chunks_per_group, include_padding);
  return check_launch("token_group_mean_static(finish)");
}

extern "C" int nob200_hadamard128_rows(long long num_rows, const void* input, void* output, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(num_rows > 0 && num_rows <= 0x7fffffffll, "hadamard128_rows: row count %lld out of range", num_rows);
  return nob200_hadamard128_heads(static_cast<int>(num_rows), 0, input, output, 1, 1, stream);
}

extern "C" int nob200_hadamard128_heads(int tokens, int head_offset, const void* input, void* output, int heads,
                                        int total_heads, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(tokens > 0 && heads > 0 && total_heads > 0, "hadamard128_heads: sizes must be positive");
  NOB_REQUIRE(head_offset >= 0 && head_offset <= total_heads - heads, "hadamard128_heads: head_offset %d outside [0, %d]",
              head_offset, total_heads - heads);
  NOB_REQUIRE(input && output, "hadamard128_heads: NULL tensor");
  const long long rows = static_cast<long long>(tokens) * heads;
  const long long ctas = (rows + 15) / 16;
  hadamard_rows_kernel<<<static_cast<unsigned>(ctas < 148 * 16 ? ctas : 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(input), static_cast<__nv_bfloat16*>(output), rows, heads, total_heads, head_offset);
  return check_launch("hadamard128_heads");
}
