// Per-head RMS norm and split-half RoPE of Q and K, alone (bf16 out) or fused into the int8 query quantiser.
// HBM-bound CUDA-core kernels: one pass over the projected activations instead of a bf16 round trip.
//
// Reference programs replaced here:
//   h3_head_norm_rope   src/nano_omni/kernels/specialized/h3_head_norm_rope.py:36-97
//   h3_query_prepare    src/nano_omni/kernels/specialized/h3_query_prepare.py:42-125
//
// For every (token, head) row x of 128 channels:
//   r = 1 / sqrt(sum(x^2) / 128 + 1e-5);  v = (x * r) * weight;
//   with RoPE, channels j < 48 and j + 48 form a pair rotated by (cos, sin)[token, j]:
//     out[j] = v[j] cos - v[j+48] sin,  out[j+48] = v[j] sin + v[j+48] cos;  channels 96..127 pass;
//   out is rounded to bf16 (stored, or quantised to int8 with one scale per head and 32 tokens).
// The reference leaves the order of the sum and the kind of reciprocal square root to its compiler (and its two
// ref_programs differ: mean of squares vs squared vector norm).  Here every step is an IEEE fp32 operation in a
// fixed order, which the CPU restatement repeats: a row lies on 16 lanes, 8 consecutive channels each; a lane adds
// its squares in channel order starting from 0, the 16 partial sums are combined by an xor butterfly with strides
// 8, 4, 2, 1; divide by 128, add 1e-5, square root, divide 1 by it; products and the sum or difference of the
// rotation are rounded one by one (no fused multiply-add).
#include "common.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

struct Row8 {
  float v[8];
};

__device__ __forceinline__ Row8 load_row8(const __nv_bfloat16* p) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  Row8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    r.v[2 * i] = __uint_as_float(w[i] << 16);
    r.v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
  return r;
}

__device__ __forceinline__ Row8 row8_of(const uint4& raw) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  Row8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    r.v[2 * i] = __uint_as_float(w[i] << 16);
    r.v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
  return r;
}

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// x[k]: 8 channels [8 lane16, 8 lane16 + 8) of row k; w: the norm weight of those channels.  On return x holds the
// normalised, rotated rows rounded to bf16 precision.  All 16 lanes of the rows' group must call it.  N rows go
// through each stage together so that their loads, shuffles and the divide / square root sequences overlap.
template <int N, int NW = 1>  // NW = 1: one weight for all rows; NW = N: a weight per row
__device__ __forceinline__ void norm_rope_rows(Row8 (&x)[N], const Row8 (&w)[NW], const float* __restrict__ cosines,
                                               const float* __restrict__ sines, const int (&token)[N], int lane16,
                                               bool use_rope) {
  // lanes 0-5 hold channels 0-47 (first), lanes 6-11 channels 48-95 (second), lanes 12-15 pass through
  const int partner = lane16 < 6 ? lane16 + 6 : lane16 - 6;
  const bool first = lane16 < 6, rotates = use_rope && lane16 < 12;
  float4 c[N][2], s[N][2];
  if (rotates) {
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const int at = token[k] * 48 + 8 * (first ? lane16 : lane16 - 6);
      c[k][0] = *reinterpret_cast<const float4*>(cosines + at);
      c[k][1] = *reinterpret_cast<const float4*>(cosines + at + 4);
      s[k][0] = *reinterpret_cast<const float4*>(sines + at);
      s[k][1] = *reinterpret_cast<const float4*>(sines + at + 4);
    }
  }
  float ss[N];
#pragma unroll
  for (int k = 0; k < N; ++k) {
    ss[k] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss[k] = __fadd_rn(ss[k], __fmul_rn(x[k].v[i], x[k].v[i]));
  }
#pragma unroll
  for (int m = 8; m > 0; m >>= 1) {
#pragma unroll
    for (int k = 0; k < N; ++k) ss[k] = __fadd_rn(ss[k], __shfl_xor_sync(0xffffffffu, ss[k], m));
  }
#pragma unroll
  for (int k = 0; k < N; ++k) {
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss[k], 0.0078125f), 1e-5f)));
#pragma unroll
    for (int i = 0; i < 8; ++i) x[k].v[i] = __fmul_rn(__fmul_rn(x[k].v[i], r), w[NW == 1 ? 0 : k].v[i]);
  }
  if (use_rope) {
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const float cc[8] = {c[k][0].x, c[k][0].y, c[k][0].z, c[k][0].w, c[k][1].x, c[k][1].y, c[k][1].z, c[k][1].w};
      const float sn[8] = {s[k][0].x, s[k][0].y, s[k][0].z, s[k][0].w, s[k][1].x, s[k][1].y, s[k][1].z, s[k][1].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float other = __shfl_sync(0xffffffffu, x[k].v[i], partner & 15, 16);
        if (rotates) {
          x[k].v[i] = first ? __fsub_rn(__fmul_rn(x[k].v[i], cc[i]), __fmul_rn(other, sn[i]))
                            : __fadd_rn(__fmul_rn(other, sn[i]), __fmul_rn(x[k].v[i], cc[i]));
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < N; ++k) {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[k].v[i] = round_bf16(x[k].v[i]);
  }
}

__device__ __forceinline__ uint32_t pack_bf16_pair(float lo, float hi) {
  return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xffff0000u);  // both already bf16-representable
}

// One group of 16 lanes per (token, head) row: 16 rows per CTA round (more rows per group cost occupancy and were
// measured slower).  In place is allowed.
__global__ void __launch_bounds__(256)
head_norm_rope_kernel(const __nv_bfloat16* src, const __nv_bfloat16* __restrict__ weight,
                      const float* __restrict__ cosines, const float* __restrict__ sines, __nv_bfloat16* dst,
                      long long rows, int heads, int use_rope) {  // src and dst may be the same tensor
  constexpr int kRows = 1;
  const int lane16 = threadIdx.x & 15;
  const Row8 w[1] = {load_row8(weight + 8 * lane16)};
  const long long stride = static_cast<long long>(gridDim.x) * (16 * kRows);
  // every lane of a warp runs the same number of rounds (the shuffles need all of them).  The piece of the next
  // round is loaded before this round's shuffles, which the compiler would not move a load across: two rows of a
  // thread are in flight instead of one.  (In place: the next round's rows are other rows than this round's.)
  auto piece_at = [&](long long base) {
    const long long row = base + (threadIdx.x >> 4);
    return *reinterpret_cast<const uint4*>(src + (row < rows ? row : 0) * 128 + 8 * lane16);
  };
  const long long first_base = static_cast<long long>(blockIdx.x) * 16;
  uint4 next_piece = first_base < rows ? piece_at(first_base) : make_uint4(0u, 0u, 0u, 0u);
  for (long long base = first_base; base < rows; base += stride) {
    Row8 x[kRows];
    int token[kRows];
    long long at[kRows];
    bool live[kRows];
    const uint4 piece = next_piece;
    if (base + stride < rows) next_piece = piece_at(base + stride);
#pragma unroll
    for (int k = 0; k < kRows; ++k) {
      const long long row = base + 16 * k + (threadIdx.x >> 4);
      live[k] = row < rows;
      at[k] = (live[k] ? row : 0) * 128 + 8 * lane16;
      token[k] = static_cast<int>((live[k] ? row : 0) / heads);
      x[k] = row8_of(piece);
    }
    norm_rope_rows<kRows>(x, w, cosines, sines, token, lane16, use_rope != 0);
#pragma unroll
    for (int k = 0; k < kRows; ++k) {
      if (live[k]) {
        uint4 out;
        out.x = pack_bf16_pair(x[k].v[0], x[k].v[1]);
        out.y = pack_bf16_pair(x[k].v[2], x[k].v[3]);
        out.z = pack_bf16_pair(x[k].v[4], x[k].v[5]);
        out.w = pack_bf16_pair(x[k].v[6], x[k].v[7]);
        *reinterpret_cast<uint4*>(dst + at[k]) = out;
      }
    }
  }
}

// Q and K of the same (token, head) in one launch, in place: a 16-lane group takes the query row and the key row
// together, so their loads are in flight at once and both use one read of the RoPE table entries.
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(__nv_bfloat16* query, __nv_bfloat16* key, const __nv_bfloat16* __restrict__ query_weight,
                    const __nv_bfloat16* __restrict__ key_weight, const float* __restrict__ cosines,
                    const float* __restrict__ sines, long long rows, int heads) {
  const int lane16 = threadIdx.x & 15;
  const Row8 w[2] = {load_row8(query_weight + 8 * lane16), load_row8(key_weight + 8 * lane16)};
  const long long stride = static_cast<long long>(gridDim.x) * 16;
  // every lane of a warp runs the same number of rounds (the shuffles need all of them)
  // the pieces of the next round are loaded before this round's shuffles (see head_norm_rope_kernel)
  auto offset_at = [&](long long base) {
    const long long row = base + (threadIdx.x >> 4);
    return (row < rows ? row : 0) * 128 + 8 * lane16;
  };
  const long long first_base = static_cast<long long>(blockIdx.x) * 16;
  uint4 next_q = make_uint4(0u, 0u, 0u, 0u), next_k = next_q;
  if (first_base < rows) {
    next_q = *reinterpret_cast<const uint4*>(query + offset_at(first_base));
    next_k = *reinterpret_cast<const uint4*>(key + offset_at(first_base));
  }
  for (long long base = first_base; base < rows; base += stride) {
    const long long row = base + (threadIdx.x >> 4);
    const bool live = row < rows;
    const long long at = (live ? row : 0) * 128 + 8 * lane16;
    Row8 x[2] = {row8_of(next_q), row8_of(next_k)};
    if (base + stride < rows) {
      next_q = *reinterpret_cast<const uint4*>(query + offset_at(base + stride));
      next_k = *reinterpret_cast<const uint4*>(key + offset_at(base + stride));
    }
    const int tok = static_cast<int>((live ? row : 0) / heads);
    const int token[2] = {tok, tok};
    norm_rope_rows<2, 2>(x, w, cosines, sines, token, lane16, true);
    if (live) {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        uint4 out;
        out.x = pack_bf16_pair(x[k].v[0], x[k].v[1]);
        out.y = pack_bf16_pair(x[k].v[2], x[k].v[3]);
        out.z = pack_bf16_pair(x[k].v[4], x[k].v[5]);
        out.w = pack_bf16_pair(x[k].v[6], x[k].v[7]);
        *reinterpret_cast<uint4*>((k ? key : query) + at) = out;
      }
    }
  }
}

// One CTA per (32-token group, head): 128 threads, 8 rows per pass, 4 passes.
__global__ void __launch_bounds__(128)
query_prepare_kernel(const __nv_bfloat16* __restrict__ src, const __nv_bfloat16* __restrict__ weight,
                     const float* __restrict__ cosines, const float* __restrict__ sines,
                     int8_t* __restrict__ quantized, float* __restrict__ scales, int tokens, int heads, int groups,
                     int use_rope) {
  const int head = blockIdx.x, group = blockIdx.y;  // heads fastest: CTAs in flight read whole rows of the source
  const int lane16 = threadIdx.x & 15, row_in_pass = threadIdx.x >> 4;
  const Row8 w[1] = {load_row8(weight + 8 * lane16)};
  const size_t columns = static_cast<size_t>(heads) * 128;
  Row8 x[4];
  float amax = 0.f;
  uint4 loaded[4];  // the four rows' loads are in flight together; the shuffles below would keep them apart
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int t = group * 32 + p * 8 + row_in_pass;
    loaded[p] = __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(t < tokens ? t : 0) * columns + head * 128 +
                                                     8 * lane16));
  }
  // kTogether rows go through the norm and the rotation together.  One at a time is fastest (175 us at 32768 tokens x
  // 24 heads; two 211, four 246: the registers of the extra rows cost more occupancy than the overlap gains).
  constexpr int kTogether = 1;
#pragma unroll
  for (int p0 = 0; p0 < 4; p0 += kTogether) {
    int token[kTogether];
    bool live[kTogether];
    Row8 rows_now[kTogether];
#pragma unroll
    for (int k = 0; k < kTogether; ++k) {
      const int t = group * 32 + (p0 + k) * 8 + row_in_pass;
      live[k] = t < tokens;
      token[k] = live[k] ? t : 0;
      rows_now[k] = row8_of(loaded[p0 + k]);
    }
    norm_rope_rows<kTogether>(rows_now, w, cosines, sines, token, lane16, use_rope != 0);
#pragma unroll
    for (int k = 0; k < kTogether; ++k) {
      x[p0 + k] = rows_now[k];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (!live[k]) x[p0 + k].v[i] = 0.f;  // rows past the end quantise to zero and do not count in the maximum
        amax = fmaxf(amax, fabsf(x[p0 + k].v[i]));
      }
    }
  }
  __shared__ float warp_max[4];
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(warp_max[0], warp_max[1]), fmaxf(warp_max[2], warp_max[3]));
  const float scale = fmaxf(amax / 127.0f, 1e-10f);
  const float inv_scale = __frcp_rn(scale);
  if (threadIdx.x == 0) scales[static_cast<size_t>(head) * groups + group] = scale;
  int8_t* dst_base = quantized + (static_cast<size_t>(head) * groups + group) * 32 * 128;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int r = p * 8 + row_in_pass;
    uint32_t word[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // rint(RN(x / scale)): the product with RN(1/scale) rounds to the same integer unless it lies within 4e-5
      // of a half-integer; only then the IEEE division is done (as in the int8 Q/K quantiser).
      float a = x[p].v[i] * inv_scale;
      float q = rintf(a);
      if (0.5f - fabsf(a - q) < 4e-5f) q = rintf(__fdiv_rn(x[p].v[i], scale));
      q = fminf(fmaxf(q, -128.f), 127.f);
      word[i >> 2] |= (static_cast<uint32_t>(static_cast<int>(q)) & 0xffu) << (8 * (i & 3));
    }
    *reinterpret_cast<uint2*>(dst_base + r * 128 + lane16 * 8) = make_uint2(word[0], word[1]);
  }
}

}  // namespace
}  // namespace nob200

extern "C" int nob200_h3_head_norm_rope(int tokens, const void* input, const void* weight, const void* cosines,
                                        const void* sines, void* output, int heads, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(tokens > 0 && heads > 0, "h3_head_norm_rope: sizes must be positive");
  NOB_REQUIRE(input && weight && output, "h3_head_norm_rope: NULL tensor");
  NOB_REQUIRE((cosines == nullptr) == (sines == nullptr), "h3_head_norm_rope: cosines and sines come together");
  const long long rows = static_cast<long long>(tokens) * heads;
  const long long ctas = (rows + 15) / 16;
  const unsigned grid = static_cast<unsigned>(ctas < 148 * 16 ? ctas : 148 * 16);
  head_norm_rope_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(input), static_cast<const __nv_bfloat16*>(weight),
      static_cast<const float*>(cosines), static_cast<const float*>(sines), static_cast<__nv_bfloat16*>(output), rows,
      heads, cosines != nullptr);
  return check_launch("h3_head_norm_rope");
}

extern "C" int nob200_h3_qk_norm_rope(int tokens, void* query, void* key, const void* query_weight,
                                      const void* key_weight, const void* cosines, const void* sines, int heads,
                                      void* stream) {
  using namespace nob200;
  NOB_REQUIRE(tokens > 0 && heads > 0, "h3_qk_norm_rope: sizes must be positive");
  NOB_REQUIRE(query && key && query_weight && key_weight && cosines && sines, "h3_qk_norm_rope: NULL tensor");
  const long long rows = static_cast<long long>(tokens) * heads;
  const long long ctas = (rows + 15) / 16;
  const unsigned grid = static_cast<unsigned>(ctas < 148 * 16 ? ctas : 148 * 16);
  qk_norm_rope_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(query), static_cast<__nv_bfloat16*>(key),
      static_cast<const __nv_bfloat16*>(query_weight), static_cast<const __nv_bfloat16*>(key_weight),
      static_cast<const float*>(cosines), static_cast<const float*>(sines), rows, heads);
  return check_launch("h3_qk_norm_rope");
}

extern "C" int nob200_h3_query_prepare(int tokens, const void* source, const void* weight, const void* cosines,
                                       const void* sines, void* quantized, void* scales, int heads, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(tokens > 0 && heads > 0, "h3_query_prepare: sizes must be positive");
  NOB_REQUIRE(source && weight && quantized && scales, "h3_query_prepare: NULL tensor");
  NOB_REQUIRE((cosines == nullptr) == (sines == nullptr), "h3_query_prepare: cosines and sines come together");
  const int groups = (tokens + 31) / 32;
  NOB_REQUIRE(groups <= 65535, "h3_query_prepare: %d token groups exceed the grid limit", groups);
  query_prepare_kernel<<<dim3(heads, groups), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(source), static_cast<const __nv_bfloat16*>(weight),
      static_cast<const float*>(cosines), static_cast<const float*>(sines), static_cast<int8_t*>(quantized),
      static_cast<float*>(scales), tokens, heads, groups, cosines != nullptr);
  return check_launch("h3_query_prepare");
}

// ------------------------------------------------- row-wise int8 of the projection inputs, with group rotation
// Replaces int8_rowwise (src/nano_omni/kernels/quantization/int8_rowwise.py:107-116) and convrot_int8
// (src/nano_omni/kernels/quantization/convrot_int8.py:130-161): optionally rotate every group of 256 columns by
// B (x) B (x) B (x) B / 16 with B = [[1,1,1,-1],[1,1,-1,1],[1,-1,1,1],[-1,1,1,1]], round to bf16, then one scale per
// row, max(amax / 127, 1e-30), and round-half-even to int8 in [-127, 127].
// The reference multiplies by the 256 x 256 matrix and leaves the summation order to the GEMM; here the rotation is
// four radix-4 stages over the base-4 digits of the column index, lowest digit first, each stage computing from
// (a, b, c, d) = the values at digit 0..3:  p = a + b, q = a - b, r = c + d, u = c - d;  y0 = p + u, y1 = p - u,
// y2 = q + r, y3 = r - q  (every operation rounded to fp32); the CPU restatement repeats that.
namespace nob200 {
namespace {

__device__ __forceinline__ void radix4(float& a, float& b, float& c, float& d) {
  const float p = __fadd_rn(a, b), q = __fsub_rn(a, b), r = __fadd_rn(c, d), u = __fsub_rn(c, d);
  a = __fadd_rn(p, u);
  b = __fsub_rn(p, u);
  c = __fadd_rn(q, r);
  d = __fsub_rn(r, q);
}

// One CTA per row; a group of 256 columns lies on 16 lanes with 16 consecutive columns each.
__global__ void __launch_bounds__(128)
rowwise_int8_kernel(const __nv_bfloat16* __restrict__ src, int8_t* __restrict__ dst, float* __restrict__ scales,
                    int columns, int rotate) {
  extern __shared__ __nv_bfloat16 rotated[];  // the row after rotation and bf16 rounding
  __shared__ float warp_max[4];
  __shared__ float transpose[8][16 * 17];  // one 256-column group per half-warp
  const size_t row = blockIdx.x;
  const int lane16 = threadIdx.x & 15, half_warp = threadIdx.x >> 4;
  const __nv_bfloat16* in = src + row * columns;
  float amax = 0.f;
  // both half-warps of a warp run every round (the warp synchronises around the transpose); a half-warp past the
  // last group works on group 0 again and discards the result
  const int groups = columns / 256;
  for (int first = 0; first < groups; first += 8) {
    const bool live = first + half_warp < groups;
    const int g = live ? first + half_warp : 0;
    float x[16];
    const Row8 lo = load_row8(in + g * 256 + 16 * lane16), hi = load_row8(in + g * 256 + 16 * lane16 + 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = lo.v[i], x[8 + i] = hi.v[i];
    if (rotate) {
#pragma unroll
      for (int i = 0; i < 16; i += 4) radix4(x[i], x[i + 1], x[i + 2], x[i + 3]);  // digit 0: column stride 1
#pragma unroll
      for (int i = 0; i < 4; ++i) radix4(x[i], x[i + 4], x[i + 8], x[i + 12]);  // digit 1: column stride 4
      // digits 2 and 3 (column strides 16 and 64) lie across the lanes: transpose through shared memory so that a
      // lane holds columns lane16 + 16 r, r = 0..15, and they become register digits too (rows padded to 17 words)
      float* scratch = transpose[half_warp];
#pragma unroll
      for (int i = 0; i < 16; ++i) scratch[17 * lane16 + i] = x[i];
      __syncwarp();
#pragma unroll
      for (int r = 0; r < 16; ++r) x[r] = scratch[17 * r + lane16];
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 16; i += 4) radix4(x[i], x[i + 1], x[i + 2], x[i + 3]);  // digit 2
#pragma unroll
      for (int i = 0; i < 4; ++i) radix4(x[i], x[i + 4], x[i + 8], x[i + 12]);  // digit 3
#pragma unroll
      for (int i = 0; i < 16; ++i) x[i] = round_bf16(__fmul_rn(x[i], 0.0625f));
      if (live) {
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          amax = fmaxf(amax, fabsf(x[r]));
          rotated[g * 256 + lane16 + 16 * r] = __float2bfloat16_rn(x[r]);  // exact: already bf16-representable
        }
      }
    } else if (live) {
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        amax = fmaxf(amax, fmaxf(fabsf(x[2 * i]), fabsf(x[2 * i + 1])));
        w[i] = pack_bf16_pair(x[2 * i], x[2 * i + 1]);
      }
      uint4* out = reinterpret_cast<uint4*>(rotated + g * 256 + 16 * lane16);
      out[0] = make_uint4(w[0], w[1], w[2], w[3]);
      out[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  }
  // columns beyond the last whole group (row-wise form only; a multiple of 8)
  for (int c = groups * 256 + 8 * threadIdx.x; c < columns; c += 8 * 128) {
    const Row8 v = load_row8(in + c);
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      amax = fmaxf(amax, fmaxf(fabsf(v.v[2 * i]), fabsf(v.v[2 * i + 1])));
      w[i] = pack_bf16_pair(v.v[2 * i], v.v[2 * i + 1]);
    }
    *reinterpret_cast<uint4*>(rotated + c) = make_uint4(w[0], w[1], w[2], w[3]);
  }
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(warp_max[0], warp_max[1]), fmaxf(warp_max[2], warp_max[3]));
  const float scale = fmaxf(amax / 127.0f, 1e-30f);
  const float inv_scale = __frcp_rn(scale);
  if (threadIdx.x == 0) scales[row] = scale;
  int8_t* out = dst + row * columns;
  for (int c = 8 * threadIdx.x; c < columns; c += 8 * 128) {
    const Row8 v = load_row8(rotated + c);
    uint32_t word[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // rint(RN(x / scale)) as in the other int8 quantisers: exact division only near a rounding boundary
      float a = v.v[i] * inv_scale;
      float q = rintf(a);
      if (!(0.5f - fabsf(a - q) >= 4e-5f)) q = rintf(__fdiv_rn(v.v[i], scale));
      q = fminf(fmaxf(q, -127.f), 127.f);
      word[i >> 2] |= (static_cast<uint32_t>(static_cast<int>(q)) & 0xffu) << (8 * (i & 3));
    }
    *reinterpret_cast<uint2*>(out + c) = make_uint2(word[0], word[1]);
  }
}

}  // namespace
}  // namespace nob200

extern "C" int nob200_int8_rowwise(int num_tokens, const void* input, void* output, void* scales, int columns,
                                   int rotation_group, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(num_tokens > 0 && columns > 0, "int8_rowwise: sizes must be positive");
  NOB_REQUIRE(input && output && scales, "int8_rowwise: NULL tensor");
  NOB_REQUIRE(rotation_group == 0 || rotation_group == 256, "int8_rowwise: rotation group must be 0 (none) or 256 (got %d)",
              rotation_group);
  NOB_REQUIRE(columns % 8 == 0 && (rotation_group == 0 || columns % 256 == 0),
              "int8_rowwise: columns (%d) must be a multiple of 8, and of the rotation group", columns);
  NOB_REQUIRE(columns <= 65536, "int8_rowwise: at most 65536 columns (the row is staged in shared memory)");
  const size_t smem = static_cast<size_t>(columns) * 2;
  if (smem + 9 * 1024 > 48 * 1024) {  // the kernel also holds 8.5 KiB of static shared memory (the transpose)
    cudaError_t err = cudaFuncSetAttribute(rowwise_int8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess)
      return fail(kCudaError, "int8_rowwise: cannot reserve %zu B of shared memory: %s", smem, cudaGetErrorString(err));
  }
  rowwise_int8_kernel<<<num_tokens, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(input), static_cast<int8_t*>(output), static_cast<float*>(scales), columns,
      rotation_group == 256);
  return check_launch("int8_rowwise");
}
