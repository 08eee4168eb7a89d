// Dense non-causal bf16 attention forward for head_dim 128 on sm_100a.
//
// Replaces the reference program dense_bf16_attention
// (src/nano_omni/kernels/attention/dense_bf16.py:46-195): O = softmax(Q K^T / sqrt(128)) V with
// fp32 online softmax in the exp2 domain, Q/K/V bf16 [tokens, heads, 128], O bf16
// [tokens, total_heads, 128] written at head_offset.
//
// One CTA owns 256 query rows of one head (two 128-row tiles, "A" and "B") and
// walks the keys in tiles of 128:
//   warp 8      TMA producer: Q once, then K_j / V_j alternately into a 4-stage ring
//   warp 9      tcgen05 issuer: S_t = Q_t K_j^T (SS form, fp32 in TMEM), O_t += P_t V_j
//               (P read from TMEM, V consumed N-major straight from the TMA tile); the PV
//               MMAs of a tile start when the first 64 keys of P are written
//   warps 0-3   softmax for tile A: one thread per row, S row -> registers, row maximum with
//               3-input max, exp2 on packed fp32 pairs, bf16 P written back over S in TMEM
//   warps 4-7   the same for tile B, so one tile's softmax overlaps the other's MMAs
// TMEM columns: S_A 0-127, S_B 128-255, O_A 256-383, O_B 384-511 (P_t aliases S_t).
// The running maximum is only raised when a row's maximum grew by more than 2^8
// (then O and the row sum are rescaled in place); it is exact for the first tile.
#include <cuda.h>

#include "common.cuh"
#include "fa_common.cuh"
#include "tensor_map.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

constexpr int kTile = 128;                     // query rows per tile and keys per tile
constexpr int kHalfBytes = kTile * 64 * 2;     // one 64-channel half of a tile (128B rows)
constexpr int kTileBytes = 2 * kHalfBytes;     // 32 KiB
constexpr int kStages = 4;
constexpr int kThreads = 384;                 // warpgroups: softmax A, softmax B, {TMA, MMA, 2 idle}
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;      // log2 units

struct __align__(1024) Shared {
  uint8_t q[2][kTileBytes];
  uint8_t kv[kStages][kTileBytes];
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];
  uint64_t p_full[2][2];
  uint64_t o_final[2];
  uint32_t tmem_base;
  uint32_t abort;
};

// POLY: of every 4 pairs of probabilities, how many are exponentiated on the FMA pipe
// instead of the MUFU.  SPLIT: hand P to the PV MMA in two halves of 64 keys.
template <int POLY, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
fa_fwd_bf16_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const OutRoute out, int num_tokens,
                   int total_heads, int head_offset, float scale_log2, uint32_t* status,
                   __nv_bfloat16* __restrict__ partial_out, float* __restrict__ partial_lse) {
  extern __shared__ uint8_t smem_raw[];
  Shared& S = *reinterpret_cast<Shared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int q0 = blockIdx.x * (2 * kTile);
  const bool two = q0 + kTile < num_tokens;  // second tile holds at least one row
  // gridDim.z > 1: this CTA covers only a contiguous share of the key tiles and writes a normalised
  // partial result with its log-sum-exp; a second kernel merges the shares.
  const int n_kv_total = (num_tokens + kTile - 1) / kTile;
  const int kv_begin = static_cast<int>(static_cast<long long>(n_kv_total) * blockIdx.z / gridDim.z);
  const int kv_end = static_cast<int>(static_cast<long long>(n_kv_total) * (blockIdx.z + 1) / gridDim.z);
  const int n_kv = kv_end - kv_begin;
  volatile uint32_t* abort_flag = &S.abort;

  if (threadIdx.x == 0) {
    mbar_init(&S.q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&S.kv_full[s], 1);
      mbar_init(&S.kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&S.s_full[t], 1);
      mbar_init(&S.p_full[t][0], 4);
      mbar_init(&S.p_full[t][1], 4);
      mbar_init(&S.o_final[t], 1);
    }
    S.abort = 0;
    mbar_fence_init();
  }
  if (warp == kProducerWarp) {
    tmem_alloc(&S.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = S.tmem_base;

  if (warp >= 8) {
   reg_dealloc<56>();
   if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_expect_tx(&S.q_full, two ? 2 * kTileBytes : kTileBytes);
      tma_load_3d(S.q[0], &map_q, &S.q_full, 0, head, q0);
      tma_load_3d(S.q[0] + kHalfBytes, &map_q, &S.q_full, 64, head, q0);
      if (two) {
        tma_load_3d(S.q[1], &map_q, &S.q_full, 0, head, q0 + kTile);
        tma_load_3d(S.q[1] + kHalfBytes, &map_q, &S.q_full, 64, head, q0 + kTile);
      }
      const int loads = 2 * n_kv;
      int issued = 0;
      for (int i = 0; i < loads; ++i) {
        const int st = i % kStages;
        if (i >= kStages) {
          if (!mbar_wait(&S.kv_empty[st], ((i / kStages) - 1) & 1, abort_flag, status, kWaitTimeoutRing)) break;
        }
        mbar_expect_tx(&S.kv_full[st], kTileBytes);
        const CUtensorMap* map = (i & 1) ? &map_v : &map_k;
        const int tok = (kv_begin + (i >> 1)) * kTile;
        tma_load_3d(S.kv[st], map, &S.kv_full[st], 0, head, tok);
        tma_load_3d(S.kv[st] + kHalfBytes, map, &S.kv_full[st], 64, head, tok);
        issued = i + 1;
      }
      if (*abort_flag) {
        // Gave up: let the copies already in flight land before the CTA exits.
        for (int i = (issued > kStages ? issued - kStages : 0); i < issued; ++i) {
          uint64_t* bar = &S.kv_full[i % kStages];
          const uint32_t parity = (i / kStages) & 1;
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(bar, parity); ++spin) {
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------- tcgen05 issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(kDF32, kFmtBF16, kFmtBF16, 0, 0, kTile, kTile);
      constexpr uint32_t idesc_pv = umma_idesc(kDF32, kFmtBF16, kFmtBF16, 0, 1, kTile, 128);
      // Descriptors are kept as (low word, high word): the tile address lives in the low 14 bits of
      // the low word, so stepping through a tile is one 32-bit add and the issuing thread spends
      // only a handful of instructions per MMA (it must stay well under the MMA's 64 cycles).
      const uint64_t desc_k_major = umma_smem_desc(0, 16, 1024, kSwizzle128B);
      const uint64_t desc_n_major = umma_smem_desc(0, kHalfBytes, 1024, kSwizzle128B);
      const uint32_t hi_k = static_cast<uint32_t>(desc_k_major >> 32), hi_n = static_cast<uint32_t>(desc_n_major >> 32);
      const uint32_t lo_k = static_cast<uint32_t>(desc_k_major), lo_n = static_cast<uint32_t>(desc_n_major);
      const uint32_t q_lo[2] = {lo_k + (smem_u32(S.q[0]) >> 4), lo_k + (smem_u32(S.q[1]) >> 4)};
      const uint32_t kv_k_lo = lo_k + (smem_u32(S.kv[0]) >> 4);  // + stage * (kTileBytes >> 4)
      const uint32_t kv_n_lo = lo_n + (smem_u32(S.kv[0]) >> 4);
      auto mma_ss = [&](uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t acc) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
            "setp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d),
            "r"(a_lo), "r"(hi_k), "r"(b_lo), "r"(hi_k), "r"(idesc_qk), "r"(acc)
            : "memory");
      };
      auto mma_ts = [&](uint32_t d, uint32_t a_tmem, uint32_t b_lo, uint32_t acc) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
            "mov.b64 db, {%2, %3};\n\t"
            "setp.ne.b32 p, %5, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d),
            "r"(a_tmem), "r"(b_lo), "r"(hi_n), "r"(idesc_pv), "r"(acc)
            : "memory");
      };
      auto issue_qk = [&](int t, int st) {
        const uint32_t a = q_lo[t], b = kv_k_lo + st * (kTileBytes >> 4), d = tmem + t * kTile;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 channels = 32 bytes inside a 64-channel half; halves are kHalfBytes apart
          const uint32_t off = ((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4;
          mma_ss(d, a + off, b + off, kk > 0);
        }
      };
      auto issue_pv = [&](int t, int st, bool accumulate, int k_begin, int k_end) {
        const uint32_t b = kv_n_lo + st * (kTileBytes >> 4), d = tmem + 256 + t * kTile, a = tmem + t * kTile;
#pragma unroll
        for (int kk = k_begin; kk < k_end; ++kk) {
          // 16 keys = 16 rows of 128 B = 2048 B; P holds two keys per 32-bit column
          mma_ts(d, a + kk * 8, b + kk * (2048 >> 4), (accumulate || kk > 0) ? 1u : 0u);
        }
      };
      auto full_parity = [](int i) { return (uint32_t)((i / kStages) & 1); };

      bool ok = mbar_wait(&S.q_full, 0, abort_flag, status, kWaitTimeoutLoad);
      ok = ok && mbar_wait(&S.kv_full[0], 0, abort_flag, status, kWaitTimeoutLoad);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        tc_commit(&S.s_full[0]);
        if (two) {
          issue_qk(1, 0);
          tc_commit(&S.s_full[1]);
        }
        tc_commit(&S.kv_empty[0]);
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const int iv = 2 * j + 1, ik = 2 * j + 2;
        const int sv = iv % kStages, sk = ik % kStages;
        const bool more = j + 1 < n_kv;
        if (!(ok = mbar_wait(&S.kv_full[sv], full_parity(iv), abort_flag, status, kWaitTimeoutLoad))) break;
        if (!(ok = mbar_wait(&S.p_full[0][0], j & 1, abort_flag, status, kWaitTimeoutSoftmax))) break;
        tc_fence_after();
        if (SPLIT) {
          issue_pv(0, sv, j > 0, 0, 4);
          if (!(ok = mbar_wait(&S.p_full[0][1], j & 1, abort_flag, status, kWaitTimeoutSoftmax))) break;
          tc_fence_after();
          issue_pv(0, sv, j > 0, 4, 8);
        } else {
          issue_pv(0, sv, j > 0, 0, 8);
        }
        if (more) {
          if (!(ok = mbar_wait(&S.kv_full[sk], full_parity(ik), abort_flag, status, kWaitTimeoutLoad))) break;
          tc_fence_after();
          issue_qk(0, sk);
          tc_commit(&S.s_full[0]);
        }
        if (two) {
          if (!(ok = mbar_wait(&S.p_full[1][0], j & 1, abort_flag, status, kWaitTimeoutSoftmax))) break;
          tc_fence_after();
          if (SPLIT) {
            issue_pv(1, sv, j > 0, 0, 4);
            if (!(ok = mbar_wait(&S.p_full[1][1], j & 1, abort_flag, status, kWaitTimeoutSoftmax))) break;
            tc_fence_after();
            issue_pv(1, sv, j > 0, 4, 8);
          } else {
            issue_pv(1, sv, j > 0, 0, 8);
          }
        }
        tc_commit(&S.kv_empty[sv]);
        if (more) {
          if (two) {
            issue_qk(1, sk);
            tc_commit(&S.s_full[1]);
          }
          tc_commit(&S.kv_empty[sk]);
        }
      }
      if (ok) {
        tc_commit(&S.o_final[0]);
        if (two) tc_commit(&S.o_final[1]);
      }
    }
   }
  } else {
    // ------------------------------------------------- softmax + epilogue warps
    reg_alloc<224>();
    const int t = warp >> 2;
    if (t == 0 || two) {
      const int row = (warp & 3) * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t s_addr = tmem + lane_base + t * kTile;
      const uint32_t o_addr = tmem + lane_base + 256 + t * kTile;
      float m_used = 0.f;
      uint64_t la = 0ull, lb = 0ull;  // four partial row sums as two fp32 pairs
      bool ok = true;
      for (int j = 0; j < n_kv; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(&S.s_full[t], j & 1, abort_flag, status, kWaitTimeoutMma));
        if (!ok) break;
        tc_fence_after();
        uint32_t s[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&s[32 * c]));
        tc_wait_ld();
        if (kv_begin + j == n_kv_total - 1) {
          const int valid = num_tokens - (kv_begin + j) * kTile;
          if (valid < kTile) {
#pragma unroll
            for (int i = 0; i < 128; ++i)
              if (i >= valid) s[i] = 0xff800000u;  // -inf
          }
        }
        float mx0 = __uint_as_float(s[0]), mx1 = __uint_as_float(s[1]);
#pragma unroll
        for (int i = 2; i < 126; i += 4) {
          mx0 = max3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
          mx1 = max3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        }
        mx0 = max3(mx0, __uint_as_float(s[126]), __uint_as_float(s[127]));
        const float mx = fmaxf(mx0, mx1) * scale_log2;
        if (j == 0) {
          m_used = mx;
        } else if (__any_sync(0xffffffffu, mx > m_used + kRescaleThreshold)) {
          const float m_new = fmaxf(m_used, mx);
          const float alpha = ex2(m_used - m_new);
          const uint64_t alpha2 = pack2(alpha, alpha);
          la = fma2(la, alpha2, 0ull);
          lb = fma2(lb, alpha2, 0ull);
          // S_t(j) is complete, hence so is O_t += P_t V_{j-1}; the next PV waits for our arrival.
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(o_addr + 32 * c, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_addr + 32 * c, o);
          }
          tc_wait_st();
          m_used = m_new;
        }
        const uint64_t scale2 = pack2(scale_log2, scale_log2);
        const uint64_t neg_m2 = pack2(-m_used, -m_used);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t p[32];
#pragma unroll
          for (int i = 0; i < 64; i += 4) {
            const int e = half * 64 + i;
            const uint64_t xa = fma2(pack2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), scale2, neg_m2);
            const uint64_t xb = fma2(pack2(__uint_as_float(s[e + 2]), __uint_as_float(s[e + 3])), scale2, neg_m2);
            float a, b, c, d;
            // pairs are numbered e/2; pair k uses the FMA-pipe exponential when k % 4 < POLY
            if (((e / 2) & 3) < POLY) {
              exp2_poly_pair(xa, a, b);
            } else {
              float x0, x1;
              unpack2(xa, x0, x1);
              a = ex2(x0), b = ex2(x1);
            }
            if (((e / 2 + 1) & 3) < POLY) {
              exp2_poly_pair(xb, c, d);
            } else {
              float x0, x1;
              unpack2(xb, x0, x1);
              c = ex2(x0), d = ex2(x1);
            }
            la = add2(la, pack2(a, b));
            lb = add2(lb, pack2(c, d));
            p[i / 2] = pack_bf16(a, b);
            p[i / 2 + 1] = pack_bf16(c, d);
          }
          tmem_st32(s_addr + 32 * half, p);
          if (SPLIT || half == 1) {
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&S.p_full[t][SPLIT ? half : 0]);
          }
        }
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&S.o_final[t], 0, abort_flag, status, kWaitTimeoutMma));
      if (ok) {
        tc_fence_after();
        float l0, l1, l2, l3;
        unpack2(la, l0, l1);
        unpack2(lb, l2, l3);
        const float l = (l0 + l1) + (l2 + l3);
        const float inv = 1.0f / l;
        const int token = q0 + t * kTile + row;
        __nv_bfloat16* dst = out.row(token < num_tokens ? token : 0, total_heads, head + head_offset);
        if (gridDim.z > 1) {
          const size_t at = (static_cast<size_t>(blockIdx.z) * num_tokens + token) * gridDim.y + head;
          dst = partial_out + at * 128;
          if (token < num_tokens) partial_lse[at] = m_used + log2f(l);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + 32 * c, o);
          tc_wait_ld();
          if (token < num_tokens) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
              v.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              v.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              v.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + 32 * c + i) = v;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem, kTmemCols);
}

// Merge of split-KV shares: out = sum_z w_z * partial_z with w_z = 2^(lse_z - max lse) / sum of those.
__global__ void __launch_bounds__(256)
fa_merge_splits_kernel(const __nv_bfloat16* __restrict__ partial_out, const float* __restrict__ partial_lse,
                       const OutRoute out, int num_tokens, int heads, int total_heads, int head_offset,
                       int splits) {
  const long long item = blockIdx.x * 256ll + threadIdx.x;  // (token, head, 8-channel piece)
  const long long total = static_cast<long long>(num_tokens) * heads * 16;
  if (item >= total) return;
  const int piece = static_cast<int>(item & 15);
  const long long th = item >> 4;  // token * heads + head
  const int head = static_cast<int>(th % heads);
  const long long token = th / heads;
  const size_t share = static_cast<size_t>(num_tokens) * heads;
  float mx = -INFINITY;
  for (int z = 0; z < splits; ++z) mx = fmaxf(mx, partial_lse[z * share + th]);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float wsum = 0.f;
  for (int z = 0; z < splits; ++z) {
    const float w = exp2f(partial_lse[z * share + th] - mx);
    wsum += w;
    const uint4 raw = *reinterpret_cast<const uint4*>(partial_out + (z * share + th) * 128 + piece * 8);
    const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += w * __uint_as_float(r[i] << 16);
      acc[2 * i + 1] += w * __uint_as_float(r[i] & 0xffff0000u);
    }
  }
  const float inv = 1.0f / wsum;
  uint4 v;
  v.x = pack_bf16(acc[0] * inv, acc[1] * inv);
  v.y = pack_bf16(acc[2] * inv, acc[3] * inv);
  v.z = pack_bf16(acc[4] * inv, acc[5] * inv);
  v.w = pack_bf16(acc[6] * inv, acc[7] * inv);
  *reinterpret_cast<uint4*>(out.row(static_cast<int>(token), total_heads, head + head_offset) + piece * 8) = v;
}

int launch_dense_bf16(int num_tokens, int head_offset, const void* query, const void* key, const void* value,
                      const OutRoute& route, int heads, int total_heads, int kv_splits, void* workspace,
                      size_t workspace_bytes, void* stream) {
  const char* name = "dense_bf16_attention_d128";
  NOB_REQUIRE(num_tokens > 0 && heads > 0 && total_heads > 0, "%s: sizes must be positive", name);
  NOB_REQUIRE(head_offset >= 0 && head_offset <= total_heads - heads, "%s: head_offset %d outside [0, %d]", name,
              head_offset, total_heads - heads);
  NOB_REQUIRE(query && key && value && route.peer[0], "%s: NULL tensor", name);
  NOB_REQUIRE(heads <= 65535, "%s: heads %d exceeds grid limit", name, heads);
  const int n_kv = (num_tokens + kTile - 1) / kTile;
  NOB_REQUIRE(kv_splits >= 1 && kv_splits <= 64 && kv_splits <= n_kv, "%s: kv_splits %d outside [1, min(64, %d)]",
              name, kv_splits, n_kv);
  const size_t share = static_cast<size_t>(num_tokens) * heads;
  const size_t partial_bytes = (static_cast<size_t>(kv_splits) * share * 128 * 2 + 255) / 256 * 256;
  const size_t need = kv_splits > 1 ? partial_bytes + static_cast<size_t>(kv_splits) * share * 4 : 0;
  NOB_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), "%s: %zu B of workspace required for %d key splits, %zu B given",
              name, need, kv_splits, workspace_bytes);
  uint32_t* status = status_word_device_ptr();
  if (!status) return fail(kCudaError, "%s: no current CUDA device", name);

  CUtensorMap mq, mk, mv;
  const uint64_t head_stride = 128 * 2, token_stride = static_cast<uint64_t>(heads) * 128 * 2;
  int rc;
  if ((rc = make_tensor_map_3d(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, query, 128, heads, num_tokens, head_stride,
                               token_stride, 64, 1, kTile)))
    return rc;
  if ((rc = make_tensor_map_3d(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, key, 128, heads, num_tokens, head_stride,
                               token_stride, 64, 1, kTile)))
    return rc;
  if ((rc = make_tensor_map_3d(&mv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, value, 128, heads, num_tokens, head_stride,
                               token_stride, 64, 1, kTile)))
    return rc;

  const size_t smem = sizeof(Shared) + 1024;
  // No exponentials on the FMA pipe and P handed over in two halves: the fastest measured combination.
  auto kernel = fa_fwd_bf16_kernel<0, true>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess)
    return fail(kCudaError, "%s: cannot reserve %zu B of shared memory: %s", name, smem, cudaGetErrorString(err));
  const float scale_log2 = 0.08838834764831845f * 1.4426950408889634f;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* partial_out = static_cast<__nv_bfloat16*>(workspace);
  float* partial_lse = kv_splits > 1 ? reinterpret_cast<float*>(static_cast<char*>(workspace) + partial_bytes) : nullptr;
  dim3 grid((num_tokens + 2 * kTile - 1) / (2 * kTile), heads, kv_splits);
  kernel<<<grid, kThreads, smem, s>>>(mq, mk, mv, route, num_tokens, total_heads, head_offset, scale_log2, status,
                                      partial_out, partial_lse);
  if ((rc = check_launch(name))) return rc;
  if (kv_splits > 1) {
    const long long items = static_cast<long long>(share) * 16;
    fa_merge_splits_kernel<<<static_cast<unsigned>((items + 255) / 256), 256, 0, s>>>(
        partial_out, partial_lse, route, num_tokens, heads, total_heads, head_offset, kv_splits);
    rc = check_launch("dense_bf16_attention_d128(merge)");
  }
  return rc;
}

}  // namespace

int launch_merge_splits(const __nv_bfloat16* partial_out, const float* partial_lse, const OutRoute& route, int num_tokens,
                        int heads, int total_heads, int head_offset, int splits, void* stream) {
  const long long items = static_cast<long long>(num_tokens) * heads * 16;
  fa_merge_splits_kernel<<<static_cast<unsigned>((items + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      partial_out, partial_lse, route, num_tokens, heads, total_heads, head_offset, splits);
  return check_launch("attention(merge of key splits)");
}

}  // namespace nob200

extern "C" int nob200_dense_bf16_attention_d128(int num_tokens, int head_offset, const void* query, const void* key,
                                                const void* value, void* output, int heads, int total_heads,
                                                void* stream) {
  nob200::OutRoute route = {};
  route.peer[0] = static_cast<__nv_bfloat16*>(output);
  return nob200::launch_dense_bf16(num_tokens, head_offset, query, key, value, route, heads, total_heads, 1, nullptr, 0,
                                   stream);
}

extern "C" size_t nob200_dense_bf16_attention_d128_splitkv_workspace_bytes(int num_tokens, int heads, int kv_splits) {
  if (num_tokens <= 0 || heads <= 0 || kv_splits <= 1) return 0;
  const size_t share = static_cast<size_t>(num_tokens) * heads;
  return (static_cast<size_t>(kv_splits) * share * 128 * 2 + 255) / 256 * 256 + static_cast<size_t>(kv_splits) * share * 4;
}

extern "C" int nob200_dense_bf16_attention_d128_splitkv(int num_tokens, int head_offset, const void* query,
                                                        const void* key, const void* value, void* output, int heads,
                                                        int total_heads, int kv_splits, void* workspace,
                                                        size_t workspace_bytes, void* stream) {
  nob200::OutRoute route = {};
  route.peer[0] = static_cast<__nv_bfloat16*>(output);
  return nob200::launch_dense_bf16(num_tokens, head_offset, query, key, value, route, heads, total_heads, kv_splits,
                                   workspace, workspace_bytes, stream);
}

extern "C" int nob200_dense_bf16_attention_d128_scatter(int num_tokens, int head_offset, const void* query,
                                                        const void* key, const void* value,
                                                        void* const* peer_outputs, int world, int heads,
                                                        int total_heads, int kv_splits, void* workspace,
                                                        size_t workspace_bytes, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(peer_outputs && world >= 1 && world <= kMaxWorld, "dense_bf16_attention_d128_scatter: world %d outside [1, %d]",
              world, kMaxWorld);
  NOB_REQUIRE(num_tokens > 0 && num_tokens % world == 0,
              "dense_bf16_attention_d128_scatter: tokens (%d) must be divisible by the world size (%d)", num_tokens, world);
  OutRoute route = {};
  for (int r = 0; r < world; ++r) {
    NOB_REQUIRE(peer_outputs[r], "dense_bf16_attention_d128_scatter: NULL output for rank %d", r);
    route.peer[r] = static_cast<__nv_bfloat16*>(peer_outputs[r]);
  }
  route.tokens_per_rank = num_tokens / world;
  return launch_dense_bf16(num_tokens, head_offset, query, key, value, route, heads, total_heads, kv_splits, workspace,
                           workspace_bytes, stream);
}
