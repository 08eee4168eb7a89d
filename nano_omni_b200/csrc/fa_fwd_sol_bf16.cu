// "sol" block-sparse bf16 attention forward for head_dim 128 on sm_100a.
//
// Replaces the reference program sol_attention (src/nano_omni/kernels/attention/sol_attention.py:53-249)
// and, for the mask-driven form, the exact + finalize pair of the quantised sol paths
// (src/nano_omni/kernels/attention/nvfp4/sol_finalize.py:38-144).  For query block qb and head h:
//   - key blocks with mask[qb, h, kb] != 0 attend exactly;
//   - every other key block contributes one pseudo-key: logit q . pooled_k[h, kb] / sqrt(128),
//     weight = block length in the denominator, value = pooled_v[h, kb] (the SUM of the block's V)
//     in the numerator;
// all in one online softmax.  The mask comes from the router (sol_route.cu); blocks are 64 tokens
// (reference) or 128 tokens (the tile of this kernel).
//
// The same kernel also runs the two halves separately, as the reference's quantised paths split them:
//   kExactState  exact blocks only; writes the un-normalised numerator (bf16, probabilities relative to the
//                row maximum) and the state (row maximum in raw q.k units, sum of probabilities), the contract of
//                src/nano_omni/kernels/attention/sol_nvfp4.py:764-813 and .../int8_fp8/sol.py:167-225;
//   kFinalize    starts from such a numerator and state and merges the pooled pseudo-keys of the unselected
//                blocks (src/nano_omni/kernels/attention/nvfp4/sol_finalize.py:212-270); the output may alias
//                the numerator, every thread reads its own row before it writes it.
//
// CTA organisation.  One CTA owns 128 query rows of one head.  The TMA producer first builds the list of
// 128-key tiles that one of the CTA's query blocks selects, with one flag per (query block, 64-key half), followed
// by the tiles of pooled pseudo-keys.  The entries of that list are dealt alternately to two STREAMS: stream 0
// takes entries 0, 2, 4, ..., stream 1 entries 1, 3, 5, ...  Each stream is a complete online softmax over its
// share of the keys with its own score buffer, accumulator (TMEM) and (maximum, sum), run by one softmax
// warpgroup; the tcgen05 issuer ping-pongs between them as the dense kernel does between its two query tiles, so
// a stream's softmax always overlaps the other stream's MMAs however sparse or irregular the mask is.  The
// epilogue merges the two partial results (log-sum-exp merge), each warpgroup writing 64 of the 128 channels.
//   - a softmax thread masks the 64-key halves its own query block did not select (exact phase) or the columns
//     of selected blocks (pooled phase) and weights pooled columns by the block length; unselected halves are
//     neither loaded nor exponentiated;
//   - a row may see no key at all for several tiles, so the running maximum starts at -inf.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "fa_common.cuh"
#include "tensor_map.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

constexpr int kTile = 128;
constexpr int kHalfBytes = kTile * 64 * 2;
constexpr int kTileBytes = 2 * kHalfBytes;
constexpr int kStages = 5;
constexpr int kThreads = 384;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kMaxTiles = 2048;  // key tiles of 128 tokens: up to 262144 tokens

struct __align__(1024) Shared {
  uint8_t q[kTileBytes];
  uint8_t kv[kStages][kTileBytes];
  uint16_t tile_list[kMaxTiles];
  uint8_t tile_flags[kMaxTiles];  // bit 2*(query block inside the tile) + half: selected
  float4 merge[2][kTile];         // per stream and row: (maximum used, sum, raw maximum, stream has a result)
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];
  uint64_t p_full[2][2];
  uint64_t o_final[2];
  uint64_t list_ready;
  uint64_t merge_ready;
  int num_exact;
  uint32_t tmem_base;
  uint32_t abort;
};

static_assert(256 * 224 + 128 * 56 <= 384 * 168, "setmaxnreg split exceeds the registers the CTA owns");

enum SolMode : int { kFused = 0, kExactState = 1, kFinalize = 2 };

struct SolParams {
  const uint8_t* mask;  // [q_blocks, heads, k_blocks]
  const __nv_bfloat16* exact_in;  // kFinalize: numerator [tokens, exact_total_heads, 128] at exact_head_offset
  const float* state_in;          // kFinalize: [tokens, exact_total_heads, 2]
  int exact_total_heads, exact_head_offset;
  float* state_out;               // kExactState: [tokens, total_heads, 2]
  int force_first_block;          // kExactState: key block 0 attends whatever the mask says
  OutRoute out;         // local output tensor, or the owners' tensors on the peers
  int num_tokens, heads, total_heads, head_offset;
  int block;       // 64 or 128
  int num_blocks;  // ceil(num_tokens / block)
  int pooled_k_plane, pooled_v_plane;  // plane indices inside the pooled tensor
  float scale_log2;
  uint32_t* status;
};

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
fa_fwd_sol_bf16_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_pooled,
                       const SolParams P) {
  extern __shared__ uint8_t smem_raw[];
  Shared& S = *reinterpret_cast<Shared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int q0 = blockIdx.x * kTile;
  const int num_tokens = P.num_tokens;
  const int n_kv = (num_tokens + kTile - 1) / kTile;             // key tiles of the exact phase
  const int n_pool = MODE == kExactState ? 0 : (P.num_blocks + kTile - 1) / kTile;  // tiles of pooled pseudo-keys
  volatile uint32_t* abort_flag = &S.abort;
  uint32_t* status = P.status;
  const size_t mask_row_stride = static_cast<size_t>(P.heads) * P.num_blocks;  // between query blocks

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
    mbar_init(&S.list_ready, 1);
    mbar_init(&S.merge_ready, 8);
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

  // Order in which the issuer consumes K and V tiles of the entry sequence: K(0), K(1), then for every entry j
  // V(j) followed by K(j+2).  Producer and issuer both walk it with a running counter that names ring stage and
  // barrier phase.
  if (warp >= 8) {
    reg_dealloc<56>();
    if (warp == kProducerWarp) {
      // ---------------------------------------------- tile list, then TMA producer
      const int qb_first = q0 / P.block;
      const int qb_per_tile = kTile / P.block;  // 2 or 1
      // Every lane looks at 8 consecutive key tiles per round, all their mask bytes in flight at once; a warp scan
      // keeps the list in ascending tile order.
      int count = 0;
      constexpr int kPerLane = 8;
      for (int base = 0; MODE != kFinalize && base < n_kv; base += 32 * kPerLane) {
        const int kt0 = base + kPerLane * lane;
        uint32_t flags[kPerLane];
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) flags[i] = 0;
        for (int u = 0; u < qb_per_tile; ++u) {
          const int qb = qb_first + u;
          if (qb >= P.num_blocks) continue;
          const uint8_t* row = P.mask + qb * mask_row_stride + static_cast<size_t>(head) * P.num_blocks;
#pragma unroll
          for (int i = 0; i < kPerLane; ++i) {
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int kb = (P.block == 64) ? 2 * (kt0 + i) + h2 : kt0 + i;
              if (kt0 + i < n_kv && kb < P.num_blocks && (row[kb] || (P.force_first_block && kb == 0)))
                flags[i] |= 1u << (2 * u + h2);
            }
          }
        }
        int mine = 0;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) mine += flags[i] != 0;
        int before = mine;  // inclusive scan over the lanes
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int other = __shfl_up_sync(0xffffffffu, before, d);
          if (lane >= d) before += other;
        }
        const int total = __shfl_sync(0xffffffffu, before, 31);
        int at = count + before - mine;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
          if (flags[i]) {
            if (NOB_CHECK(at >= 0 && at < kMaxTiles, status)) {
              S.tile_list[at] = static_cast<uint16_t>(kt0 + i);
              S.tile_flags[at] = static_cast<uint8_t>(flags[i]);
            }
            ++at;
          }
        }
        count += total;
      }
      __syncwarp();
      if (lane == 0) {
        S.num_exact = count;
        mbar_arrive(&S.list_ready);  // release: the list and its length are visible to the waiters

        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_pooled);
        mbar_expect_tx(&S.q_full, kTileBytes);
        tma_load_3d(S.q, &map_q, &S.q_full, 0, head, q0);
        tma_load_3d(S.q + kHalfBytes, &map_q, &S.q_full, 64, head, q0);
        const int n_it = count + n_pool;
        int issued = 0;
        // load number `issued` of the consumption order: K-like (is_v = 0) or V-like tile of entry j
        auto load = [&](int j, int is_v) -> bool {
          const int st = issued % kStages;
          if (issued >= kStages) {
            if (!mbar_wait(&S.kv_empty[st], ((issued / kStages) - 1) & 1, abort_flag, status, kWaitTimeoutRing)) return false;
          }
          mbar_expect_tx(&S.kv_full[st], kTileBytes);
          if (j < count) {
            const CUtensorMap* map = is_v ? &map_v : &map_k;
            const int tok = S.tile_list[j] * kTile;
            tma_load_3d(S.kv[st], map, &S.kv_full[st], 0, head, tok);
            tma_load_3d(S.kv[st] + kHalfBytes, map, &S.kv_full[st], 64, head, tok);
          } else {
            const int plane = is_v ? P.pooled_v_plane : P.pooled_k_plane;
            const int row = (j - count) * kTile;
            tma_load_3d(S.kv[st], &map_pooled, &S.kv_full[st], 0, row, plane * P.heads + head);
            tma_load_3d(S.kv[st] + kHalfBytes, &map_pooled, &S.kv_full[st], 64, row, plane * P.heads + head);
          }
          ++issued;
          return true;
        };
        bool fed = n_it == 0 || load(0, 0);
        if (fed && n_it > 1) fed = load(1, 0);
        for (int j = 0; fed && j < n_it; ++j) {
          fed = load(j, 1);
          if (fed && j + 2 < n_it) fed = load(j + 2, 0);
        }
        if (*abort_flag) {
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
      // All 32 lanes run the warp-uniform control flow; one elected lane issues (see elect_one()), one asm block per
      // group of MMAs with ready-made 64-bit descriptors.  The waits on the probabilities are on every entry's chain
      // (P stored -> PV -> next QK of the stream -> scores complete) and poll; K / V tiles were loaded long before
      // and their waits may sleep.
      {
        constexpr uint32_t idesc_qk = umma_idesc(kDF32, kFmtBF16, kFmtBF16, 0, 0, kTile, kTile);
        constexpr uint32_t idesc_pv = umma_idesc(kDF32, kFmtBF16, kFmtBF16, 0, 1, kTile, 128);
        const uint64_t desc_k_major = umma_smem_desc(0, 16, 1024, kSwizzle128B);
        const uint64_t desc_n_major = umma_smem_desc(0, kHalfBytes, 1024, kSwizzle128B);
        const uint64_t q_desc = desc_k_major + (smem_u32(S.q) >> 4);
        const uint64_t kv_k_desc = desc_k_major + (smem_u32(S.kv[0]) >> 4);
        const uint64_t kv_n_desc = desc_n_major + (smem_u32(S.kv[0]) >> 4);
        // S_t = Q K^T: eight MMAs of 16 channels (two 64-channel halves of a tile, 32 bytes per step), then the commits
        auto issue_qk = [&](int t, int st) {
          const uint64_t a = q_desc, b = kv_k_desc + st * (kTileBytes >> 4);
          const uint64_t h = kHalfBytes >> 4;
          const uint32_t d = tmem + t * kTile;
          if (elect_one()) {
            asm volatile(
                "{\n\t.reg .pred p0, p1;\n\t"
                "setp.ne.b32 p0, 0, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %10, %1, p0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %11, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %12, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %13, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %6, %14, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %15, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %8, %16, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %9, %17, %1, p1;\n\t}" ::"r"(d),
                "r"(idesc_qk), "l"(a), "l"(a + 2), "l"(a + 4), "l"(a + 6), "l"(a + h), "l"(a + h + 2), "l"(a + h + 4),
                "l"(a + h + 6), "l"(b), "l"(b + 2), "l"(b + 4), "l"(b + 6), "l"(b + h), "l"(b + h + 2), "l"(b + h + 4),
                "l"(b + h + 6)
                : "memory");
            tc_commit(&S.s_full[t]);
            tc_commit(&S.kv_empty[st]);
          }
        };
        // O_t += P_t[:, 64 half ...] V[...]: four MMAs of 16 keys (16 rows of 128 B = 2048 B of V; 8 TMEM columns of P)
        auto issue_pv = [&](int t, int st, bool accumulate, int half, bool last) {
          const uint64_t b = kv_n_desc + st * (kTileBytes >> 4) + half * (4 * 2048 >> 4);
          const uint32_t d = tmem + 256 + t * kTile, a = tmem + t * kTile + half * 32;
          if (elect_one()) {
            asm volatile(
                "{\n\t.reg .pred p0, p1;\n\t"
                "setp.ne.b32 p0, %2, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], %7, %1, p0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %8, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %9, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], [%6], %10, %1, p1;\n\t}" ::"r"(d),
                "r"(idesc_pv), "r"((accumulate || half > 0) ? 1u : 0u), "r"(a), "r"(a + 8), "r"(a + 16), "r"(a + 24), "l"(b),
                "l"(b + (2048 >> 4)), "l"(b + 2 * (2048 >> 4)), "l"(b + 3 * (2048 >> 4))
                : "memory");
            if (last) tc_commit(&S.kv_empty[st]);
          }
        };

        bool ok = warp_rest(&S.list_ready, 0, abort_flag, status, kWaitTimeoutLoad);
        const int n_it = ok ? S.num_exact + n_pool : 0;
        ok = ok && warp_rest(&S.q_full, 0, abort_flag, status, kWaitTimeoutLoad);
        int taken = 0;  // loads consumed so far, in the order the producer issues them
        // waits for the next load of the order and returns its stage (-1: gave up)
        auto next_stage = [&]() -> int {
          const int st = taken % kStages;
          if (!warp_rest(&S.kv_full[st], (taken / kStages) & 1, abort_flag, status, kWaitTimeoutLoad)) return -1;
          ++taken;
          return st;
        };
        // scores of entries 0 and 1: one per stream
        for (int j = 0; ok && j < 2 && j < n_it; ++j) {
          const int st = next_stage();
          ok = st >= 0;
          if (!ok) break;
          tc_fence_after();
          issue_qk(j, st);
        }
        for (int j = 0; ok && j < n_it; ++j) {
          const int t = j & 1;                 // the stream of entry j
          const uint32_t parity = (j >> 1) & 1;  // its (j >> 1)-th entry
          const bool accumulate = (j >> 1) > 0 || (MODE == kFinalize && t == 0);
          const int sv = next_stage();
          ok = sv >= 0;
          if (!ok) break;
          // the stream's next K tile is awaited before the probabilities, so that PV and QK go out back to back
          int sk = -1;
          if (j + 2 < n_it) {
            sk = next_stage();
            ok = sk >= 0;
            if (!ok) break;
          }
          if (!(ok = warp_poll(&S.p_full[t][0], parity, abort_flag, status, kWaitTimeoutSoftmax))) break;
          tc_fence_after();
          issue_pv(t, sv, accumulate, 0, false);
          if (!(ok = warp_poll(&S.p_full[t][1], parity, abort_flag, status, kWaitTimeoutSoftmax))) break;
          tc_fence_after();
          issue_pv(t, sv, accumulate, 1, true);
          if (sk >= 0) issue_qk(t, sk);  // in order behind this stream's PV: S is free once P has been consumed
        }
        if (ok && elect_one()) {
          tc_commit(&S.o_final[0]);
          tc_commit(&S.o_final[1]);
        }
      }
    }
  } else {
    // ------------------------------------------------- softmax + epilogue warps: warpgroup t runs stream t
    reg_alloc<224>();
    const int t = warp >> 2;
    {
      const int row = (warp & 3) * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t s_addr = tmem + lane_base + t * kTile;
      const uint32_t o_addr = tmem + lane_base + 256 + t * kTile;
      const int token = q0 + row;
      // all 32 rows of a warp lie in one query block (blocks are 64 or 128 rows)
      const int u = (P.block == 64) ? (row >> 6) : 0;  // query block inside the tile
      const int qb = min(token / P.block, P.num_blocks - 1);
      const uint8_t* mask_row = P.mask + qb * mask_row_stride + static_cast<size_t>(head) * P.num_blocks;
      const float block_len = static_cast<float>(P.block);
      const float tail_len = static_cast<float>(num_tokens - (P.num_blocks - 1) * P.block);
      const float scale_log2 = P.scale_log2;
      float m_used = -INFINITY;
      float m_raw = -INFINITY;  // kExactState: true row maximum, raw q.k units
      uint64_t la = 0ull, lb = 0ull;
      int done = 0;  // entries this stream has processed: phase of its S/P barriers
      bool ok = __all_sync(0xffffffffu, mbar_wait(&S.list_ready, 0, abort_flag, status, kWaitTimeoutLoad));
      const int num_exact = ok ? S.num_exact : 0;
      const int n_it = ok ? num_exact + n_pool : 0;
      if (MODE == kFinalize && t == 0) {
        // stream 0 starts from the exact stage's numerator (accumulator) and its (maximum, sum)
        const bool live = token < num_tokens;
        const size_t at = (static_cast<size_t>(live ? token : 0) * P.exact_total_heads + head + P.exact_head_offset);
        if (live) {
          m_used = P.state_in[2 * at] * scale_log2;
          la = pack2(P.state_in[2 * at + 1], 0.0f);
        }
        const uint4* src = reinterpret_cast<const uint4*>(P.exact_in + at * 128);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v = live ? src[4 * c + i] : make_uint4(0u, 0u, 0u, 0u);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              o[8 * i + 2 * k] = w[k] << 16;
              o[8 * i + 2 * k + 1] = w[k] & 0xffff0000u;
            }
          }
          tmem_st32(o_addr + 32 * c, o);
        }
        tc_wait_st();  // ordered before the issuer's first PV by the first P arrival of this thread
      }

      // One tile of scores for this row: bit i of valid[i/32] says whether column i counts.
      auto run_tile = [&](const uint32_t (&valid)[4], bool pooled_phase, int last_col) -> bool {
        const bool none_valid = (valid[0] | valid[1] | valid[2] | valid[3]) == 0u;
        if (!warp_poll(&S.s_full[t], done & 1, abort_flag, status, kWaitTimeoutMma)) return false;  // on the entry's chain: poll
        tc_fence_after();
        if (none_valid) {
          // this row's query block did not select the tile: P = 0, nothing else changes
          uint32_t zero[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) zero[i] = 0u;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            tmem_st32(s_addr + 32 * half, zero);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&S.p_full[t][half]);
          }
          return true;
        }
        // A 64-key half without a valid column (its block was not selected by this row's query block, or lies
        // past the end) is neither loaded nor exponentiated: its P is zero.  Rows of a warp share the decision,
        // and each combination of live halves is its own straight-line code.
        auto body = [&](auto first_tag, auto second_tag) {
          constexpr bool kLive[2] = {decltype(first_tag)::value, decltype(second_tag)::value};
          constexpr int kFirst = kLive[0] ? 0 : 64, kCount = (kLive[0] ? 64 : 0) + (kLive[1] ? 64 : 0);
          uint32_t s[kCount];  // columns kFirst .. kFirst + kCount - 1
#pragma unroll
          for (int c = 0; c < kCount; c += 32) tmem_ld32(s_addr + kFirst + c, *reinterpret_cast<uint32_t(*)[32]>(&s[c]));
          tc_wait_ld();
          bool full = true;
#pragma unroll
          for (int w = kFirst / 32; w < (kFirst + kCount) / 32; ++w) full = full && valid[w] == 0xffffffffu;
          if (!full) {
#pragma unroll
            for (int i = 0; i < kCount; ++i)
              if (!((valid[(kFirst + i) >> 5] >> ((kFirst + i) & 31)) & 1u)) s[i] = 0xff800000u;  // -inf
          }
          float mx0 = __uint_as_float(s[0]), mx1 = __uint_as_float(s[1]);
#pragma unroll
          for (int i = 2; i < kCount - 2; i += 4) {
            mx0 = max3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
            mx1 = max3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
          }
          mx0 = max3(mx0, __uint_as_float(s[kCount - 2]), __uint_as_float(s[kCount - 1]));
          if (MODE == kExactState) m_raw = fmaxf(m_raw, fmaxf(mx0, mx1));
          const float mx = fmaxf(mx0, mx1) * scale_log2;  // finite: at least one column counts
          if (MODE != kFinalize && done == 0) {
            m_used = mx;  // O is overwritten by the tile's first PV; nothing to rescale
          } else if (__any_sync(0xffffffffu, mx > m_used + kRescaleThreshold)) {
            const float m_new = fmaxf(m_used, mx);
            const float alpha = (m_new == -INFINITY) ? 1.0f : ex2(m_used - m_new);  // 0 when the row had no key yet
            const uint64_t alpha2 = pack2(alpha, alpha);
            la = fma2(la, alpha2, 0ull);
            lb = fma2(lb, alpha2, 0ull);
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
          const uint64_t weight2 = pack2(block_len, block_len);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t p[32];
            if (!kLive[half]) {
#pragma unroll
              for (int i = 0; i < 32; ++i) p[i] = 0u;
            } else {
#pragma unroll
              for (int i = 0; i < 64; i += 4) {
                const int e = half * 64 + i;  // column of the tile
                const int r = e - kFirst;     // register
                const uint64_t xa = fma2(pack2(__uint_as_float(s[r]), __uint_as_float(s[r + 1])), scale2, neg_m2);
                const uint64_t xb = fma2(pack2(__uint_as_float(s[r + 2]), __uint_as_float(s[r + 3])), scale2, neg_m2);
                float x0, x1, x2, x3;
                unpack2(xa, x0, x1);
                unpack2(xb, x2, x3);
                const float a = ex2(x0), b = ex2(x1), c = ex2(x2), d = ex2(x3);  // exp2(-inf) = 0 for masked columns
                if (!pooled_phase) {
                  la = add2(la, pack2(a, b));
                  lb = add2(lb, pack2(c, d));
                } else {
                  // a pooled column stands for `block` keys (the last block possibly fewer)
                  uint64_t wa = weight2, wb = weight2;
                  if (last_col >= e && last_col < e + 4) {
                    wa = pack2(last_col == e ? tail_len : block_len, last_col == e + 1 ? tail_len : block_len);
                    wb = pack2(last_col == e + 2 ? tail_len : block_len, last_col == e + 3 ? tail_len : block_len);
                  }
                  la = fma2(pack2(a, b), wa, la);
                  lb = fma2(pack2(c, d), wb, lb);
                }
                p[i / 2] = pack_bf16(a, b);
                p[i / 2 + 1] = pack_bf16(c, d);
              }
            }
            tmem_st32(s_addr + 32 * half, p);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&S.p_full[t][half]);
          }
        };
        const bool first = (valid[0] | valid[1]) != 0u, second = (valid[2] | valid[3]) != 0u;
        if (first && second) {
          body(std::true_type{}, std::true_type{});
        } else if (first) {
          body(std::true_type{}, std::false_type{});
        } else {
          body(std::false_type{}, std::true_type{});
        }
        return true;
      };

      // ---- this stream's entries: exact tiles first, then tiles of pooled pseudo-keys
      for (int j = t; ok && j < n_it; j += 2) {
        uint32_t valid[4];
        if (j < num_exact) {
          const uint32_t mine = (S.tile_flags[j] >> (2 * u)) & 3u;
          const int limit = num_tokens - S.tile_list[j] * kTile;  // keys of the tile that exist
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            const int n_valid = ((mine >> h2) & 1u) ? max(0, min(64, limit - 64 * h2)) : 0;
            valid[2 * h2] = n_valid >= 32 ? 0xffffffffu : ((1u << n_valid) - 1u);
            valid[2 * h2 + 1] = n_valid >= 64 ? 0xffffffffu : (n_valid > 32 ? ((1u << (n_valid - 32)) - 1u) : 0u);
          }
          ok = run_tile(valid, false, -1);
        } else {
          // one pseudo-key per key block this row's query block did NOT select
          const int kb0 = (j - num_exact) * kTile;
          // the 32 rows of a warp share their query block: each lane tests one block, a ballot builds the word
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const int kb = kb0 + 32 * w + lane;
            valid[w] = __ballot_sync(0xffffffffu, kb < P.num_blocks && mask_row[kb] == 0);
          }
          ok = run_tile(valid, true, P.num_blocks - 1 - kb0);
        }
        ++done;
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&S.o_final[t], 0, abort_flag, status, kWaitTimeoutMma));
      if (ok) {
        // ---- merge of the two streams; this warpgroup writes channels [64 t, 64 t + 64) of every row
        tc_fence_after();
        float l0, l1, l2, l3;
        unpack2(la, l0, l1);
        unpack2(lb, l2, l3);
        const bool has = done > 0 || (MODE == kFinalize && t == 0);  // this stream's accumulator holds something
        const float4 mine4 = make_float4(m_used, (l0 + l1) + (l2 + l3), m_raw, has ? 1.0f : 0.0f);
        S.merge[t][row] = mine4;
        __syncwarp();
        if (lane == 0) mbar_arrive(&S.merge_ready);  // release: the other warpgroup sees the row's entry
        ok = __all_sync(0xffffffffu, mbar_wait(&S.merge_ready, 0, abort_flag, status, kWaitTimeoutSoftmax));
        if (ok) {
          const float4 other4 = S.merge[t ^ 1][row];
          // reference point of the merged result: the larger used maximum (fused, finalize) or the true raw maximum
          float factor_mine, factor_other, total;
          if (MODE == kExactState) {
            const float top_raw = fmaxf(mine4.z, other4.z);
            const float top = top_raw * scale_log2;
            factor_mine = (mine4.w != 0.f && mine4.x != -INFINITY && top_raw != -INFINITY) ? ex2(mine4.x - top) : 0.f;
            factor_other = (other4.w != 0.f && other4.x != -INFINITY && top_raw != -INFINITY) ? ex2(other4.x - top) : 0.f;
            total = mine4.y * factor_mine + other4.y * factor_other;
            if (t == 0 && token < num_tokens && NOB_CHECK(head + P.head_offset < P.total_heads, status)) {
              float* st = P.state_out + 2 * (static_cast<size_t>(token) * P.total_heads + head + P.head_offset);
              *reinterpret_cast<float2*>(st) = make_float2(top_raw, total);
            }
          } else {
            const float top = fmaxf(mine4.w != 0.f ? mine4.x : -INFINITY, other4.w != 0.f ? other4.x : -INFINITY);
            factor_mine = (mine4.w != 0.f && mine4.x != -INFINITY) ? ex2(mine4.x - top) : 0.f;
            factor_other = (other4.w != 0.f && other4.x != -INFINITY) ? ex2(other4.x - top) : 0.f;
            total = mine4.y * factor_mine + other4.y * factor_other;
            const float inv = 1.0f / total;
            factor_mine *= inv;
            factor_other *= inv;
          }
          const uint32_t mine_addr = tmem + lane_base + 256 + t * kTile + 64 * t;
          const uint32_t other_addr = tmem + lane_base + 256 + (t ^ 1) * kTile + 64 * t;
          __nv_bfloat16* dst = P.out.row(token < num_tokens ? token : 0, P.total_heads, head + P.head_offset) + 64 * t;
          const bool store =
              token < num_tokens && route_open(P.out, status) &&
              NOB_CHECK(head + P.head_offset < P.total_heads &&
                            (P.out.tokens_per_rank == 0 ||
                             (token / P.out.tokens_per_rank < kMaxWorld && P.out.peer[token / P.out.tokens_per_rank])),
                        status);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t a[32], b[32];
            tmem_ld32(mine_addr + 32 * c, a);
            tmem_ld32(other_addr + 32 * c, b);
            tc_wait_ld();
            if (store) {
              float r[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                // an accumulator that was never written holds arbitrary bits: select, do not multiply by zero
                const float x = factor_mine != 0.f ? __uint_as_float(a[i]) * factor_mine : 0.f;
                const float y = factor_other != 0.f ? __uint_as_float(b[i]) * factor_other : 0.f;
                r[i] = x + y;
              }
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 v;
                v.x = pack_bf16(r[i], r[i + 1]);
                v.y = pack_bf16(r[i + 2], r[i + 3]);
                v.z = pack_bf16(r[i + 4], r[i + 5]);
                v.w = pack_bf16(r[i + 6], r[i + 7]);
                *reinterpret_cast<uint4*>(dst + 32 * c + i) = v;
              }
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

}  // namespace
}  // namespace nob200

namespace nob200 {
namespace {
struct SolExtra {
  int mode = kFused;
  const void* exact_in = nullptr;
  const void* state_in = nullptr;
  int exact_total_heads = 0, exact_head_offset = 0;  // 0 total: same indexing as the output
  void* state_out = nullptr;
  int force_first_block = 0;
};

int launch_sol(int num_tokens, int head_offset, const void* query, const void* key, const void* value,
               const void* pooled, const void* mask, const OutRoute& route, int heads, int total_heads, int block,
               int pooled_planes, void* stream, const SolExtra& extra = SolExtra()) {
  void* output = route.peer[0];
  const int mode = extra.mode;
  if (mode == kFinalize) key = value = query;          // no exact phase: the maps are never used
  if (mode == kExactState) { pooled = query; pooled_planes = 2; }  // no pooled phase
  NOB_REQUIRE(num_tokens > 0 && heads > 0 && total_heads > 0, "sol_attention_d128: sizes must be positive");
  NOB_REQUIRE(head_offset >= 0 && head_offset <= total_heads - heads,
              "sol_attention_d128: head_offset %d outside [0, %d]", head_offset, total_heads - heads);
  NOB_REQUIRE(block == 64 || block == 128, "sol_attention_d128: block must be 64 or 128 (got %d)", block);
  NOB_REQUIRE(pooled_planes == 2 || pooled_planes == 3, "sol_attention_d128: pooled must have 2 or 3 planes");
  NOB_REQUIRE(query && key && value && pooled && mask && output, "sol_attention_d128: NULL tensor");
  NOB_REQUIRE(heads <= 65535, "sol_attention_d128: heads %d exceeds grid limit", heads);
  NOB_REQUIRE((num_tokens + kTile - 1) / kTile <= kMaxTiles, "sol_attention_d128: at most %d tokens", kMaxTiles * kTile);
  uint32_t* status = status_word_device_ptr();
  if (!status) return fail(kCudaError, "sol_attention_d128: no current CUDA device");
  const int num_blocks = (num_tokens + block - 1) / block;

  CUtensorMap mq, mk, mv, mp;
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
  // pooled [planes, heads, blocks, 128]: rows = blocks, outer = plane * heads + head
  if (mode == kExactState) {
    mp = mq;
  } else if ((rc = make_tensor_map_3d(&mp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, pooled, 128, num_blocks,
                                      static_cast<uint64_t>(pooled_planes) * heads, 256,
                                      static_cast<uint64_t>(num_blocks) * 256, 64, kTile, 1))) {
    return rc;
  }

  SolParams params;
  params.mask = static_cast<const uint8_t*>(mask);
  params.out = route;
  params.num_tokens = num_tokens;
  params.heads = heads;
  params.total_heads = total_heads;
  params.head_offset = head_offset;
  params.block = block;
  params.num_blocks = num_blocks;
  // fused: plain block means (plane 0) against un-centred keys; finalize: centred means (plane 1), as the exact
  // stage of the quantised paths works on centred keys
  params.pooled_k_plane = mode == kFinalize ? 1 : 0;
  params.pooled_v_plane = pooled_planes - 1;
  params.exact_in = static_cast<const __nv_bfloat16*>(extra.exact_in);
  params.state_in = static_cast<const float*>(extra.state_in);
  params.exact_total_heads = extra.exact_total_heads > 0 ? extra.exact_total_heads : total_heads;
  params.exact_head_offset = extra.exact_total_heads > 0 ? extra.exact_head_offset : head_offset;
  params.state_out = static_cast<float*>(extra.state_out);
  params.force_first_block = extra.force_first_block;
  params.scale_log2 = 0.08838834764831845f * 1.4426950408889634f;
  params.status = status;

  const size_t smem = sizeof(Shared) + 1024;
  auto* kernel = mode == kFused        ? fa_fwd_sol_bf16_kernel<kFused>
                 : mode == kExactState ? fa_fwd_sol_bf16_kernel<kExactState>
                                       : fa_fwd_sol_bf16_kernel<kFinalize>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess)
    return fail(kCudaError, "sol_attention_d128: cannot reserve %zu B of shared memory: %s", smem,
                cudaGetErrorString(err));
  dim3 grid((num_tokens + kTile - 1) / kTile, heads);
  kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, mp, params);
  return check_launch("sol_attention_d128");
}
}  // namespace
}  // namespace nob200

extern "C" int nob200_sol_attention_d128(int num_tokens, int head_offset, const void* query, const void* key,
                                         const void* value, const void* pooled, const void* mask, void* output,
                                         int heads, int total_heads, int block, int pooled_planes, void* stream) {
  nob200::OutRoute route = {};
  route.peer[0] = static_cast<__nv_bfloat16*>(output);
  return nob200::launch_sol(num_tokens, head_offset, query, key, value, pooled, mask, route, heads, total_heads, block,
                            pooled_planes, stream);
}

extern "C" int nob200_sol_attention_d128_scatter(int num_tokens, int head_offset, const void* query, const void* key,
                                                 const void* value, const void* pooled, const void* mask,
                                                 void* const* peer_outputs, int world, int heads, int total_heads,
                                                 int block, int pooled_planes, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(peer_outputs && world >= 1 && world <= kMaxWorld, "sol_attention_d128_scatter: world %d outside [1, %d]",
              world, kMaxWorld);
  NOB_REQUIRE(num_tokens > 0 && num_tokens % world == 0,
              "sol_attention_d128_scatter: tokens (%d) must be divisible by the world size (%d)", num_tokens, world);
  OutRoute route = {};
  for (int r = 0; r < world; ++r) {
    NOB_REQUIRE(peer_outputs[r], "sol_attention_d128_scatter: NULL output for rank %d", r);
    route.peer[r] = static_cast<__nv_bfloat16*>(peer_outputs[r]);
  }
  route.tokens_per_rank = num_tokens / world;
  return launch_sol(num_tokens, head_offset, query, key, value, pooled, mask, route, heads, total_heads, block,
                    pooled_planes, stream);
}

extern "C" int nob200_sol_exact_state_bf16_d128(int num_tokens, int head_offset, const void* query, const void* key,
                                                const void* value, const void* selected, void* output, void* state,
                                                int heads, int total_heads, int block, int force_first_block,
                                                void* stream) {
  using namespace nob200;
  NOB_REQUIRE(state, "sol_exact_state_bf16_d128: NULL state");
  OutRoute route = {};
  route.peer[0] = static_cast<__nv_bfloat16*>(output);
  SolExtra extra;
  extra.mode = kExactState;
  extra.state_out = state;
  extra.force_first_block = force_first_block != 0;
  return launch_sol(num_tokens, head_offset, query, key, value, nullptr, selected, route, heads, total_heads, block, 2,
                    stream, extra);
}

extern "C" int nob200_sol_nvfp4_finalize(int num_tokens, int head_offset, const void* query, const void* pooled,
                                         const void* selected, const void* exact, const void* state, void* output,
                                         int heads, int total_heads, int block, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(exact && state, "sol_nvfp4_finalize: NULL exact numerator or state");
  OutRoute route = {};
  route.peer[0] = static_cast<__nv_bfloat16*>(output);
  SolExtra extra;
  extra.mode = kFinalize;
  extra.exact_in = exact;
  extra.state_in = state;
  return launch_sol(num_tokens, head_offset, query, nullptr, nullptr, pooled, selected, route, heads, total_heads, block,
                    3, stream, extra);
}

extern "C" int nob200_sol_nvfp4_finalize_scatter(int num_tokens, int head_offset, const void* query, const void* pooled,
                                                 const void* selected, const void* exact, const void* state,
                                                 void* const* peer_outputs, int world, int heads, int total_heads,
                                                 int block, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(exact && state, "sol_nvfp4_finalize_scatter: NULL exact numerator or state");
  NOB_REQUIRE(peer_outputs && world >= 1 && world <= kMaxWorld, "sol_nvfp4_finalize_scatter: world %d outside [1, %d]",
              world, kMaxWorld);
  NOB_REQUIRE(num_tokens > 0 && num_tokens % world == 0,
              "sol_nvfp4_finalize_scatter: tokens (%d) must be divisible by the world size (%d)", num_tokens, world);
  OutRoute route = {};
  for (int r = 0; r < world; ++r) {
    NOB_REQUIRE(peer_outputs[r], "sol_nvfp4_finalize_scatter: NULL output for rank %d", r);
    route.peer[r] = static_cast<__nv_bfloat16*>(peer_outputs[r]);
  }
  route.tokens_per_rank = num_tokens / world;
  SolExtra extra;
  extra.mode = kFinalize;
  extra.exact_in = exact;
  extra.state_in = state;
  extra.exact_total_heads = heads;  // the numerator and state of this rank's heads are local tensors
  extra.exact_head_offset = 0;
  return launch_sol(num_tokens, head_offset, query, nullptr, nullptr, pooled, selected, route, heads, total_heads, block,
                    3, stream, extra);
}
