// NVFP4 attention forward for head_dim 128 on sm_100a: block-scaled fp4 tensor-core MMAs for both products.
//
// Replaces the reference programs dense_nvfp4_attention_d128
// (src/nano_omni/kernels/attention/dense_nvfp4.py:54-561) and sol_nvfp4_attention_d128
// (src/nano_omni/kernels/attention/sol_nvfp4.py:82-620).  Operands are the layouts nob200_nvfp4_prepare writes:
// Q, K packed e2m1 [heads, P, 64 bytes] with ue4m3 scales [heads, P, 8]; V packed [heads, 128, Pk/2 bytes]
// (channel-major, 16-token groups) with scales [heads, 128, Pk/16]; scales in 512-byte atoms of 128 rows x 4 groups.
//
//   S = Q4 K4^T        tcgen05.mma kind::mxf4nvf4.block_scale.block16 (K = 64 per MMA, two per 128-key tile), both
//                      operands from shared memory (64-byte rows, 64-byte swizzle), scale factors copied from the
//                      atoms to TMEM with tcgen05.cp, fp32 scores in TMEM
//   softmax            one thread per query row; running maximum in raw q.k units raised with every key tile (exact,
//                      as the reference does per key block: dense_nvfp4.py:250-266, sol_nvfp4.py:793-803), probabilities
//                      p = exp2((s - m) log2e/sqrt(128) + log2(2688)), row sum of the unrounded p
//   P -> e2m1          per 16 keys: scale = max p / 6, stored as ue4m3; codes = round(p / scale) on the e2m1 grid
//                      (dense_nvfp4.py:255-289; arithmetic of sol_nvfp4.py:764-781); eight codes per 32-bit TMEM column,
//                      the row's four scales of a 64-key step in one column of the row's lane quadrant
//   O += P4 V4         the same block-scaled MMA with P (and its scales) read from TMEM, V K-major from shared memory
//
// CTA organisation as the bf16 kernel: 256 query rows of one head (tiles A and B), one score buffer used by A and B in
// turn, warps 0-3 / 4-7 softmax for A / B, warp 8 TMA producer, warp 9 issues the score MMAs, warp 10 the value MMAs.
// TMEM columns: S 0-127, P_A 128-143, P_B 144-159, scales of P_A 160-167, P_B 168-175, Q_A 176-183, Q_B 184-191,
// K 192-199, V 200-207, O_A 256-383, O_B 384-511.
//
// kSol: each query tile visits only the 64-key blocks that one of its two 64-row query blocks selects (mask u8
// [query blocks, heads, key blocks] of 64-token blocks; key block 0 always attends), so tiles A and B walk lists of
// their own, a list entry being one key block with a flag per query block, and every score / value MMA group brings
// its own K / V tile through the ring.  K data come as the 128-row tile that starts at the block's first token, K
// scales as the two atoms of the aligned 128-row tile the block lies in: the score MMAs have N = 64 and read the
// scales of an odd block two TMEM columns in (key row n of an atom sits in lane n % 32, column n / 32).  V comes as
// [channel][64 bytes] from the block's first token on with the one scale atom of its four 16-token groups: one
// value MMA of K = 64 per entry.  A softmax warp whose query block did not select the entry stores zero codes.
// The running maximum is raised per 64-key block, as the reference does.  The result is the un-normalised numerator
// divided by 2688 and the state (running maximum in raw units, sum of p / 2688) that nob200_sol_nvfp4_finalize
// consumes.
#include <cuda.h>

#include "common.cuh"
#include "fa_common.cuh"
#include "tensor_map.cuh"
#include "../../include/nano_omni_b200.h"

#ifndef NOB200_PFULL_WAIT
#define NOB200_PFULL_WAIT spin
#endif

namespace nob200 {
namespace {

constexpr int kTile = 128;
constexpr int kTileBytes = kTile * 64;  // 128 rows of 128 e2m1 = 8 KiB
constexpr int kSfBytes = 1024;          // two 512-byte scale atoms (128 rows x 8 groups)
constexpr int kStages = 8;
constexpr int kThreads = 384;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kPvWarp = 10;
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxTiles = 4096;  // list entries of a sol query tile: 64-key blocks (262144 keys)
constexpr float kLog2PScale = 11.39231742277876f;  // log2(6 * 448)
constexpr float kInvPScale = 1.0f / 2688.0f;

constexpr uint32_t kColS = 0, kColP = 128, kColSfP = 160, kColSfQ = 176, kColSfK = 192, kColSfV = 200, kColO = 256;

constexpr int kServiceRegs = 88;
constexpr int kSoftmaxRegs = (384 * 168 - 128 * kServiceRegs) / 256 / 8 * 8;
static_assert(256 * kSoftmaxRegs + 128 * kServiceRegs <= 384 * 168, "setmaxnreg split exceeds the registers the CTA owns");

struct __align__(1024) Shared {
  uint8_t q[2][kTileBytes];
  uint8_t kv[kStages][kTileBytes];
  uint8_t q_sf[2][kSfBytes];
  uint8_t kv_sf[kStages][kSfBytes];
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];
  uint64_t s_taken[2];
  uint64_t p_full[2][2];
  uint64_t pv_done[2];
  uint64_t list_ready;
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t qk_issued;
  int list_len[2];
  uint16_t list[2][kMaxTiles];
  uint8_t flags[2][kMaxTiles];  // bit (query block inside the tile): that query block selected the key block
};

struct Params {
  const float* unused;
  const uint8_t* q_sf;
  const uint8_t* k_sf;
  const uint8_t* v_sf;
  const uint8_t* selected;  // kSol
  __nv_bfloat16* out;
  float* state;             // kSol
  int num_query_tokens, num_kv_tokens, heads, total_heads, head_offset;
  float scale_log2;         // log2e / sqrt(128) x the global scales of Q and K
  float out_scale;          // global scale of V
  uint32_t* status;
};

// untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on an mbarrier
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// one 512-byte scale atom (32 rows x 16 bytes) -> 4 TMEM columns, replicated over the four lane quadrants
__device__ __forceinline__ void cp_scale_atom(uint32_t taddr, uint32_t smem_addr) {
  const uint64_t desc = umma_smem_desc(smem_addr, 16, 128, kSwizzleNone);
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}
// eight e2m1 codes (round to nearest even on the e2m1 grid, saturating): element i in bits 4i
__device__ __forceinline__ uint32_t pack_e2m1x8(const float* y) {
  uint32_t d;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(d)
      : "f"(y[0]), "f"(y[1]), "f"(y[2]), "f"(y[3]), "f"(y[4]), "f"(y[5]), "f"(y[6]), "f"(y[7]));
  return d;
}
// two ue4m3 bytes (round to nearest even, saturating at 448): `lo` in bits 0-7
__device__ __forceinline__ uint32_t pack_e4m3x2(float lo, float hi) {
  uint16_t d;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
  return d;
}

// block-scaled instruction descriptor: e2m1 x e2m1 (format 1 in bits 7-9 / 10-12), both K-major, N >> 3 in bits 17-22,
// ue4m3 scales (bit 23 clear), M >> 4 in bits 24-28, scale-factor ids 0
constexpr uint32_t idesc_for(uint32_t n) { return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24); }
constexpr uint32_t kIdesc = idesc_for(128);

template <bool kSol>
__global__ void __launch_bounds__(kThreads, 1)
fa_fwd_nvfp4_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const Params P) {
  extern __shared__ uint8_t smem_raw[];
  Shared& S = *reinterpret_cast<Shared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int q0 = blockIdx.x * (2 * kTile);
  const bool two = q0 + kTile < P.num_query_tokens;
  // Dense: a step is a key tile of 128.  Sol: a step is one 64-key routing block of the tile's list, so that no MMA,
  // load or exponential is spent on a neighbour block nobody selected; K and V still arrive as 128-key tiles that
  // start at the block's first token, and the block-scaled MMAs read their first 64 keys.
  constexpr int kKeys = kSol ? 64 : kTile;
  const int n_kv_total = (P.num_kv_tokens + kTile - 1) / kTile;
  const int q_row_blocks = (P.num_query_tokens + kTile - 1) / kTile;  // 128-row blocks of the padded operands
  volatile uint32_t* abort_flag = &S.abort;
  uint32_t* status = P.status;

  if (threadIdx.x == 0) {
    mbar_init(&S.q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&S.kv_full[s], 1);
      mbar_init(&S.kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&S.s_full[t], 1);
      mbar_init(&S.s_taken[t], 4);
      mbar_init(&S.p_full[t][0], 4);
      mbar_init(&S.p_full[t][1], 4);
      mbar_init(&S.pv_done[t], 1);
    }
    mbar_init(&S.list_ready, 1);
    S.abort = 0;
    S.qk_issued = 0;
    S.list_len[0] = S.list_len[1] = 0;
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

  // key tiles of query tile t: all of them (dense; both tiles share each K / V tile), or the tile's own list
  auto tile_count = [&](int t) { return kSol ? S.list_len[t] : n_kv_total; };
  auto tile_at = [&](int t, int i) { return kSol ? static_cast<int>(S.list[t][i]) : i; };
  auto wait_list = [&](uint32_t bit) -> bool {
    if (!kSol) return true;
    return __all_sync(0xffffffffu, mbar_wait(&S.list_ready, 0, abort_flag, status, bit));
  };

  if (warp >= 8) {
    reg_dealloc<kServiceRegs>();
    if (warp == kProducerWarp) {
      // ------------------------------------------------------------ TMA producer (and tile list)
      if (kSol) {
        const int q_blocks = (P.num_query_tokens + 63) / 64, k_blocks = (P.num_kv_tokens + 63) / 64;
        for (int t = 0; t < (two ? 2 : 1); ++t) {
          const int qb0 = q0 / 64 + 2 * t;
          int count = 0;
          for (int base = 0; base < k_blocks; base += 32) {
            const int kb = base + lane;
            uint32_t f = 0;
            if (kb < k_blocks) {
#pragma unroll
              for (int qi = 0; qi < 2; ++qi) {
                if (qb0 + qi >= q_blocks) continue;
                const uint8_t* row = P.selected + (static_cast<size_t>(qb0 + qi) * P.heads + head) * k_blocks;
                if (kb == 0 || row[kb] != 0) f |= 1u << qi;
              }
            }
            const uint32_t hit = __ballot_sync(0xffffffffu, f != 0);
            if (f != 0) {
              const int at = count + __popc(hit & ((1u << lane) - 1));
              if (NOB_CHECK(at < kMaxTiles, status) && at < kMaxTiles) {
                S.list[t][at] = static_cast<uint16_t>(kb);
                S.flags[t][at] = static_cast<uint8_t>(f);
              }
            }
            count += __popc(hit);
          }
          if (lane == 0) S.list_len[t] = count < kMaxTiles ? count : kMaxTiles;
        }
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          mbar_arrive(&S.list_ready);
        }
        __syncwarp();
      }
      if (lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        const int tiles_q = two ? 2 : 1;
        mbar_expect_tx(&S.q_full, tiles_q * (kTileBytes + kSfBytes));
        for (int t = 0; t < tiles_q; ++t) {
          tma_load_3d(S.q[t], &map_q, &S.q_full, 0, q0 + t * kTile, head);
          bulk_load(S.q_sf[t], P.q_sf + (static_cast<size_t>(head) * q_row_blocks + (q0 / kTile + t)) * kSfBytes, kSfBytes,
                    &S.q_full);
        }
        // dense: unit u = key tile u, read by both query tiles; sol: unit u = the u-th score group in issue order
        // (A(0), B(0), A(1), B(1), ... while both lists last, then the rest of the longer one), read by one tile
        const int n_a = tile_count(0), n_b = two ? tile_count(1) : 0;
        const int units = kSol ? n_a + n_b : n_a;
        int next[2] = {0, 0};
        int issued = 0;
        for (int u = 0; u < units; ++u) {
          int kt = u;
          if (kSol) {
            const int t = (next[0] < n_a && (next[0] <= next[1] || next[1] >= n_b)) ? 0 : 1;
            kt = tile_at(t, next[t]++);
          }
          bool ok = true;
          for (int part = 0; part < 2 && ok; ++part) {  // K at 2u, V at 2u+1
            const int i = 2 * u + part, st = i % kStages;
            if (i >= kStages) ok = mbar_wait(&S.kv_empty[st], ((i / kStages) - 1) & 1, abort_flag, status, kWaitTimeoutRing);
            if (!ok) break;
            if (kSol) {
              // kt is a 64-key block: data tiles from its first token on; K scales are the two atoms (channel halves)
              // of the 128-row tile it lies in, V scales the one atom of its four 16-token groups
              if (part) {
                mbar_expect_tx(&S.kv_full[st], kTileBytes + 512);
                tma_load_3d(S.kv[st], &map_v, &S.kv_full[st], kt * 32, 0, head);  // [channel][64 bytes from token 64 kt]
                bulk_load(S.kv_sf[st], P.v_sf + (static_cast<size_t>(head) * n_kv_total * 2 + kt) * 512, 512, &S.kv_full[st]);
              } else {
                mbar_expect_tx(&S.kv_full[st], kTileBytes + kSfBytes);
                tma_load_3d(S.kv[st], &map_k, &S.kv_full[st], 0, kt * 64, head);  // [token][64 bytes]
                bulk_load(S.kv_sf[st], P.k_sf + (static_cast<size_t>(head) * n_kv_total + (kt >> 1)) * kSfBytes, kSfBytes,
                          &S.kv_full[st]);
              }
            } else {
              mbar_expect_tx(&S.kv_full[st], kTileBytes + kSfBytes);
              if (part) {
                tma_load_3d(S.kv[st], &map_v, &S.kv_full[st], kt * 64, 0, head);  // [channel][64 bytes = 128 tokens]
                bulk_load(S.kv_sf[st], P.v_sf + (static_cast<size_t>(head) * n_kv_total + kt) * kSfBytes, kSfBytes, &S.kv_full[st]);
              } else {
                tma_load_3d(S.kv[st], &map_k, &S.kv_full[st], 0, kt * kTile, head);  // [token][64 bytes]
                bulk_load(S.kv_sf[st], P.k_sf + (static_cast<size_t>(head) * n_kv_total + kt) * kSfBytes, kSfBytes, &S.kv_full[st]);
              }
            }
            issued = i + 1;
          }
          if (!ok) break;
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
    } else if (warp == kMmaWarp || warp == kPvWarp) {
      // --------------------------------------------------------- tcgen05 issuers (whole warp, one elected lane issues)
      auto full_parity = [](int i) { return (uint32_t)((i / kStages) & 1); };
      auto spin = [&](uint64_t* bar, uint32_t parity, uint32_t bit) { return warp_poll(bar, parity, abort_flag, status, bit); };
      auto rest = [&](uint64_t* bar, uint32_t parity, uint32_t bit) { return warp_rest(bar, parity, abort_flag, status, bit); };
      const uint64_t desc = umma_smem_desc(0, 16, 512, kSwizzle64B);  // K-major, 64-byte rows, 8-row groups of 512 B
      bool ok = wait_list(kWaitTimeoutLoad);
      const int n_a = ok ? tile_count(0) : 0, n_b = (ok && two) ? tile_count(1) : 0;
      // Score groups in issue order.  Dense: A(0), B(0), A(1), ... on shared key tiles (ring unit = key tile).
      // Sol: the same interleaving while both lists last, then the rest of the longer one (ring unit = group).
      auto next_tile = [&](const int (&next)[2]) { return (next[0] < n_a && (next[0] <= next[1] || next[1] >= n_b)) ? 0 : 1; };
      const int groups = n_a + n_b;
      if (warp == kMmaWarp) {
        const uint64_t q_desc[2] = {desc + (smem_u32(S.q[0]) >> 4), desc + (smem_u32(S.q[1]) >> 4)};
        const uint64_t kv_desc = desc + (smem_u32(S.kv[0]) >> 4);
        uint32_t issued = 0;
        // S = Q_t K^T with the K tile of ring unit u; `first` reader waits for the tile and copies its scales,
        // `last` reader releases the stage
        // `block`: the 64-key block of a sol entry (its K scales are rows 64 (block & 1) .. of the tile's atoms: two
        // TMEM columns further on); 0 for dense
        auto qk = [&](int t, int u, bool first, bool last, uint64_t* taken, uint32_t taken_parity, int block) -> bool {
          const int ik = 2 * u, sk = ik % kStages;
          const uint64_t a0 = t ? q_desc[1] : q_desc[0], b0 = kv_desc + sk * (kTileBytes >> 4);
          if (first && !rest(&S.kv_full[sk], full_parity(ik), kWaitTimeoutLoad)) return false;
          if (taken && !spin(taken, taken_parity, kWaitTimeoutSoftmax)) return false;
          tc_fence_after();
          if (elect_one()) {
            if (first) {  // the key tile's scales, ahead of its first MMA (same pipe, in order)
              cp_scale_atom(tmem + kColSfK, smem_u32(S.kv_sf[sk]));
              cp_scale_atom(tmem + kColSfK + 4, smem_u32(S.kv_sf[sk]) + 512);
            }
            asm volatile(
                "{\n\t.reg .pred p0, p1;\n\t"
                "setp.ne.b32 p0, 0, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %2, %4, %1, [%6], [%8], p0;\n\t"
                "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %3, %5, %1, [%7], [%9], p1;\n\t}" ::"r"(
                    tmem + kColS),
                "r"(idesc_for(kKeys)), "l"(a0), "l"(a0 + 2), "l"(b0), "l"(b0 + 2), "r"(tmem + kColSfQ + 8 * t),
                "r"(tmem + kColSfQ + 8 * t + 4), "r"(tmem + kColSfK + 2 * (block & 1)),
                "r"(tmem + kColSfK + 4 + 2 * (block & 1))
                : "memory");
            tc_commit(&S.s_full[t]);
            if (last) tc_commit(&S.kv_empty[sk]);
            *reinterpret_cast<volatile uint32_t*>(&S.qk_issued) = issued + 1;
          }
          ++issued;
          return true;
        };
        ok = ok && groups > 0 && rest(&S.q_full, 0, kWaitTimeoutLoad);
        if (ok) {
          tc_fence_after();
          if (elect_one()) {
            for (int t = 0; t < (two ? 2 : 1); ++t) {
              cp_scale_atom(tmem + kColSfQ + 8 * t, smem_u32(S.q_sf[t]));
              cp_scale_atom(tmem + kColSfQ + 8 * t + 4, smem_u32(S.q_sf[t]) + 512);
            }
          }
        }
        if (kSol) {
          int next[2] = {0, 0}, prev_t = -1, prev_i = 0;
          for (int g = 0; ok && g < groups; ++g) {
            const int t = next_tile(next), i = next[t]++;
            ok = qk(t, g, true, true, prev_t < 0 ? nullptr : &S.s_taken[prev_t], prev_i & 1, tile_at(t, i));
            prev_t = t, prev_i = i;
          }
        } else {
          const bool shared = n_b > 0;
          ok = ok && qk(0, 0, true, !shared, nullptr, 0, 0);
          for (int i = 0; ok && i < n_a; ++i) {
            if (shared && !(ok = qk(1, i, false, true, &S.s_taken[0], i & 1, 0))) break;
            if (i + 1 < n_a && !(ok = qk(0, i + 1, true, !shared, &S.s_taken[shared ? 1 : 0], i & 1, 0))) break;
          }
        }
      } else {
        const uint64_t kv_desc = desc + (smem_u32(S.kv[0]) >> 4);
        // O_t += P_t(i)[:, 64 half ...] V[...] with the V tile of ring unit u: one MMA of K = 64, after `gate`
        // score groups were issued
        auto pv_half = [&](int t, int i, int u, int half, bool first, bool last, uint32_t gate) -> bool {
          const int iv = 2 * u + 1, sv = iv % kStages;
          const uint64_t b = kv_desc + sv * (kTileBytes >> 4) + half * 2;  // 64 keys = 32 bytes of a channel's row
          const uint32_t accumulate = (i > 0 || half > 0) ? 1u : 0u;
          if (gate > static_cast<uint32_t>(groups)) gate = groups;
          if (half == 0 && !rest(&S.kv_full[sv], full_parity(iv), kWaitTimeoutLoad)) return false;
          if (!NOB200_PFULL_WAIT(&S.p_full[t][half], i & 1, kWaitTimeoutSoftmax)) return false;
          if (!warp_wait_counter(&S.qk_issued, gate, abort_flag, status, kWaitTimeoutMma)) return false;
          tc_fence_after();
          if (elect_one()) {
            if (first && half == 0) {  // the value tile's scales, ahead of its first MMA
              cp_scale_atom(tmem + kColSfV, smem_u32(S.kv_sf[sv]));
              if (!kSol) cp_scale_atom(tmem + kColSfV + 4, smem_u32(S.kv_sf[sv]) + 512);
            }
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], [%1], %2, %3, [%5], [%6], p;\n\t}" ::"r"(
                    tmem + kColO + t * kTile),
                "r"(tmem + kColP + 16 * t + 8 * half), "l"(b), "r"(kIdesc), "r"(accumulate),
                "r"(tmem + kColSfP + 8 * t + 4 * half), "r"(tmem + kColSfV + 4 * half)
                : "memory");
            if (kSol || half == 1) {
              tc_commit(&S.pv_done[t]);
              if (last) tc_commit(&S.kv_empty[sv]);
            }
          }
          return true;
        };
        if (kSol) {
          // a group's value MMAs wait until the next score group is in the pipe (the one its score take released)
          int next[2] = {0, 0};
          for (int g = 0; ok && g < groups; ++g) {
            const int t = next_tile(next), i = next[t]++;
            ok = pv_half(t, i, g, 0, true, true, g + 2);  // an entry is 64 keys: one MMA
          }
        } else if (n_b > 0) {
          for (int i = 0; ok && i < n_a; ++i) {
            ok = pv_half(0, i, i, 0, true, false, 2 * i + 3) && pv_half(0, i, i, 1, true, false, 2 * i + 4) &&
                 pv_half(1, i, i, 0, false, true, 2 * i + 4) && pv_half(1, i, i, 1, false, true, 2 * i + 5);
          }
        } else {
          for (int i = 0; ok && i < n_a; ++i) ok = pv_half(0, i, i, 0, true, true, i + 2) && pv_half(0, i, i, 1, true, true, i + 2);
        }
      }
    }
  } else {
    // ------------------------------------------------- softmax + epilogue warps
    reg_alloc<kSoftmaxRegs>();
    auto poll = [&](uint64_t* bar, uint32_t parity, uint32_t bit) { return warp_poll(bar, parity, abort_flag, status, bit); };
    const int t = warp >> 2;
    if (t == 0 || two) {
      const int row = (warp & 3) * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t s_addr = tmem + lane_base + kColS;
      const uint32_t p_addr = tmem + lane_base + kColP + 16 * t;
      const uint32_t sf_addr = tmem + lane_base + kColSfP + 8 * t + (warp & 3);  // the row's lane quadrant reads this column
      const uint32_t o_addr = tmem + lane_base + kColO + t * kTile;
      const int quarter = (warp & 3) >> 1;  // 64-row query block inside the tile
      float m_run = -INFINITY;  // raw q.k units
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      bool ok = wait_list(kWaitTimeoutLoad);
      const int n = ok ? tile_count(t) : 0;
      for (int i = 0; i < n; ++i) {
        const int kt = tile_at(t, i);
        const bool selected = !kSol || ((S.flags[t][i] >> quarter) & 1u) != 0;
        ok = poll(&S.s_full[t], i & 1, kWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        uint32_t s[kKeys];
#pragma unroll
        for (int c = 0; c < kKeys / 32; ++c) tmem_ld32(s_addr + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&s[32 * c]));
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&S.s_taken[t]);
        // keys that do not exist or that this row's query block did not select count as -inf
        int hi = selected ? kKeys : 0;
        const int valid = P.num_kv_tokens - kt * kKeys;
        if (hi > valid) hi = valid;
        if (hi < kKeys) {
#pragma unroll
          for (int e = 0; e < kKeys; ++e)
            if (e >= hi) s[e] = 0xff800000u;
        }
        bool pv_waited = i == 0;
        uint32_t pw[kKeys / 8], sfw[kKeys / 64];
        if (hi <= 0) {
          // nothing of this tile for this warp's rows (uniform: a warp lies inside one query block)
#pragma unroll
          for (int c = 0; c < kKeys / 8; ++c) pw[c] = 0u;
#pragma unroll
          for (int c = 0; c < kKeys / 64; ++c) sfw[c] = 0u;
        } else {
          float mx0 = __uint_as_float(s[0]), mx1 = __uint_as_float(s[1]);
          float mx2 = __uint_as_float(s[2]), mx3 = __uint_as_float(s[3]);
#pragma unroll
          for (int e = 4; e < kKeys - 4; e += 8) {
            mx0 = max3(mx0, __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
            mx1 = max3(mx1, __uint_as_float(s[e + 2]), __uint_as_float(s[e + 3]));
            mx2 = max3(mx2, __uint_as_float(s[e + 4]), __uint_as_float(s[e + 5]));
            mx3 = max3(mx3, __uint_as_float(s[e + 6]), __uint_as_float(s[e + 7]));
          }
          mx0 = max3(mx0, __uint_as_float(s[kKeys - 4]), __uint_as_float(s[kKeys - 3]));
          mx1 = max3(mx1, __uint_as_float(s[kKeys - 2]), __uint_as_float(s[kKeys - 1]));
          const float m_new = fmaxf(m_run, fmaxf(max3(mx0, mx1, mx2), mx3));
          if (i > 0 && __any_sync(0xffffffffu, m_new > m_run)) {
            // exact running maximum: the accumulated numerator and sum move to the new reference
            const float alpha = ex2((m_run - m_new) * P.scale_log2);
            l0 *= alpha, l1 *= alpha, l2 *= alpha, l3 *= alpha;
            ok = poll(&S.pv_done[t], (i - 1) & 1, kWaitTimeoutMma);
            if (!ok) break;
            pv_waited = true;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tmem_ld32(o_addr + 32 * c, o);
              tc_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
              tmem_st32(o_addr + 32 * c, o);
            }
            tc_wait_st();
          }
          m_run = m_new;
          const float bias = kLog2PScale - m_run * P.scale_log2;
          const uint64_t scale2 = pack2(P.scale_log2, P.scale_log2), bias2 = pack2(bias, bias);
          uint64_t la = pack2(l0, l1), lb = pack2(l2, l3);
#pragma unroll
          for (int g = 0; g < kKeys / 16; ++g) {
            float p[16];
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              float x0, x1;
              unpack2(fma2(pack2(__uint_as_float(s[16 * g + e]), __uint_as_float(s[16 * g + e + 1])), scale2, bias2), x0, x1);
              p[e] = ex2(x0);
              p[e + 1] = ex2(x1);
            }
#pragma unroll
            for (int e = 0; e < 16; e += 4) {
              la = add2(la, pack2(p[e], p[e + 1]));
              lb = add2(lb, pack2(p[e + 2], p[e + 3]));
            }
            float a0 = max3(p[0], p[1], p[2]), a1 = max3(p[3], p[4], p[5]), a2 = max3(p[6], p[7], p[8]);
            float a3 = max3(p[9], p[10], p[11]), a4 = max3(p[12], p[13], p[14]);
            const float gmax = fmaxf(max3(a0, a1, a2), max3(a3, a4, p[15]));
            // block scale max/6 (at most 448 because p <= 2688), the codes are p over the unrounded scale.  The
            // reciprocal is the MUFU approximation (1 ulp): it moves a code only when p / scale sits within an ulp
            // of a rounding boundary of the e2m1 grid.
            const float bs = gmax * (1.0f / 6.0f);
            float inv;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(bs));
            inv = bs > 0.f ? inv : 0.f;
            const uint64_t inv2 = pack2(inv, inv);
#pragma unroll
            for (int e = 0; e < 16; e += 2) unpack2(mul2(pack2(p[e], p[e + 1]), inv2), p[e], p[e + 1]);
            pw[2 * g] = pack_e2m1x8(p);
            pw[2 * g + 1] = pack_e2m1x8(p + 8);
            const uint32_t byte = pack_e4m3x2(bs, 0.f) & 0xffu;
            if ((g & 3) == 0) sfw[g >> 2] = 0u;
            sfw[g >> 2] |= byte << (8 * (g & 3));
          }
          unpack2(la, l0, l1);
          unpack2(lb, l2, l3);
        }
        if (!pv_waited) {
          // the previous tile's value MMAs still read P_t and its scales until this completes
          ok = poll(&S.pv_done[t], (i - 1) & 1, kWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
        }
#pragma unroll
        for (int half = 0; half < kKeys / 64; ++half) {
          tmem_st8(p_addr + 8 * half, pw + 8 * half);
          tmem_st1(sf_addr + 4 * half, sfw[half]);
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&S.p_full[t][half]);
        }
      }
      if (ok && n > 0) ok = poll(&S.pv_done[t], (n - 1) & 1, kWaitTimeoutMma);
      if (ok && n > 0) {
        tc_fence_after();
        const float l = (l0 + l1) + (l2 + l3);
        const int token = q0 + t * kTile + row;
        const bool store = token < P.num_query_tokens && NOB_CHECK(head + P.head_offset < P.total_heads, status);
        const size_t at = (static_cast<size_t>(store ? token : 0) * P.total_heads + head + P.head_offset);
        __nv_bfloat16* dst = P.out + at * 128;
        float factor;
        if (kSol) {
          factor = kInvPScale * P.out_scale;
          if (store) {
            P.state[at * 2] = m_run;
            P.state[at * 2 + 1] = l * kInvPScale;
          }
        } else {
          factor = P.out_scale / l;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + 32 * c, o);
          tc_wait_ld();
          if (store) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(o[e]) * factor, __uint_as_float(o[e + 1]) * factor);
              v.y = pack_bf16(__uint_as_float(o[e + 2]) * factor, __uint_as_float(o[e + 3]) * factor);
              v.z = pack_bf16(__uint_as_float(o[e + 4]) * factor, __uint_as_float(o[e + 5]) * factor);
              v.w = pack_bf16(__uint_as_float(o[e + 6]) * factor, __uint_as_float(o[e + 7]) * factor);
              *reinterpret_cast<uint4*>(dst + 32 * c + e) = v;
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

int launch_nvfp4(bool sol, const char* name, int num_query_tokens, int num_kv_tokens, int head_offset, const void* query,
                 const void* key, const void* value, const void* query_scales, const void* key_scales,
                 const void* value_scales, float query_global, float key_global, float value_global,
                 const void* selected, void* output, void* state, int heads, int total_heads, void* stream) {
  NOB_REQUIRE(num_query_tokens > 0 && num_kv_tokens > 0 && heads > 0 && total_heads > 0, "%s: sizes must be positive", name);
  NOB_REQUIRE(head_offset >= 0 && head_offset <= total_heads - heads, "%s: head_offset %d outside [0, %d]", name,
              head_offset, total_heads - heads);
  NOB_REQUIRE(query && key && value && query_scales && key_scales && value_scales && output, "%s: NULL tensor", name);
  NOB_REQUIRE(!sol || (selected && state), "%s: NULL mask or state", name);
  NOB_REQUIRE(heads <= 65535, "%s: heads %d exceeds grid limit", name, heads);
  NOB_REQUIRE(query_global > 0.f && key_global > 0.f && value_global > 0.f, "%s: global scales must be positive", name);
  NOB_REQUIRE(!sol || (num_kv_tokens + 63) / 64 <= kMaxTiles, "%s: %d key tokens exceed the %d this kernel lists", name,
              num_kv_tokens, kMaxTiles * 64);
  uint32_t* status = status_word_device_ptr();
  if (!status) return fail(kCudaError, "%s: no current CUDA device", name);
  const uint64_t q_rows = (static_cast<uint64_t>(num_query_tokens) + 127) / 128 * 128;
  const uint64_t k_rows = (static_cast<uint64_t>(num_kv_tokens) + 127) / 128 * 128;

  CUtensorMap mq, mk, mv;
  int rc;
  // Q, K: [heads][rows][64 bytes]; V: [heads][128 channels][k_rows / 2 bytes]
  if ((rc = make_tensor_map_3d(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, query, 64, q_rows, heads, 64, q_rows * 64, 64, kTile, 1,
                               CU_TENSOR_MAP_SWIZZLE_64B)))
    return rc;
  if ((rc = make_tensor_map_3d(&mk, CU_TENSOR_MAP_DATA_TYPE_UINT8, key, 64, k_rows, heads, 64, k_rows * 64, 64, kTile, 1,
                               CU_TENSOR_MAP_SWIZZLE_64B)))
    return rc;
  if ((rc = make_tensor_map_3d(&mv, CU_TENSOR_MAP_DATA_TYPE_UINT8, value, k_rows / 2, 128, heads, k_rows / 2,
                               k_rows / 2 * 128, 64, kTile, 1, CU_TENSOR_MAP_SWIZZLE_64B)))
    return rc;

  Params params = {};
  params.q_sf = static_cast<const uint8_t*>(query_scales);
  params.k_sf = static_cast<const uint8_t*>(key_scales);
  params.v_sf = static_cast<const uint8_t*>(value_scales);
  params.selected = static_cast<const uint8_t*>(selected);
  params.out = static_cast<__nv_bfloat16*>(output);
  params.state = static_cast<float*>(state);
  params.num_query_tokens = num_query_tokens, params.num_kv_tokens = num_kv_tokens;
  params.heads = heads, params.total_heads = total_heads, params.head_offset = head_offset;
  params.scale_log2 = 0.08838834764831845f * 1.4426950408889634f * query_global * key_global;
  params.out_scale = value_global;
  params.status = status;

  const size_t smem = sizeof(Shared) + 1024;
  auto kernel = sol ? fa_fwd_nvfp4_kernel<true> : fa_fwd_nvfp4_kernel<false>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess)
    return fail(kCudaError, "%s: cannot reserve %zu B of shared memory: %s", name, smem, cudaGetErrorString(err));
  dim3 grid((num_query_tokens + 2 * kTile - 1) / (2 * kTile), heads);
  kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, params);
  return check_launch(name);
}

}  // namespace
}  // namespace nob200

using namespace nob200;

extern "C" size_t nob200_dense_nvfp4_attention_d128_workspace_bytes(int, int, int) { return 0; }
extern "C" size_t nob200_sol_nvfp4_attention_d128_workspace_bytes(int, int, int) { return 0; }

extern "C" int nob200_dense_nvfp4_attention_d128(int num_query_tokens, int num_kv_tokens, int head_offset,
                                                 const void* query, const void* key, const void* value,
                                                 const void* query_scales, const void* key_scales,
                                                 const void* value_scales, void* output, int heads, int total_heads,
                                                 void* workspace, size_t workspace_bytes, void* stream) {
  (void)workspace, (void)workspace_bytes;
  return launch_nvfp4(false, "dense_nvfp4_attention_d128", num_query_tokens, num_kv_tokens, head_offset, query, key, value,
                      query_scales, key_scales, value_scales, 1.0f, 1.0f, 1.0f, nullptr, output, nullptr, heads,
                      total_heads, stream);
}

extern "C" int nob200_dense_nvfp4_attention_d128_global(int num_query_tokens, int num_kv_tokens, int head_offset,
                                                        const void* query, const void* key, const void* value,
                                                        const void* query_scales, const void* key_scales,
                                                        const void* value_scales, float query_global, float key_global,
                                                        float value_global, void* output, int heads, int total_heads,
                                                        void* workspace, size_t workspace_bytes, void* stream) {
  (void)workspace, (void)workspace_bytes;
  return launch_nvfp4(false, "dense_nvfp4_attention_d128", num_query_tokens, num_kv_tokens, head_offset, query, key, value,
                      query_scales, key_scales, value_scales, query_global, key_global, value_global, nullptr, output,
                      nullptr, heads, total_heads, stream);
}

extern "C" int nob200_sol_nvfp4_attention_d128(int num_query_tokens, int num_kv_tokens, int head_offset,
                                               const void* query, const void* key, const void* value,
                                               const void* query_scales, const void* key_scales,
                                               const void* value_scales, const void* selected, void* output,
                                               void* state, int heads, int total_heads, void* workspace,
                                               size_t workspace_bytes, void* stream) {
  (void)workspace, (void)workspace_bytes;
  return launch_nvfp4(true, "sol_nvfp4_attention_d128", num_query_tokens, num_kv_tokens, head_offset, query, key, value,
                      query_scales, key_scales, value_scales, 1.0f, 1.0f, 1.0f, selected, output, state, heads,
                      total_heads, stream);
}
