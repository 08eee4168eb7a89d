// Exact stage of the int8-fp8 "sol" block-sparse attention for head_dim 128 on sm_100a.
//
// Replaces the reference program sol_int8_fp8_attention_d128
// (src/nano_omni/kernels/attention/int8_fp8/sol.py:27-225).  For every 64-row query block qb and head h only the
// 64-key blocks with selected[qb, h, kb] != 0 attend.  Nothing is normalised here: the kernel writes
//   output[token, head_offset + h, :] = sum_k p_k * v_k            (bf16; p relative to the row maximum)
//   state[token, head_offset + h]     = (row maximum in raw dequantised q.k units, sum_k p_k)
// with p_k = exp((q.k - max) / sqrt(128)); the finalize step (fa_fwd_sol_bf16.cu, kFinalize) merges the pooled
// pseudo-keys of the unselected blocks and divides.
//
// Arithmetic is that of the dense int8-fp8 kernel (fa_fwd_i8f8.cu): int8 QK with kind::i8, probabilities rounded
// to e4m3 into TMEM, PV with kind::f8f6f4.  One CTA owns 128 query rows (two query blocks) of one head.  The producer
// builds the list of 64-key blocks that one of the two query blocks selects, with a flag per query block: a list
// entry is one routing block, so no MMA or load is spent on a neighbour block that nobody selected (with 16 % of the
// blocks selected, 31 % of the 64-key blocks are on a CTA's list, against 52 % of the 128-key tiles).  The entries
// are dealt alternately to two streams, each a complete online softmax with its own accumulator in TMEM, run by one
// softmax warpgroup and fed by one issuing warp; the epilogue merges the two partial results.  Each stream has TWO
// score buffers of 64 columns
// (2 x 2 x 64 + 2 x 128 = 512 TMEM columns): the scores of the stream's next entry are computed while the softmax
// warps work on the current one, so a stream's pace is its softmax, not the chain P stored -> PV -> QK -> scores
// complete.  A softmax warp whose query block did not select an entry's key block neither loads nor exponentiates it
// (it stores zero probabilities).  K and V arrive as 128-row tiles starting at the entry's first token; the MMAs read
// the first 64 keys of them.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "fa_common.cuh"
#include "tensor_map.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

constexpr int kTile = 128;
constexpr int kTileBytes = kTile * 128;  // 16 KiB: 128 rows of 128 one-byte elements
constexpr int kStages = 8;
constexpr int kThreads = 384;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr float kHeadroomLog2 = 3.0f;              // P <= 448 while the stale maximum lags by <= 2^3
constexpr float kLog2PScale = 8.807354922057604f - kHeadroomLog2;  // log2(448) - 3
constexpr uint32_t kMagicBits = 0x4B400000u;       // 12582912.0f
constexpr float kMagic = 12582912.0f;
constexpr int kBlock = 64;       // routing block of the reference path: one list entry, one MMA group
constexpr int kMaxBlocks = 4096; // key blocks a CTA can list: up to 262144 tokens
constexpr int kAhead = 4;        // entries whose scores are in flight: two per stream (the stream's two score buffers)

struct __align__(1024) Shared {
  uint8_t q[kTileBytes];
  uint8_t kv[kStages][kTileBytes];
  uint16_t block_list[kMaxBlocks];
  uint8_t block_flags[kMaxBlocks];  // bit u: query block u of the CTA selected the key block
  float4 merge[2][kTile];         // per stream and row: (maximum used, sum, raw maximum, stream has a result)
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2][2];  // [stream][score buffer]
  uint64_t p_full[2][2];
  uint64_t pv_done[2];    // the stream's latest value MMAs are complete (for the rare rescale of O)
  uint64_t o_final[2];
  uint64_t list_ready;
  uint64_t merge_ready;
  int num_exact;
  uint32_t tmem_base;
  uint32_t abort;
};

static_assert(256 * 224 + 128 * 56 <= 384 * 168, "setmaxnreg split exceeds the registers the CTA owns");

// two e4m3 bytes: `lo` in bits 0-7, `hi` in bits 8-15
__device__ __forceinline__ uint32_t pack_e4m3(float lo, float hi) {
  uint16_t d;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
  return d;
}

struct SolI8Params {
  const float* query_scale;  // [heads, ceil(T/32)]
  const float* key_scale;    // [heads, ceil(T/64)]
  const float* value_scale;  // [heads, 128]
  const uint8_t* selected;   // [blocks, heads, blocks]
  __nv_bfloat16* out;        // [T, total_heads, 128]
  float* state;              // [T, total_heads, 2]
  int num_tokens, heads, total_heads, head_offset, num_blocks;
  float scale_log2;
  uint32_t* status;
};

__global__ void __launch_bounds__(kThreads, 1)
fa_fwd_sol_i8f8_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const SolI8Params P) {
  extern __shared__ uint8_t smem_raw[];
  Shared& S = *reinterpret_cast<Shared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int q0 = blockIdx.x * kTile;
  const int num_tokens = P.num_tokens;
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
      for (int b = 0; b < 2; ++b) {
        mbar_init(&S.s_full[t][b], 1);
        mbar_init(&S.p_full[t][b], 4);
      }
      mbar_init(&S.pv_done[t], 1);
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

  if (warp >= 8) {
    reg_dealloc<56>();
    if (warp == kProducerWarp) {
      // ---------------------------------------------- block list, then TMA producer
      // The list holds every 64-key block that one of the CTA's two query blocks selects, with a flag per query
      // block.  Every lane looks at 8 consecutive key blocks per round, their mask bytes in flight at once; a warp
      // scan keeps the list in ascending order.
      const int qb_first = q0 / kBlock;
      int count = 0;
      constexpr int kPerLane = 8;
      for (int base = 0; base < P.num_blocks; base += 32 * kPerLane) {
        const int kb0 = base + kPerLane * lane;
        uint32_t flags[kPerLane];
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) flags[i] = 0;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int qb = qb_first + u;
          if (qb >= P.num_blocks) continue;
          const uint8_t* row = P.selected + qb * mask_row_stride + static_cast<size_t>(head) * P.num_blocks;
#pragma unroll
          for (int i = 0; i < kPerLane; ++i)
            if (kb0 + i < P.num_blocks && row[kb0 + i]) flags[i] |= 1u << u;
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
            if (NOB_CHECK(at >= 0 && at < kMaxBlocks, status)) {
              S.block_list[at] = static_cast<uint16_t>(kb0 + i);
              S.block_flags[at] = static_cast<uint8_t>(flags[i]);
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
        mbar_expect_tx(&S.q_full, kTileBytes);
        tma_load_3d(S.q, &map_q, &S.q_full, 0, q0, head);
        // The issuer consumes K(0) .. K(kAhead - 1), then for every entry j: V(j) followed by K(j + kAhead).  A tile of
        // 128 rows is loaded from the entry's first token on; the MMAs read its first 64 keys.
        int issued = 0;
        auto load = [&](int j, int is_v) -> bool {
          const int st = issued % kStages;
          if (issued >= kStages) {
            if (!mbar_wait(&S.kv_empty[st], ((issued / kStages) - 1) & 1, abort_flag, status, kWaitTimeoutRing)) return false;
          }
          mbar_expect_tx(&S.kv_full[st], kTileBytes);
          const int tok = S.block_list[j] * kBlock;
          if (is_v) {
            tma_load_3d(S.kv[st], &map_v, &S.kv_full[st], tok, 0, head);  // [channel][token] tile
          } else {
            tma_load_3d(S.kv[st], &map_k, &S.kv_full[st], 0, tok, head);  // [token][channel] tile
          }
          ++issued;
          return true;
        };
        bool fed = true;
        for (int j = 0; fed && j < kAhead && j < count; ++j) fed = load(j, 0);
        for (int j = 0; fed && j < count; ++j) {
          fed = load(j, 1);
          if (fed && j + kAhead < count) fed = load(j + kAhead, 0);
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
    } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
      // ---------------------------------------------------------- tcgen05 issuer
      // All 32 lanes run the warp-uniform control flow; one elected lane issues (see elect_one()).  The waits on the
      // probabilities are on every entry's chain (P stored -> PV -> next QK of the stream -> scores complete) and
      // poll; K / V tiles were loaded long before and their waits may sleep.
      {
        constexpr uint32_t idesc_qk = umma_idesc(kDS32, kFmtS8, kFmtS8, 0, 0, kTile, kBlock);
        constexpr uint32_t idesc_pv = umma_idesc(kDF32, kFmtE4M3, kFmtE4M3, 0, 0, kTile, 128);
        const uint64_t desc = umma_smem_desc(0, 16, 1024, kSwizzle128B);
        const uint64_t q_desc = desc + (smem_u32(S.q) >> 4);
        const uint64_t kv_desc = desc + (smem_u32(S.kv[0]) >> 4);
        // S_t[buffer] = Q K^T for the 64 keys of an entry (the first 64 rows of the loaded tile): four MMAs of 32
        // channels (32 bytes of a row = 2 descriptor units), then the commits
        auto issue_qk = [&](int t, int buffer, int st) {
          const uint64_t a = q_desc, b = kv_desc + st * (kTileBytes >> 4);
          const uint32_t d = tmem + t * kTile + buffer * kBlock;
          if (elect_one()) {
            asm volatile(
                "{\n\t.reg .pred p0, p1;\n\t"
                "setp.ne.b32 p0, 0, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %2, %6, %1, p0;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %3, %7, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %4, %8, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %5, %9, %1, p1;\n\t}" ::"r"(d),
                "r"(idesc_qk), "l"(a), "l"(a + 2), "l"(a + 4), "l"(a + 6), "l"(b), "l"(b + 2), "l"(b + 4), "l"(b + 6)
                : "memory");
            tc_commit(&S.s_full[t][buffer]);
            tc_commit(&S.kv_empty[st]);
          }
        };
        // O_t += P_t[buffer] V for the entry's 64 keys (the first 64 bytes of every channel row of the loaded tile):
        // two MMAs of 32 keys (8 TMEM columns of P each), then the commits
        auto issue_pv = [&](int t, int buffer, int st, bool accumulate) {
          const uint64_t b = kv_desc + st * (kTileBytes >> 4);
          const uint32_t d = tmem + 256 + t * kTile, a = tmem + t * kTile + buffer * kBlock;
          if (elect_one()) {
            asm volatile(
                "{\n\t.reg .pred p0, p1;\n\t"
                "setp.ne.b32 p0, %2, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%3], %5, %1, p0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%4], %6, %1, p1;\n\t}" ::"r"(d),
                "r"(idesc_pv), "r"(accumulate ? 1u : 0u), "r"(a), "r"(a + 8), "l"(b), "l"(b + 2)
                : "memory");
            tc_commit(&S.pv_done[t]);
            tc_commit(&S.kv_empty[st]);
          }
        };
        // One issuing warp per stream: with 64-key entries the issue of an entry's six MMAs and four commits is what
        // paces the kernel, and each warp carries half of it.  The producer issues its loads in the order K_0 ..
        // K_{kAhead-1}, then V_j and K_{j+kAhead} for every entry j; a warp takes the loads of its own entries by
        // their place in that order.
        const int t = warp - kMmaWarp;
        bool ok = warp_rest(&S.list_ready, 0, abort_flag, status, kWaitTimeoutLoad);
        const int n_it = ok ? S.num_exact : 0;
        ok = ok && warp_rest(&S.q_full, 0, abort_flag, status, kWaitTimeoutLoad);
        const int first_loads = n_it < kAhead ? n_it : kAhead;  // K tiles loaded ahead of the first V tile
        const int keys_end = n_it > kAhead ? n_it - kAhead : 0;  // entries from here on are not followed by a K load
        auto stage_of = [&](int load) -> int {  // waits for load number `load` of the producer's order
          const int st = load % kStages;
          if (!warp_rest(&S.kv_full[st], (load / kStages) & 1, abort_flag, status, kWaitTimeoutLoad)) return -1;
          return st;
        };
        auto value_load = [&](int j) { return first_loads + 2 * j - (j > keys_end ? j - keys_end : 0); };
        auto key_load = [&](int j) { return j < kAhead ? j : first_loads + 2 * (j - kAhead) + 1; };
        // Entry j belongs to stream j & 1, is that stream's (j >> 1)-th entry and uses its score buffer (j >> 1) & 1.
        // The scores of the first entry of each buffer go out at once; from then on the scores of entry j + kAhead
        // follow the value MMAs of entry j into the buffer those have just read, so the softmax warps of a stream
        // always find the next entry's scores waiting in the other buffer.
        for (int j = t; ok && j < kAhead && j < n_it; j += 2) {
          const int st = stage_of(key_load(j));
          ok = st >= 0;
          if (!ok) break;
          tc_fence_after();
          issue_qk(t, (j >> 1) & 1, st);
        }
        for (int j = t; ok && j < n_it; j += 2) {
          const int e = j >> 1, buffer = e & 1;
          const int sv = stage_of(value_load(j));
          ok = sv >= 0;
          if (!ok) break;
          int sk = -1;
          if (j + kAhead < n_it) {
            sk = stage_of(key_load(j + kAhead));
            ok = sk >= 0;
            if (!ok) break;
          }
          if (!(ok = warp_poll(&S.p_full[t][buffer], (e >> 1) & 1, abort_flag, status, kWaitTimeoutSoftmax))) break;
          tc_fence_after();
          issue_pv(t, buffer, sv, e > 0);
          if (sk >= 0) issue_qk(t, buffer, sk);  // in order behind the PV that read this buffer
        }
        if (ok && elect_one()) tc_commit(&S.o_final[t]);
      }
    }
  } else {
    // ------------------------------------------------- softmax + epilogue warps
    reg_alloc<224>();
    const int t = warp >> 2;  // warpgroup t runs stream t
    {
      const int row = (warp & 3) * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t s_addr = tmem + lane_base + t * kTile;
      const uint32_t o_addr = tmem + lane_base + 256 + t * kTile;
      const int token = q0 + row;
      const int u = row >> 6;  // query block inside the tile; all 32 rows of a warp share it
      const int q_blocks = (num_tokens + 31) / 32, k_blocks = P.num_blocks;
      const float qs = P.query_scale[static_cast<size_t>(head) * q_blocks + min(token >> 5, q_blocks - 1)];
      const float* ks_head = P.key_scale + static_cast<size_t>(head) * k_blocks;
      const float scale_log2 = P.scale_log2;
      float m_used = -INFINITY, m_raw = -INFINITY;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      int done = 0;
      bool ok = __all_sync(0xffffffffu, mbar_wait(&S.list_ready, 0, abort_flag, status, kWaitTimeoutLoad));
      const int num_exact = ok ? S.num_exact : 0;
      for (int j = t; ok && j < num_exact; j += 2) {
        const int buffer = done & 1;  // the stream's entries alternate between its two score buffers
        const bool mine = (S.block_flags[j] >> u) & 1u;
        const int kb = S.block_list[j];
        // keys of the entry that count for this row: none when its query block did not select the key block
        const int n = mine ? min(kBlock, num_tokens - kb * kBlock) : 0;
        const float ks = ks_head[kb];  // fetched before the wait so that its latency hides behind it
        ok = warp_poll(&S.s_full[t][buffer], (done >> 1) & 1, abort_flag, status, kWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        uint32_t p[16];
        if (n == 0) {
          // neither loaded nor exponentiated (rows of a warp share the decision): zero probabilities
#pragma unroll
          for (int i = 0; i < 16; ++i) p[i] = 0u;
        } else {
          const float r = qs * ks, f = r * scale_log2;  // raw (dequantisation) and log2-domain factor
          uint32_t s[kBlock];
          tmem_ld32(s_addr + buffer * kBlock, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
          tmem_ld32(s_addr + buffer * kBlock + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < kBlock; ++i) s[i] += kMagicBits;  // int32 -> the float 2^23*1.5 + S
          float a = __uint_as_float(s[0]);
          if (n == kBlock) {
            float a1 = __uint_as_float(s[1]);
#pragma unroll
            for (int i = 2; i < 62; i += 4) {
              a = max3(a, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
              a1 = max3(a1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
            }
            a = fmaxf(max3(a, __uint_as_float(s[62]), __uint_as_float(s[63])), a1);
          } else {
#pragma unroll
            for (int i = 1; i < kBlock; ++i)
              if (i < n) a = fmaxf(a, __uint_as_float(s[i]));
          }
          const float mx = (a - kMagic) * f;
          m_raw = fmaxf(m_raw, (a - kMagic) * r);
          if (done == 0) {
            m_used = mx;  // O is overwritten by the stream's first PV; nothing to rescale
          } else if (__any_sync(0xffffffffu, mx > m_used + kHeadroomLog2)) {
            const float m_new = fmaxf(m_used, mx);
            const float alpha = (m_new == -INFINITY) ? 1.0f : ex2(m_used - m_new);  // 0 when the row had no key yet
            l0 *= alpha, l1 *= alpha, l2 *= alpha, l3 *= alpha;
            // O_t must hold every product issued so far; the latest is the previous entry's, and the next waits for
            // our arrival on p_full
            ok = warp_poll(&S.pv_done[t], (done - 1) & 1, abort_flag, status, kWaitTimeoutMma);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              uint32_t o[32];
              tmem_ld32(o_addr + 32 * cc, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(o_addr + 32 * cc, o);
            }
            tc_wait_st();
            m_used = m_new;
          }
          // x = ((2^23*1.5 + S) - 2^23*1.5) * f - (m - log2(448/8)).  The subtraction is exact; folding 2^23*1.5 * f
          // into the constant instead rounds it to that product's ulp, so that is only done for small factors.
          const float cst = m_used - kLog2PScale;
          if (n == kBlock) {
            uint64_t la = pack2(l0, l1), lb = pack2(l2, l3);
            auto exponentials = [&](auto fold_tag) {
              constexpr bool kFold = decltype(fold_tag)::value;
              const float c = kFold ? fmaf(kMagic, f, cst) : cst;
              const uint64_t f2 = pack2(f, f), nc2 = pack2(-c, -c), nm2 = pack2(-kMagic, -kMagic);
#pragma unroll
              for (int g = 0; g < 4; ++g) {  // groups of 16 keys; stored order inside a group: 0,1,8,9 | 2,3,10,11 | ...
                float e[16];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                  float x0, x1;
                  uint64_t sv = pack2(__uint_as_float(s[16 * g + i]), __uint_as_float(s[16 * g + i + 1]));
                  if (!kFold) sv = add2(sv, nm2);
                  unpack2(fma2(sv, f2, nc2), x0, x1);
                  e[i] = ex2(x0);
                  e[i + 1] = ex2(x1);
                }
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                  la = add2(la, pack2(e[i], e[i + 1]));
                  lb = add2(lb, pack2(e[i + 2], e[i + 3]));
                }
#pragma unroll
                for (int w = 0; w < 4; ++w)
                  p[4 * g + w] = pack_e4m3(e[2 * w], e[2 * w + 1]) | (pack_e4m3(e[8 + 2 * w], e[8 + 2 * w + 1]) << 16);
              }
            };
            if (f * kMagic < 16384.0f) {
              exponentials(std::true_type{});
            } else {
              exponentials(std::false_type{});
            }
            unpack2(la, l0, l1);
            unpack2(lb, l2, l3);
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float e[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                float x = fmaf(__uint_as_float(s[16 * g + i]) - kMagic, f, -cst);
                if (16 * g + i >= n) x = -INFINITY;
                e[i] = ex2(x);
              }
#pragma unroll
              for (int i = 0; i < 16; i += 4) {
                l0 += e[i], l1 += e[i + 1], l2 += e[i + 2], l3 += e[i + 3];
              }
#pragma unroll
              for (int w = 0; w < 4; ++w)
                p[4 * g + w] = pack_e4m3(e[2 * w], e[2 * w + 1]) | (pack_e4m3(e[8 + 2 * w], e[8 + 2 * w + 1]) << 16);
            }
          }
        }
        if (!ok) break;
        tmem_st16(s_addr + buffer * kBlock, p);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&S.p_full[t][buffer]);
        ++done;
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&S.o_final[t], 0, abort_flag, status, kWaitTimeoutMma));
      if (ok) {
        // ---- merge of the two streams; this warpgroup writes channels [64 t, 64 t + 64) of every row
        tc_fence_after();
        S.merge[t][row] = make_float4(m_used, (l0 + l1) + (l2 + l3), m_raw, done > 0 ? 1.0f : 0.0f);
        __syncwarp();
        if (lane == 0) mbar_arrive(&S.merge_ready);  // release: the other warpgroup sees the row's entry
        ok = __all_sync(0xffffffffu, mbar_wait(&S.merge_ready, 0, abort_flag, status, kWaitTimeoutSoftmax));
        tc_fence_after();  // the other stream's accumulator was completed by the other issuing warp
      }
      if (ok) {
        const float4 mine4 = S.merge[t][row], other4 = S.merge[t ^ 1][row];
        // numerator and sum in units of probabilities relative to the true maximum of the row
        const float top_raw = fmaxf(mine4.z, other4.z);
        const float top = top_raw * scale_log2 + kLog2PScale;
        const float g_mine = (mine4.w != 0.f && mine4.x != -INFINITY && top_raw != -INFINITY) ? ex2(mine4.x - top) : 0.f;
        const float g_other = (other4.w != 0.f && other4.x != -INFINITY && top_raw != -INFINITY) ? ex2(other4.x - top) : 0.f;
        const float* vs = P.value_scale + head * 128 + 64 * t;
        const size_t at = static_cast<size_t>(token < num_tokens ? token : 0) * P.total_heads + head + P.head_offset;
        __nv_bfloat16* dst = P.out + at * 128 + 64 * t;
        const bool store = token < num_tokens && NOB_CHECK(head + P.head_offset < P.total_heads, status);
        if (t == 0 && store)
          *reinterpret_cast<float2*>(P.state + 2 * at) = make_float2(top_raw, mine4.y * g_mine + other4.y * g_other);
        const uint32_t mine_addr = tmem + lane_base + 256 + t * kTile + 64 * t;
        const uint32_t other_addr = tmem + lane_base + 256 + (t ^ 1) * kTile + 64 * t;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t a[32], b[32];
          tmem_ld32(mine_addr + 32 * cc, a);
          tmem_ld32(other_addr + 32 * cc, b);
          tc_wait_ld();
          if (store) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              float r[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                // an accumulator that was never written holds arbitrary bits: select, do not multiply by zero
                const float x = g_mine != 0.f ? __uint_as_float(a[i + k]) * g_mine : 0.f;
                const float y = g_other != 0.f ? __uint_as_float(b[i + k]) * g_other : 0.f;
                r[k] = (x + y) * vs[32 * cc + i + k];
              }
              uint4 v;
              v.x = pack_bf16(r[0], r[1]);
              v.y = pack_bf16(r[2], r[3]);
              v.z = pack_bf16(r[4], r[5]);
              v.w = pack_bf16(r[6], r[7]);
              *reinterpret_cast<uint4*>(dst + 32 * cc + i) = v;
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

extern "C" int nob200_sol_int8_fp8_attention_d128(int num_tokens, int head_offset, const void* query, const void* key,
                                                  const void* value, const void* query_scale, const void* key_scale,
                                                  const void* value_scale, const void* selected, void* output,
                                                  void* state, int heads, int total_heads, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(num_tokens > 0 && heads > 0 && total_heads > 0, "sol_int8_fp8_attention_d128: sizes must be positive");
  NOB_REQUIRE(head_offset >= 0 && head_offset <= total_heads - heads,
              "sol_int8_fp8_attention_d128: head_offset %d outside [0, %d]", head_offset, total_heads - heads);
  NOB_REQUIRE(query && key && value && query_scale && key_scale && value_scale && selected && output && state,
              "sol_int8_fp8_attention_d128: NULL tensor");
  NOB_REQUIRE(heads <= 65535, "sol_int8_fp8_attention_d128: heads %d exceeds grid limit", heads);
  NOB_REQUIRE((num_tokens + kBlock - 1) / kBlock <= kMaxBlocks, "sol_int8_fp8_attention_d128: at most %d tokens",
              kMaxBlocks * kBlock);
  uint32_t* status = status_word_device_ptr();
  if (!status) return fail(kCudaError, "sol_int8_fp8_attention_d128: no current CUDA device");
  const uint64_t q_rows = (static_cast<uint64_t>(num_tokens) + 31) / 32 * 32;
  const uint64_t k_rows = (static_cast<uint64_t>(num_tokens) + 63) / 64 * 64;

  CUtensorMap mq, mk, mv;
  int rc;
  // Q, K: [heads][rows][128 bytes]; V: [heads][128 channels][k_rows bytes]
  if ((rc = make_tensor_map_3d(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, query, 128, q_rows, heads, 128, q_rows * 128, 128,
                               kTile, 1)))
    return rc;
  if ((rc = make_tensor_map_3d(&mk, CU_TENSOR_MAP_DATA_TYPE_UINT8, key, 128, k_rows, heads, 128, k_rows * 128, 128,
                               kTile, 1)))
    return rc;
  if ((rc = make_tensor_map_3d(&mv, CU_TENSOR_MAP_DATA_TYPE_UINT8, value, k_rows, 128, heads, k_rows, k_rows * 128, 128,
                               kTile, 1)))
    return rc;

  SolI8Params params;
  params.query_scale = static_cast<const float*>(query_scale);
  params.key_scale = static_cast<const float*>(key_scale);
  params.value_scale = static_cast<const float*>(value_scale);
  params.selected = static_cast<const uint8_t*>(selected);
  params.out = static_cast<__nv_bfloat16*>(output);
  params.state = static_cast<float*>(state);
  params.num_tokens = num_tokens;
  params.heads = heads;
  params.total_heads = total_heads;
  params.head_offset = head_offset;
  params.num_blocks = static_cast<int>(k_rows / 64);
  params.scale_log2 = 0.08838834764831845f * 1.4426950408889634f;
  params.status = status;

  const size_t smem = sizeof(Shared) + 1024;
  cudaError_t err =
      cudaFuncSetAttribute(fa_fwd_sol_i8f8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess)
    return fail(kCudaError, "sol_int8_fp8_attention_d128: cannot reserve %zu B of shared memory: %s", smem,
                cudaGetErrorString(err));
  dim3 grid((num_tokens + kTile - 1) / kTile, heads);
  fa_fwd_sol_i8f8_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, params);
  return check_launch("sol_int8_fp8_attention_d128");
}
