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
//   warp 9      tcgen05 issuer: S = Q_t K_j^T (SS form, fp32 in TMEM), O_t += P_t V_j
//               (P read from TMEM, V consumed N-major straight from the TMA tile); the PV
//               MMAs of a tile start when the first 64 keys of P are written
//   warps 0-3   softmax for tile A: one thread per row, S row -> registers, row maximum with
//               3-input max, exp2 on packed fp32 pairs, bf16 P written to TMEM
//   warps 4-7   the same for tile B
// TMEM columns: S 0-127 (one score buffer, used by A and B in turn), P_A 128-191, P_B 192-255
// (bf16, two keys per column), O_A 256-383, O_B 384-511.
// The score buffer is free again as soon as a tile's softmax warps hold its row in registers, so the
// issuer computes the other tile's scores (and this tile's next ones) while the exponentials run: no
// softmax waits for an MMA that itself waits for that softmax's probabilities, and the two tiles are
// half a period apart by construction (B's scores can only be computed after A has taken its own).
// Issue order per key tile j: [A took S(j)] QK_B(j), [P_B(j-1)] PV_B(j-1), [B took S(j)] QK_A(j+1),
// [P_A(j)] PV_A(j).
// The running maximum is only raised when a row's maximum grew by more than 2^8
// (then O and the row sum are rescaled in place); it is exact for the first tile.
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

constexpr int kTile = 128;                     // query rows per tile and keys per tile
constexpr int kHalfBytes = kTile * 64 * 2;     // one 64-channel half of a tile (128B rows)
constexpr int kTileBytes = 2 * kHalfBytes;     // 32 KiB
constexpr int kStages = 4;
constexpr int kThreads = 384;                 // warpgroups: softmax A, softmax B, {TMA, MMA, 2 idle}
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;   // issues the score MMAs (S = Q K^T)
constexpr int kPvWarp = 10;   // issues the value MMAs (O += P V)
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;      // log2 units

struct __align__(1024) Shared {
  uint8_t q[2][kTileBytes];
  uint8_t kv[kStages][kTileBytes];
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];     // scores of tile t are in TMEM
  uint64_t s_taken[2];    // the softmax warps of tile t hold them in registers: the buffer is free
  uint64_t p_full[2][2];  // a 64-key half of P_t is written
  uint64_t pv_done[2];    // O_t += P_t V_j has completed: P_t may be overwritten, O_t may be rescaled
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t qk_issued;     // score MMA groups issued so far (written by the score issuer, polled by the value issuer)
};

// Register split after setmaxnreg: the CTA owns 384 x 168 registers; an increase beyond them would never return.
#ifndef NOB200_SERVICE_REGS
#define NOB200_SERVICE_REGS 88
#endif
constexpr int kServiceRegs = NOB200_SERVICE_REGS;
constexpr int kSoftmaxRegs = (384 * 168 - 128 * kServiceRegs) / 256 / 8 * 8;
static_assert(256 * kSoftmaxRegs + 128 * kServiceRegs <= 384 * 168, "setmaxnreg split exceeds the registers the CTA owns");

constexpr uint32_t kColS = 0, kColP = 128, kColO = 256;  // TMEM columns; P_t at kColP + 64 t, O_t at kColO + 128 t

// Build with -DNOB200_TRACE to record cycle stamps of one CTA (CTA 1 of head 0, first 64 key tiles) into a device
// array read back with nob200_debug_trace: rows 2 / 3 the score / value issuer, rows 4-11 the softmax warps.
#ifdef NOB200_TRACE
__device__ long long g_trace[12][64][8];
#define TRACE(role, j, k)                                                         \
  do {                                                                            \
    if (blockIdx.x == 1 && blockIdx.y == 0 && (j) < 64) g_trace[role][j][k] = clock64(); \
  } while (0)
#else
#define TRACE(role, j, k) \
  do {                    \
  } while (0)
#endif

#ifndef NOB200_BF16_POLY
#define NOB200_BF16_POLY 0
#endif

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
      mbar_init(&S.s_taken[t], 4);
      mbar_init(&S.p_full[t][0], 4);
      mbar_init(&S.p_full[t][1], 4);
      mbar_init(&S.pv_done[t], 1);
    }
    S.abort = 0;
    S.qk_issued = 0;
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
   reg_dealloc<kServiceRegs>();
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
      const int loads = 2 * n_kv;  // K_j at 2j, V_j at 2j+1
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
  } else if (warp == kMmaWarp || warp == kPvWarp) {
    // --------------------------------------------------------- tcgen05 issuers
    // Two issuing warps: warp 9 the score MMAs, warp 10 the value MMAs.  The issuing lane stalls on each
    // tcgen05.mma until the tensor pipe accepts it, so whatever it executes between two MMAs adds to the pipe's
    // 64 cycles per MMA: a group of MMAs is therefore ONE asm statement with all descriptors computed before it.
    {
      constexpr uint32_t idesc_qk = umma_idesc(kDF32, kFmtBF16, kFmtBF16, 0, 0, kTile, kTile);
      constexpr uint32_t idesc_pv = umma_idesc(kDF32, kFmtBF16, kFmtBF16, 0, 1, kTile, 128);
      auto full_parity = [](int i) { return (uint32_t)((i / kStages) & 1); };
      auto spin = [&](uint64_t* bar, uint32_t parity, uint32_t bit) { return warp_poll(bar, parity, abort_flag, status, bit); };
      auto rest = [&](uint64_t* bar, uint32_t parity, uint32_t bit) { return warp_rest(bar, parity, abort_flag, status, bit); };
      // Order between the two threads.  The score buffer is handed from tile A to tile B and back, so the time from
      // "tile t holds S(j) in registers" to "the other tile's scores are complete" is the critical ring of the
      // kernel, while a tile's value MMAs only have to finish before its next probabilities are written.  Value
      // MMAs must therefore not sit in the tensor pipe's queue when a score group becomes issuable: each half of
      // them is held until the score group that becomes issuable at about the same time has been issued
      // (S.qk_issued counts the issued score groups, numbered n = 2 j + t):
      //   [A took S(j)]  QK_B(j)   then PV_A(j-1) keys 64-127, PV_B(j-1) keys 0-63
      //   [B took S(j)]  QK_A(j+1) then PV_B(j-1) keys 64-127, PV_A(j) keys 0-63
      if (warp == kMmaWarp) {
        const uint64_t desc_k_major = umma_smem_desc(0, 16, 1024, kSwizzle128B);
        const uint64_t q_desc[2] = {desc_k_major + (smem_u32(S.q[0]) >> 4), desc_k_major + (smem_u32(S.q[1]) >> 4)};
        const uint64_t kv_k_desc = desc_k_major + (smem_u32(S.kv[0]) >> 4);  // + stage * (kTileBytes >> 4)
        const uint32_t d = tmem + kColS;
        uint32_t issued = 0;
        auto qk = [&](int t, int j, uint64_t* taken, uint32_t taken_parity) -> bool {  // S = Q_t K_j^T
          const int ik = 2 * j, sk = ik % kStages;
          // 16 channels = 32 bytes inside a 64-channel half; halves are kHalfBytes apart
          const uint64_t a0 = t ? q_desc[1] : q_desc[0], b0 = kv_k_desc + sk * (kTileBytes >> 4);
          const uint64_t a1 = a0 + 2, a2 = a0 + 4, a3 = a0 + 6, a4 = a0 + (kHalfBytes >> 4), a5 = a4 + 2, a6 = a4 + 4, a7 = a4 + 6;
          const uint64_t b1 = b0 + 2, b2 = b0 + 4, b3 = b0 + 6, b4 = b0 + (kHalfBytes >> 4), b5 = b4 + 2, b6 = b4 + 4, b7 = b4 + 6;
          if (t == 0 && !rest(&S.kv_full[sk], full_parity(ik), kWaitTimeoutLoad)) return false;
          if (taken && !spin(taken, taken_parity, kWaitTimeoutSoftmax)) return false;  // last: the critical hand-over
          tc_fence_after();
          if (elect_one()) {
          TRACE(2, j, 2 * t);
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
              "r"(idesc_qk), "l"(a0), "l"(a1), "l"(a2), "l"(a3), "l"(a4), "l"(a5), "l"(a6), "l"(a7), "l"(b0), "l"(b1),
              "l"(b2), "l"(b3), "l"(b4), "l"(b5), "l"(b6), "l"(b7)
              : "memory");
          tc_commit(&S.s_full[t]);
          if (t == 1 || !two) tc_commit(&S.kv_empty[sk]);  // last reader of K_j
          *reinterpret_cast<volatile uint32_t*>(&S.qk_issued) = issued + 1;
          TRACE(2, j, 2 * t + 1);
          }
          ++issued;
          return true;
        };
        bool ok = rest(&S.q_full, 0, kWaitTimeoutLoad) && qk(0, 0, nullptr, 0);
        for (int j = 0; ok && j < n_kv; ++j) {
          if (two && !(ok = qk(1, j, &S.s_taken[0], j & 1))) break;
          if (j + 1 < n_kv && !(ok = qk(0, j + 1, &S.s_taken[two ? 1 : 0], j & 1))) break;
        }
      } else {
        const uint64_t desc_n_major = umma_smem_desc(0, kHalfBytes, 1024, kSwizzle128B);
        const uint64_t kv_n_desc = desc_n_major + (smem_u32(S.kv[0]) >> 4);
        const uint32_t total_qk = (two ? 2 : 1) * n_kv;
        // O_t += P_t(j)[:, 64 half : 64 half + 64] V_j[64 half : 64 half + 64, :], after `gate` score groups
        auto pv_half = [&](int t, int j, int half, uint32_t gate) -> bool {
          const int iv = 2 * j + 1, sv = iv % kStages;
          // 16 keys = 16 rows of 128 B = 2048 B; P holds two keys per 32-bit column
          const uint64_t b0 = kv_n_desc + sv * (kTileBytes >> 4) + half * (4 * 2048 >> 4);
          const uint64_t b1 = b0 + (2048 >> 4), b2 = b0 + 2 * (2048 >> 4), b3 = b0 + 3 * (2048 >> 4);
          const uint32_t d = tmem + kColO + t * kTile, a0 = tmem + kColP + t * 64 + half * 32;
          const uint32_t accumulate = (j > 0 || half > 0) ? 1u : 0u;
          if (gate > total_qk) gate = total_qk;
          if (half == 0 && !rest(&S.kv_full[sv], full_parity(iv), kWaitTimeoutLoad)) return false;
          if (!NOB200_PFULL_WAIT(&S.p_full[t][half], j & 1, kWaitTimeoutSoftmax)) return false;
          if (!warp_wait_counter(&S.qk_issued, gate, abort_flag, status, kWaitTimeoutMma)) return false;
          tc_fence_after();
          if (elect_one()) {
          TRACE(3, j, 4 * t + 2 * half);
          asm volatile(
              "{\n\t.reg .pred p0, p1;\n\t"
              "setp.ne.b32 p0, %2, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], %7, %1, p0;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %8, %1, p1;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %9, %1, p1;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], [%6], %10, %1, p1;\n\t}" ::"r"(d),
              "r"(idesc_pv), "r"(accumulate), "r"(a0), "r"(a0 + 8), "r"(a0 + 16), "r"(a0 + 24), "l"(b0), "l"(b1), "l"(b2),
              "l"(b3)
              : "memory");
          if (half == 1) {
            tc_commit(&S.pv_done[t]);
            if (t == 1 || !two) tc_commit(&S.kv_empty[sv]);  // last reader of V_j
          }
          TRACE(3, j, 4 * t + 2 * half + 1);
          }
          return true;
        };
        bool ok = true;
        if (two) {
          // score groups are numbered n = 2 j + t; "n + 1 issued" means group n is in the pipe
          for (int j = 0; ok && j < n_kv; ++j) {
            ok = pv_half(0, j, 0, 2 * j + 3)        // after QK_A(j+1)
                 && pv_half(0, j, 1, 2 * j + 4)     // after QK_B(j+1)
                 && pv_half(1, j, 0, 2 * j + 4)     // after QK_B(j+1)
                 && pv_half(1, j, 1, 2 * j + 5);    // after QK_A(j+2)
          }
        } else {
          for (int j = 0; ok && j < n_kv; ++j) ok = pv_half(0, j, 0, j + 2) && pv_half(0, j, 1, j + 2);
        }
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
      const uint32_t p_addr = tmem + lane_base + kColP + t * 64;
      const uint32_t o_addr = tmem + lane_base + kColO + t * kTile;
      float m_used = 0.f;
      uint64_t la = 0ull, lb = 0ull;  // four partial row sums as two fp32 pairs
      bool ok = true;
      for (int j = 0; j < n_kv; ++j) {
        ok = poll(&S.s_full[t], j & 1, kWaitTimeoutMma);
        if (!ok) break;
        if (lane == 0) TRACE(4 + warp, j, 0);
        tc_fence_after();
        uint32_t s[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&s[32 * c]));
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&S.s_taken[t]);
        if (lane == 0) TRACE(4 + warp, j, 1);
        if (kv_begin + j == n_kv_total - 1) {
          const int valid = num_tokens - (kv_begin + j) * kTile;
          if (valid < kTile) {
#pragma unroll
            for (int i = 0; i < 128; ++i)
              if (i >= valid) s[i] = 0xff800000u;  // -inf
          }
        }
        float mx0 = __uint_as_float(s[0]), mx1 = __uint_as_float(s[1]);
        float mx2 = __uint_as_float(s[2]), mx3 = __uint_as_float(s[3]);
#pragma unroll
        for (int i = 4; i < 124; i += 8) {
          mx0 = max3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
          mx1 = max3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
          mx2 = max3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
          mx3 = max3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
        }
        mx0 = max3(mx0, __uint_as_float(s[124]), __uint_as_float(s[125]));
        mx1 = max3(mx1, __uint_as_float(s[126]), __uint_as_float(s[127]));
        const float mx = fmaxf(max3(mx0, mx1, mx2), mx3) * scale_log2;
        if (lane == 0) TRACE(4 + warp, j, 2);
        bool pv_waited = j == 0;  // P_t and O_t are untouched by the tensor core before the first PV
        if (j == 0) {
          m_used = mx;
        } else if (__any_sync(0xffffffffu, mx > m_used + kRescaleThreshold)) {
          const float m_new = fmaxf(m_used, mx);
          const float alpha = ex2(m_used - m_new);
          const uint64_t alpha2 = pack2(alpha, alpha);
          la = fma2(la, alpha2, 0ull);
          lb = fma2(lb, alpha2, 0ull);
          // O_t += P_t V_{j-1} must have completed; the next PV waits for our arrival on p_full.
          ok = poll(&S.pv_done[t], (j - 1) & 1, kWaitTimeoutMma);
          if (!ok) break;
          pv_waited = true;
          tc_fence_after();
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
          if (half == 0 && !pv_waited) {
            // the previous tile's PV still reads P_t until this completes (normally long ago)
            ok = poll(&S.pv_done[t], (j - 1) & 1, kWaitTimeoutMma);
            if (!ok) break;
            tc_fence_after();
          }
          if (lane == 0) TRACE(4 + warp, j, 3 + 2 * half);
          tmem_st32(p_addr + 32 * half, p);
          if (SPLIT || half == 1) {
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&S.p_full[t][SPLIT ? half : 0]);
          }
          if (lane == 0) TRACE(4 + warp, j, 4 + 2 * half);
        }
        if (!ok) break;
      }
      if (ok) ok = poll(&S.pv_done[t], (n_kv - 1) & 1, kWaitTimeoutMma);
      if (ok) {
        tc_fence_after();
        float l0, l1, l2, l3;
        unpack2(la, l0, l1);
        unpack2(lb, l2, l3);
        const float l = (l0 + l1) + (l2 + l3);
        const float inv = 1.0f / l;
        const int token = q0 + t * kTile + row;
        __nv_bfloat16* dst = out.row(token < num_tokens ? token : 0, total_heads, head + head_offset);
        bool store = token < num_tokens;
        if (gridDim.z > 1) {
          const size_t at = (static_cast<size_t>(blockIdx.z) * num_tokens + token) * gridDim.y + head;
          dst = partial_out + at * 128;
          store = store && NOB_CHECK(at < static_cast<size_t>(gridDim.z) * num_tokens * gridDim.y, status);
          if (store) partial_lse[at] = m_used + log2f(l);
        } else {
          store = store && route_open(out, status);
          store = store && NOB_CHECK(head + head_offset < total_heads &&
                                         (out.tokens_per_rank == 0 ||
                                          (token / out.tokens_per_rank < kMaxWorld && out.peer[token / out.tokens_per_rank])),
                                     status);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + 32 * c, o);
          tc_wait_ld();
          if (store) {
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
                       int splits, const uint32_t* status) {
  const long long item = blockIdx.x * 256ll + threadIdx.x;  // (token, head, 8-channel piece)
  const long long total = static_cast<long long>(num_tokens) * heads * 16;
  if (item >= total || !route_open(out, status)) return;
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
  auto kernel = fa_fwd_bf16_kernel<NOB200_BF16_POLY, true>;
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
        partial_out, partial_lse, route, num_tokens, heads, total_heads, head_offset, kv_splits, status);
    rc = check_launch("dense_bf16_attention_d128(merge)");
  }
  return rc;
}

}  // namespace

int launch_merge_splits(const __nv_bfloat16* partial_out, const float* partial_lse, const OutRoute& route, int num_tokens,
                        int heads, int total_heads, int head_offset, int splits, void* stream) {
  const long long items = static_cast<long long>(num_tokens) * heads * 16;
  uint32_t* status = status_word_device_ptr();
  if (!status) return fail(kCudaError, "attention(merge of key splits): no current CUDA device");
  fa_merge_splits_kernel<<<static_cast<unsigned>((items + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      partial_out, partial_lse, route, num_tokens, heads, total_heads, head_offset, splits, status);
  return check_launch("attention(merge of key splits)");
}

}  // namespace nob200

#ifdef NOB200_TRACE
extern "C" int nob200_debug_trace(long long* out) {
  return cudaMemcpyFromSymbol(out, nob200::g_trace, sizeof(long long) * 12 * 64 * 8) == cudaSuccess ? 0 : -1;
}
#endif

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
