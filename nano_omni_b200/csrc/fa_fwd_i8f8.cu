// Dense non-causal int8-QK / fp8-PV attention forward for head_dim 128 on sm_100a.
//
// Replaces the reference program dense_int8_fp8_attention
// (src/nano_omni/kernels/attention/int8_fp8/dense.py:21-315):
//   S = Q8 K8^T in int32; s = S * qscale[row/32] * kscale[key/64] * log2e/sqrt(128);
//   online softmax in fp32; P scaled into the e4m3 range and rounded to e4m3;
//   O += P8 V8 (fp32 accumulation here, fp16 partials in the reference);
//   out = O * vscale[channel] / l.
// Operands: Q int8 [heads, Tq32, 128], K int8 [heads, Tk64, 128], V e4m3 [heads, 128, Tk64]
// (channel-major; inside every 16 tokens, stored position p holds token
// [0,1,8,9,2,3,10,11,4,5,12,13,6,7,14,15][p]), f32 scales, output bf16 [Tq, heads*128].
//
// Same CTA organisation as the bf16 kernel: 256 query rows of one head per CTA (tiles A and B),
// key tiles of 128, warps 0-3 / 4-7 softmax for A / B with one thread per row, warp 8 TMA
// producer, warp 9 tcgen05 issuer.  QK is kind::i8 (K = 32 per MMA, 4 per tile), PV is
// kind::f8f6f4 with P (e4m3, four keys per 32-bit TMEM column) as the TMEM operand and the
// V tile K-major straight from TMA.  int32 scores become fp32 without a conversion
// instruction: S + 0x4B400000 read as a float is 2^23*1.5 + S exactly.
// P is scaled by 448 / 2^3 and the running maximum is raised when it grew by more than
// 2^3, so P never exceeds 448 (e4m3's largest finite value).
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
constexpr int kStages = 6;
constexpr int kThreads = 384;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr float kHeadroomLog2 = 3.0f;              // P <= 448 while the stale maximum lags by <= 2^3
constexpr float kLog2PScale = 8.807354922057604f - kHeadroomLog2;  // log2(448) - 3
constexpr uint32_t kMagicBits = 0x4B400000u;       // 12582912.0f
constexpr float kMagic = 12582912.0f;

struct __align__(1024) Shared {
  uint8_t q[2][kTileBytes];
  uint8_t kv[kStages][kTileBytes];
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t o_final[2];
  uint32_t tmem_base;
  uint32_t abort;
};

// 384 threads x 168 launch registers = 64512 owned by the CTA; the split below uses exactly that.
static_assert(256 * 224 + 128 * 56 <= 384 * 168, "setmaxnreg split exceeds the registers the CTA owns");

// two e4m3 bytes: `lo` in bits 0-7, `hi` in bits 8-15
__device__ __forceinline__ uint32_t pack_e4m3(float lo, float hi) {
  uint16_t d;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
  return d;
}
__global__ void __launch_bounds__(kThreads, 1)
fa_fwd_i8f8_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const float* __restrict__ query_scale,
                   const float* __restrict__ key_scale, const float* __restrict__ value_scale,
                   __nv_bfloat16* __restrict__ out, int num_query_tokens, int num_kv_tokens, int heads,
                   float scale_log2, uint32_t* status, int query_block, int key_block,
                   __nv_bfloat16* __restrict__ partial_out, float* __restrict__ partial_lse) {
  extern __shared__ uint8_t smem_raw[];
  Shared& S = *reinterpret_cast<Shared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int q0 = blockIdx.x * (2 * kTile);
  const bool two = q0 + kTile < num_query_tokens;
  // gridDim.z > 1: this CTA covers a contiguous share of the key tiles and writes a normalised partial result with
  // its log-sum-exp; fa_merge_splits_kernel (fa_fwd_bf16.cu) merges the shares.
  const int n_kv_total = (num_kv_tokens + kTile - 1) / kTile;
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
      mbar_init(&S.p_full[t], 4);
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
        tma_load_3d(S.q[0], &map_q, &S.q_full, 0, q0, head);
        if (two) tma_load_3d(S.q[1], &map_q, &S.q_full, 0, q0 + kTile, head);
        const int loads = 2 * n_kv;  // K_j at 2j, V_j at 2j+1
        int issued = 0;
        for (int i = 0; i < loads; ++i) {
          const int st = i % kStages;
          if (i >= kStages) {
            if (!mbar_wait(&S.kv_empty[st], ((i / kStages) - 1) & 1, abort_flag, status, kWaitTimeoutRing)) break;
          }
          mbar_expect_tx(&S.kv_full[st], kTileBytes);
          const int tok = (kv_begin + (i >> 1)) * kTile;
          if (i & 1) {
            tma_load_3d(S.kv[st], &map_v, &S.kv_full[st], tok, 0, head);  // [channel][token] tile
          } else {
            tma_load_3d(S.kv[st], &map_k, &S.kv_full[st], 0, tok, head);  // [token][channel] tile
          }
          issued = i + 1;
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
      // group of MMAs with ready-made 64-bit descriptors.  The waits on the probabilities are on the chain P stored ->
      // PV -> next QK -> scores complete and poll; K / V tiles were loaded long before and their waits may sleep.
      {
        constexpr uint32_t idesc_qk = umma_idesc(kDS32, kFmtS8, kFmtS8, 0, 0, kTile, kTile);
        constexpr uint32_t idesc_pv = umma_idesc(kDF32, kFmtE4M3, kFmtE4M3, 0, 0, kTile, 128);
        // All three smem operands are K-major tiles of 128 rows x 128 bytes (one swizzle atom per row).
        const uint64_t desc = umma_smem_desc(0, 16, 1024, kSwizzle128B);
        const uint64_t q_desc[2] = {desc + (smem_u32(S.q[0]) >> 4), desc + (smem_u32(S.q[1]) >> 4)};
        const uint64_t kv_desc = desc + (smem_u32(S.kv[0]) >> 4);
        // S_t = Q_t K^T: four MMAs of 32 channels (32 bytes of a row = 2 descriptor units), then the commits
        auto issue_qk = [&](int t, int st, bool last_reader) {
          const uint64_t a = q_desc[t], b = kv_desc + st * (kTileBytes >> 4);
          const uint32_t d = tmem + t * kTile;
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
            tc_commit(&S.s_full[t]);
            if (last_reader) tc_commit(&S.kv_empty[st]);
          }
        };
        // O_t += P_t V: four MMAs of 32 keys (32 bytes of a V row; 8 TMEM columns of P), then the commits
        auto issue_pv = [&](int t, int st, bool accumulate, bool last_reader, bool final) {
          const uint64_t b = kv_desc + st * (kTileBytes >> 4);
          const uint32_t d = tmem + 256 + t * kTile, a = tmem + t * kTile;
          if (elect_one()) {
            asm volatile(
                "{\n\t.reg .pred p0, p1;\n\t"
                "setp.ne.b32 p0, %2, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%3], %7, %1, p0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%4], %8, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%5], %9, %1, p1;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%6], %10, %1, p1;\n\t}" ::"r"(d),
                "r"(idesc_pv), "r"(accumulate ? 1u : 0u), "r"(a), "r"(a + 8), "r"(a + 16), "r"(a + 24), "l"(b), "l"(b + 2),
                "l"(b + 4), "l"(b + 6)
                : "memory");
            if (last_reader) tc_commit(&S.kv_empty[st]);
            if (final) tc_commit(&S.o_final[t]);
          }
        };
        auto full_parity = [](int i) { return (uint32_t)((i / kStages) & 1); };
        auto rest = [&](uint64_t* bar, uint32_t parity, uint32_t bit) { return warp_rest(bar, parity, abort_flag, status, bit); };
        auto spin = [&](uint64_t* bar, uint32_t parity, uint32_t bit) { return warp_poll(bar, parity, abort_flag, status, bit); };

        bool ok = rest(&S.q_full, 0, kWaitTimeoutLoad) && rest(&S.kv_full[0], 0, kWaitTimeoutLoad);
        if (ok) {
          tc_fence_after();
          issue_qk(0, 0, !two);
          if (two) issue_qk(1, 0, true);
        }
        for (int j = 0; ok && j < n_kv; ++j) {
          const int iv = 2 * j + 1, ik = 2 * j + 2;
          const int sv = iv % kStages, sk = ik % kStages;
          const bool more = j + 1 < n_kv;
          if (!(ok = rest(&S.kv_full[sv], full_parity(iv), kWaitTimeoutLoad))) break;
          if (more && !(ok = rest(&S.kv_full[sk], full_parity(ik), kWaitTimeoutLoad))) break;
          if (!(ok = spin(&S.p_full[0], j & 1, kWaitTimeoutSoftmax))) break;
          tc_fence_after();
          issue_pv(0, sv, j > 0, !two, !more);
          if (more) issue_qk(0, sk, !two);
          if (two) {
            if (!(ok = spin(&S.p_full[1], j & 1, kWaitTimeoutSoftmax))) break;
            tc_fence_after();
            issue_pv(1, sv, j > 0, true, !more);
            if (more) issue_qk(1, sk, true);
          }
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
      const int token = q0 + t * kTile + row;
      // scales per `query_block` (32, 64 or 128) query tokens and per `key_block` (64 or 128) key tokens
      const int q_blocks = (num_query_tokens + query_block - 1) / query_block;
      const int k_blocks = (num_kv_tokens + key_block - 1) / key_block;
      const int per_half = key_block / 64;  // 64-key halves per key scale
      // per-row factor: query scale of the row's block times log2e/sqrt(128)
      const float qf = query_scale[static_cast<size_t>(head) * q_blocks + min(token / query_block, q_blocks - 1)] * scale_log2;
      const float* ks_head = key_scale + static_cast<size_t>(head) * k_blocks;
      float m_used = 0.f, l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      bool ok = true;
      for (int j = 0; j < n_kv; ++j) {
        // factors of the two 64-key blocks of this tile (0 for a block past the end: fully masked below)
        const int jt = kv_begin + j;  // key tile in the whole sequence
        const float f0 = qf * ks_head[(2 * jt) / per_half];
        const float f1 = ((2 * jt + 1) / per_half < k_blocks) ? qf * ks_head[(2 * jt + 1) / per_half] : 0.f;
        ok = warp_poll(&S.s_full[t], j & 1, abort_flag, status, kWaitTimeoutMma);  // on the chain: poll
        if (!ok) break;
        tc_fence_after();
        uint32_t s[128];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld32(s_addr + 32 * cc, *reinterpret_cast<uint32_t(*)[32]>(&s[32 * cc]));
        tc_wait_ld();
        // int32 -> the float 2^23*1.5 + S (exact for |S| < 2^22; |S| <= 128*128*127 here)
#pragma unroll
        for (int i = 0; i < 128; ++i) s[i] += kMagicBits;
        const int valid = num_kv_tokens - jt * kTile;  // keys of this tile that exist (>= 1)
        float a0 = __uint_as_float(s[0]), a1 = __uint_as_float(s[64]);
        if (valid >= kTile) {
#pragma unroll
          for (int i = 1; i < 63; i += 2) {
            a0 = max3(a0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
            a1 = max3(a1, __uint_as_float(s[64 + i]), __uint_as_float(s[64 + i + 1]));
          }
          a0 = fmaxf(a0, __uint_as_float(s[63]));
          a1 = fmaxf(a1, __uint_as_float(s[127]));
        } else {
          a0 = -INFINITY, a1 = -INFINITY;
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            if (i < valid) a0 = fmaxf(a0, __uint_as_float(s[i]));
            if (64 + i < valid) a1 = fmaxf(a1, __uint_as_float(s[64 + i]));
          }
        }
        float mx = (a0 - kMagic) * f0;
        if (valid > 64) mx = fmaxf(mx, (a1 - kMagic) * f1);
        if (j == 0) {
          m_used = mx;
        } else if (__any_sync(0xffffffffu, mx > m_used + kHeadroomLog2)) {
          const float m_new = fmaxf(m_used, mx);
          const float alpha = ex2(m_used - m_new);
          l0 *= alpha, l1 *= alpha, l2 *= alpha, l3 *= alpha;
          // S_t(j) is complete, hence so is O_t += P_t V_{j-1}; the next PV waits for our arrival.
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
        // into the constant instead would round it to that product's ulp, an error of up to 4 % in P for scales near 1.
        const float cst = m_used - kLog2PScale;
        uint32_t p[32];
        if (valid >= kTile) {
          // full tile: packed fp32 pairs; four partial row sums live in two register pairs
          uint64_t la = pack2(l0, l1), lb = pack2(l2, l3);
          // Folding 2^23*1.5 * f into the FMA constant saves the subtraction but rounds the constant to half an ulp of
          // that product; taken only while this stays below 2^-11 in the exponent (0.03 % in P).  f is the same for
          // the 32 rows of a warp (one query-scale block), so the branch does not diverge.
          auto exponentials = [&](auto fold_tag) {
            constexpr bool kFold = decltype(fold_tag)::value;
            const float c0 = kFold ? fmaf(kMagic, f0, cst) : cst, c1 = kFold ? fmaf(kMagic, f1, cst) : cst;
            const uint64_t nm2 = pack2(-kMagic, -kMagic);
#pragma unroll
            for (int g = 0; g < 8; ++g) {  // groups of 16 keys; stored order inside a group: 0,1,8,9 | 2,3,10,11 | ...
              const uint64_t f2 = g < 4 ? pack2(f0, f0) : pack2(f1, f1);
              const uint64_t nc2 = g < 4 ? pack2(-c0, -c0) : pack2(-c1, -c1);
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
          if (fmaxf(f0, f1) * kMagic < 16384.0f) {
            exponentials(std::true_type{});
          } else {
            exponentials(std::false_type{});
          }
          unpack2(la, l0, l1);
          unpack2(lb, l2, l3);
        } else {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float e[16];
            const float f = g < 4 ? f0 : f1;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x = fmaf(__uint_as_float(s[16 * g + i]) - kMagic, f, -cst);
              if (16 * g + i >= valid) x = -INFINITY;
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
        tmem_st32(s_addr, p);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&S.p_full[t]);
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&S.o_final[t], 0, abort_flag, status, kWaitTimeoutMma));
      if (ok) {
        tc_fence_after();
        const float l = (l0 + l1) + (l2 + l3);
        const float inv = 1.0f / l;
        const float* vs = value_scale + head * 128;
        __nv_bfloat16* dst = out + (static_cast<size_t>(token) * heads + head) * 128;
        if (gridDim.z > 1) {
          const size_t at = (static_cast<size_t>(blockIdx.z) * num_query_tokens + token) * heads + head;
          dst = partial_out + at * 128;
          // the probability scale 448/8 is common to all shares and cancels in the merge
          if (token < num_query_tokens &&
              NOB_CHECK(at < static_cast<size_t>(gridDim.z) * num_query_tokens * heads, status))
            partial_lse[at] = m_used + log2f(l);
        }
        const bool store = token < num_query_tokens && NOB_CHECK(head < heads, status);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t o[32];
          tmem_ld32(o_addr + 32 * cc, o);
          tc_wait_ld();
          if (store) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              float r[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) r[k] = __uint_as_float(o[i + k]) * vs[32 * cc + i + k] * inv;
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

extern "C" int nob200_dense_int8_fp8_d128(int num_kv_tokens, int num_query_tokens, const void* query, const void* key,
                                          const void* value, const void* query_scale, const void* key_scale,
                                          const void* value_scale, void* output, int heads, void* stream) {
  return nob200_dense_int8_fp8_d128_blocks(num_kv_tokens, num_query_tokens, query, key, value, query_scale, key_scale,
                                           value_scale, output, heads, 32, 64, stream);
}

extern "C" int nob200_dense_int8_fp8_d128_splitkv(int num_kv_tokens, int num_query_tokens, const void* query,
                                                  const void* key, const void* value, const void* query_scale,
                                                  const void* key_scale, const void* value_scale, void* output,
                                                  int heads, int query_block, int key_block, int kv_splits,
                                                  void* workspace, size_t workspace_bytes, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(num_kv_tokens > 0 && num_query_tokens > 0 && heads > 0, "dense_int8_fp8_d128: sizes must be positive");
  NOB_REQUIRE(query && key && value && query_scale && key_scale && value_scale && output,
              "dense_int8_fp8_d128: NULL tensor");
  NOB_REQUIRE(heads <= 65535, "dense_int8_fp8_d128: heads %d exceeds grid limit", heads);
  NOB_REQUIRE(query_block == 32 || query_block == 64 || query_block == 128,
              "dense_int8_fp8_d128: query scale block must be 32, 64 or 128 tokens (got %d)", query_block);
  NOB_REQUIRE(key_block == 64 || key_block == 128, "dense_int8_fp8_d128: key scale block must be 64 or 128 tokens (got %d)",
              key_block);
  const int n_kv = (num_kv_tokens + kTile - 1) / kTile;
  NOB_REQUIRE(kv_splits >= 1 && kv_splits <= 64 && kv_splits <= n_kv,
              "dense_int8_fp8_d128: kv_splits %d outside [1, min(64, %d)]", kv_splits, n_kv);
  const size_t need = nob200_dense_bf16_attention_d128_splitkv_workspace_bytes(num_query_tokens, heads, kv_splits);
  NOB_REQUIRE(need == 0 || (workspace && workspace_bytes >= need),
              "dense_int8_fp8_d128: %zu B of workspace required for %d key splits, %zu B given", need, kv_splits,
              workspace_bytes);
  uint32_t* status = status_word_device_ptr();
  if (!status) return fail(kCudaError, "dense_int8_fp8_d128: no current CUDA device");
  const uint64_t q_rows = (static_cast<uint64_t>(num_query_tokens) + query_block - 1) / query_block * query_block;
  const uint64_t k_rows = (static_cast<uint64_t>(num_kv_tokens) + key_block - 1) / key_block * key_block;
  const uint64_t v_cols = (static_cast<uint64_t>(num_kv_tokens) + 63) / 64 * 64;  // the value quantiser pads to 64

  CUtensorMap mq, mk, mv;
  int rc;
  // Q, K: [heads][rows][128 bytes]; V: [heads][128 channels][v_cols bytes]
  if ((rc = make_tensor_map_3d(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, query, 128, q_rows, heads, 128, q_rows * 128, 128,
                               kTile, 1)))
    return rc;
  if ((rc = make_tensor_map_3d(&mk, CU_TENSOR_MAP_DATA_TYPE_UINT8, key, 128, k_rows, heads, 128, k_rows * 128, 128,
                               kTile, 1)))
    return rc;
  if ((rc = make_tensor_map_3d(&mv, CU_TENSOR_MAP_DATA_TYPE_UINT8, value, v_cols, 128, heads, v_cols, v_cols * 128, 128,
                               kTile, 1)))
    return rc;

  const size_t smem = sizeof(Shared) + 1024;
  cudaError_t err =
      cudaFuncSetAttribute(fa_fwd_i8f8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess)
    return fail(kCudaError, "dense_int8_fp8_d128: cannot reserve %zu B of shared memory: %s", smem,
                cudaGetErrorString(err));
  const float scale_log2 = 0.08838834764831845f * 1.4426950408889634f;
  const size_t share = static_cast<size_t>(num_query_tokens) * heads;
  const size_t partial_bytes = (static_cast<size_t>(kv_splits) * share * 128 * 2 + 255) / 256 * 256;
  __nv_bfloat16* partial_out = static_cast<__nv_bfloat16*>(workspace);
  float* partial_lse = kv_splits > 1 ? reinterpret_cast<float*>(static_cast<char*>(workspace) + partial_bytes) : nullptr;
  dim3 grid((num_query_tokens + 2 * kTile - 1) / (2 * kTile), heads, kv_splits);
  fa_fwd_i8f8_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      mq, mk, mv, static_cast<const float*>(query_scale), static_cast<const float*>(key_scale),
      static_cast<const float*>(value_scale), static_cast<__nv_bfloat16*>(output), num_query_tokens, num_kv_tokens,
      heads, scale_log2, status, query_block, key_block, partial_out, partial_lse);
  if ((rc = check_launch("dense_int8_fp8_d128"))) return rc;
  if (kv_splits > 1) {
    OutRoute route = {};
    route.peer[0] = static_cast<__nv_bfloat16*>(output);
    rc = launch_merge_splits(partial_out, partial_lse, route, num_query_tokens, heads, heads, 0, kv_splits, stream);
  }
  return rc;
}

extern "C" int nob200_dense_int8_fp8_d128_blocks(int num_kv_tokens, int num_query_tokens, const void* query,
                                                 const void* key, const void* value, const void* query_scale,
                                                 const void* key_scale, const void* value_scale, void* output,
                                                 int heads, int query_block, int key_block, void* stream) {
  return nob200_dense_int8_fp8_d128_splitkv(num_kv_tokens, num_query_tokens, query, key, value, query_scale, key_scale,
                                            value_scale, output, heads, query_block, key_block, 1, nullptr, 0, stream);
}
