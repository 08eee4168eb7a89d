// Routing of the "sol" block-sparse attention: block pooling, centroid statistics and the
// selection mask.  CUDA-core kernels (HBM-bound pooling; the router's pooled GEMM is small).
//
// Reference programs replaced:
//   sol_pool / sol_int8_fp8_pool / sol_nvfp4_pool   src/nano_omni/kernels/attention/sol/pool.py:29-62,
//       int8_fp8/sol_pool.py:25-58, nvfp4/sol_pool.py:34-67
//   sol_stats                                        src/nano_omni/kernels/attention/sol/stats.py:28-67
//   sol_nvfp4_select                                 src/nano_omni/kernels/attention/nvfp4/sol_select.py:42-120
//
// Masks are compared bit for bit with a CPU restatement, so every reduction has a fixed order:
// sums over the tokens of a block and over blocks are sequential fp32 additions in index order;
// dot products over the 128 channels are sequential acc = acc + a*b with product and sum each
// rounded to fp32 (__fmul_rn / __fadd_rn keep the compiler from fusing them); divisions and
// square roots are IEEE.
#include "common.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

constexpr float kSqrt128 = 11.313708498984761f;

// ---------------------------------------------------------------- pooling
// One CTA of 64 threads per (block, head); thread c2 owns channels 2*c2, 2*c2+1 and walks
// the block's tokens in order (4-byte loads, 256 B per token row across the CTA).
__global__ void __launch_bounds__(64)
sol_pool_kernel(const __nv_bfloat16* __restrict__ key, const __nv_bfloat16* __restrict__ value,
                const float* __restrict__ key_mean, __nv_bfloat16* __restrict__ out, int num_tokens, int heads,
                int block, int num_blocks) {
  const int b = blockIdx.x, head = blockIdx.y, c = threadIdx.x * 2;
  const int begin = b * block, end = min(begin + block, num_tokens);
  const size_t row_stride = static_cast<size_t>(heads) * 128;
  const __nv_bfloat16* kp = key + static_cast<size_t>(begin) * row_stride + head * 128 + c;
  const __nv_bfloat16* vp = value + static_cast<size_t>(begin) * row_stride + head * 128 + c;
  float k0 = 0.f, k1 = 0.f, v0 = 0.f, v1 = 0.f;
#pragma unroll 8
  for (int t = begin; t < end; ++t, kp += row_stride, vp += row_stride) {
    const uint32_t kr = *reinterpret_cast<const uint32_t*>(kp);
    const uint32_t vr = *reinterpret_cast<const uint32_t*>(vp);
    k0 = __fadd_rn(k0, __uint_as_float(kr << 16));
    k1 = __fadd_rn(k1, __uint_as_float(kr & 0xffff0000u));
    v0 = __fadd_rn(v0, __uint_as_float(vr << 16));
    v1 = __fadd_rn(v1, __uint_as_float(vr & 0xffff0000u));
  }
  const float len = static_cast<float>(end - begin);
  const float m0 = __fdiv_rn(k0, len), m1 = __fdiv_rn(k1, len);
  const size_t plane = static_cast<size_t>(heads) * num_blocks * 128;
  const size_t at = (static_cast<size_t>(head) * num_blocks + b) * 128 + c;
  auto store = [&](size_t offset, float a, float bb) {
    *reinterpret_cast<__nv_bfloat162*>(out + offset) = __floats2bfloat162_rn(a, bb);
  };
  store(at, m0, m1);
  if (key_mean) {
    store(plane + at, __fsub_rn(m0, key_mean[head * 128 + c]), __fsub_rn(m1, key_mean[head * 128 + c + 1]));
    store(2 * plane + at, v0, v1);
  } else {
    store(plane + at, v0, v1);
  }
}

// ------------------------------------------------------------- statistics
__global__ void __launch_bounds__(128)
sol_stats_kernel(const __nv_bfloat16* __restrict__ pooled, float* __restrict__ out, int num_blocks) {
  const int head = blockIdx.x, c = threadIdx.x;
  const __nv_bfloat16* p = pooled + static_cast<size_t>(head) * num_blocks * 128 + c;
  float sum = __bfloat162float(p[0]);
  float sq = __fmul_rn(sum, sum);
  for (int b = 1; b < num_blocks; ++b) {
    const float x = __bfloat162float(p[static_cast<size_t>(b) * 128]);
    sum = __fadd_rn(sum, x);
    sq = __fadd_rn(sq, __fmul_rn(x, x));
  }
  const float n = static_cast<float>(num_blocks);
  const float mean = __fdiv_rn(sum, n);
  const float second = __fdiv_rn(sq, n);
  out[(head * 2 + 0) * 128 + c] = mean;
  out[(head * 2 + 1) * 128 + c] = fmaxf(__fsub_rn(second, __fmul_rn(mean, mean)), 0.f);
}

// ----------------------------------------------------------------- router
// One CTA per (group of 8 query blocks, head).  Phase 1: the 8 block means of Q (sequential
// over tokens) and their thresholds.  Phase 2: for tiles of 64 key blocks, every thread
// evaluates 2 (query block, key block) scores with a sequential 128-step mul/add chain.
constexpr int kQbPerCta = 8;
constexpr int kKbTile = 64;

// Two dot products over the 128 channels at once against the same b, each in the canonical order
// acc = a[0] * b[0]; acc = acc + a[d] * b[d] for d = 1..127 with product and sum rounded separately: a2[d] holds the
// d-th element of both left operands; the packed multiply and add round each lane on its own (no fusion).
__device__ __forceinline__ float2 seq_dot_pair(const float2* a2, const float* b) {
  auto pack = [](float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
  };
  auto mul = [](uint64_t x, uint64_t y) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(x), "l"(y));
    return r;
  };
  auto add = [](uint64_t x, uint64_t y) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(x), "l"(y));
    return r;
  };
  uint64_t acc = mul(pack(a2[0].x, a2[0].y), pack(b[0], b[0]));
#pragma unroll 8
  for (int d = 1; d < 128; ++d) acc = add(acc, mul(pack(a2[d].x, a2[d].y), pack(b[d], b[d])));
  float2 out;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(out.x), "=f"(out.y) : "l"(acc));
  return out;
}

__global__ void __launch_bounds__(256)
sol_select_kernel(const __nv_bfloat16* __restrict__ query, const __nv_bfloat16* __restrict__ pooled_key,
                  const float* __restrict__ stats, uint8_t* __restrict__ mask, float* __restrict__ scores,
                  int num_tokens, int heads, int block, int num_blocks, int num_protected, float tau) {
  __shared__ float qm[kQbPerCta][128];
  __shared__ float2 qpair[kQbPerCta / 2][128];  // query blocks (g, g + 4) interleaved for the packed dot products
  __shared__ float kc[kKbTile][129];
  __shared__ float thr[kQbPerCta];
  const int head = blockIdx.y;
  const int qb0 = blockIdx.x * kQbPerCta;
  const size_t row_stride = static_cast<size_t>(heads) * 128;
  // phase 1a: block means of Q, thread (qi, c) with c in 0..127 over two passes of 4 blocks... 256 threads =
  // 2 query blocks x 128 channels per pass
  for (int pass = 0; pass < kQbPerCta / 2; ++pass) {
    const int qi = pass * 2 + (threadIdx.x >> 7), c = threadIdx.x & 127;
    const int qb = qb0 + qi;
    float acc = 0.f;
    if (qb < num_blocks) {
      const int begin = qb * block, end = min(begin + block, num_tokens);
      const __nv_bfloat16* p = query + static_cast<size_t>(begin) * row_stride + head * 128 + c;
#pragma unroll 8
      for (int t = begin; t < end; ++t, p += row_stride) acc = __fadd_rn(acc, __bfloat162float(*p));
      acc = __fdiv_rn(acc, static_cast<float>(end - begin));
    }
    qm[qi][c] = acc;
    if (qi < kQbPerCta / 2) {
      qpair[qi][c].x = acc;
    } else {
      qpair[qi - kQbPerCta / 2][c].y = acc;
    }
  }
  __syncthreads();
  // phase 1b: thresholds (one thread per query block)
  if (mask && threadIdx.x < kQbPerCta) {
    const float* mu = stats + (head * 2 + 0) * 128;
    const float* var = stats + (head * 2 + 1) * 128;
    const float* q = qm[threadIdx.x];
    float m = __fmul_rn(q[0], mu[0]);
    float v = __fmul_rn(__fmul_rn(q[0], q[0]), var[0]);
    for (int d = 1; d < 128; ++d) {
      m = __fadd_rn(m, __fmul_rn(q[d], mu[d]));
      v = __fadd_rn(v, __fmul_rn(__fmul_rn(q[d], q[d]), var[d]));
    }
    const float mean = __fdiv_rn(m, kSqrt128);
    const float variance = __fdiv_rn(v, 128.0f);
    const float deviation = __fsqrt_rn(__fadd_rn(fmaxf(variance, 0.f), 1e-6f));
    thr[threadIdx.x] = __fadd_rn(mean, __fmul_rn(tau, deviation));
  }
  // phase 2
  for (int kb0 = 0; kb0 < num_blocks; kb0 += kKbTile) {
    __syncthreads();
    for (int i = threadIdx.x; i < kKbTile * 128; i += 256) {
      const int r = i >> 7, c = i & 127;
      kc[r][c] = (kb0 + r < num_blocks)
                     ? __bfloat162float(pooled_key[(static_cast<size_t>(head) * num_blocks + kb0 + r) * 128 + c])
                     : 0.f;
    }
    __syncthreads();
    // thread (kj, g): the scores of query blocks g and g + 4 against key block kj, two lanes of one packed chain
    const int kj = threadIdx.x & 63, g = threadIdx.x >> 6;
    const float2 dots = seq_dot_pair(qpair[g], kc[kj]);
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
      const int qi = g + rep * 4;
      const int qb = qb0 + qi, kb = kb0 + kj;
      if (qb < num_blocks && kb < num_blocks) {
        const float score = __fdiv_rn(rep == 0 ? dots.x : dots.y, kSqrt128);
        const size_t at = (static_cast<size_t>(qb) * heads + head) * num_blocks + kb;
        if (scores) scores[at] = score;
        if (mask) {
          const int delta = qb - kb;
          const bool keep = kb < num_protected || score > thr[qi] || (delta >= -1 && delta <= 1);
          mask[at] = keep ? 1 : 0;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ top-k
// One CTA per (query block, head): keep the k highest scores among the unprotected key blocks
// (ties: lower block index first) plus every protected block.  Bitonic sort of 64-bit keys
// (order-preserving score bits, then inverted index) in shared memory; num_blocks <= 2048.
constexpr int kTopkMax = 2048;

__global__ void __launch_bounds__(256)
sol_topk_kernel(const float* __restrict__ scores, uint8_t* __restrict__ mask, int heads, int num_blocks,
                int num_protected, int keep) {
  __shared__ unsigned long long keys[kTopkMax];
  const int qb = blockIdx.x, head = blockIdx.y;
  const size_t base = (static_cast<size_t>(qb) * heads + head) * num_blocks;
  int n = 1;
  while (n < num_blocks) n <<= 1;
  for (int i = threadIdx.x; i < n; i += 256) {
    unsigned long long key = 0;  // sorts last
    if (i < num_blocks && i >= num_protected) {
      float x = scores[base + i];
      if (x == 0.f) x = 0.f;  // -0 and +0 rank equal
      uint32_t bits = __float_as_uint(x);
      bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);  // larger float -> larger unsigned
      key = (static_cast<unsigned long long>(bits) << 32) | (0xffffffffu - static_cast<uint32_t>(i));
      if (key == 0) key = 1;
    }
    keys[i] = key;
  }
  __syncthreads();
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < n / 2; i += 256) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool descending = (lo & size) == 0;
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a < b) == descending) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < num_blocks; i += 256) mask[base + i] = i < num_protected ? 1 : 0;
  __syncthreads();
  for (int i = threadIdx.x; i < keep && i < n; i += 256) {
    const unsigned long long key = keys[i];
    if (key != 0) mask[base + (0xffffffffu - static_cast<uint32_t>(key))] = 1;
  }
}

}  // namespace
}  // namespace nob200

using namespace nob200;

extern "C" int nob200_sol_pool(int num_tokens, const void* key, const void* value, const void* key_mean, void* output,
                               int heads, int block, void* stream) {
  NOB_REQUIRE(num_tokens > 0 && heads > 0, "sol_pool: sizes must be positive");
  NOB_REQUIRE(block == 64 || block == 128, "sol_pool: block must be 64 or 128 (got %d)", block);
  NOB_REQUIRE(key && value && output, "sol_pool: NULL tensor");
  NOB_REQUIRE(heads <= 65535, "sol_pool: heads exceed the grid limit");
  const int nb = (num_tokens + block - 1) / block;
  sol_pool_kernel<<<dim3(nb, heads), 64, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(key), static_cast<const __nv_bfloat16*>(value),
      static_cast<const float*>(key_mean), static_cast<__nv_bfloat16*>(output), num_tokens, heads, block, nb);
  return check_launch("sol_pool");
}

extern "C" int nob200_sol_stats(const void* pooled, void* output, int heads, int num_blocks, void* stream) {
  NOB_REQUIRE(heads > 0 && num_blocks > 0, "sol_stats: sizes must be positive");
  NOB_REQUIRE(pooled && output, "sol_stats: NULL tensor");
  sol_stats_kernel<<<heads, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(pooled),
                                                                       static_cast<float*>(output), num_blocks);
  return check_launch("sol_stats");
}

extern "C" size_t nob200_sol_select_workspace_bytes(int num_tokens, int heads, int block, int topk_blocks) {
  if (topk_blocks <= 0 || num_tokens <= 0 || heads <= 0 || block <= 0) return 0;
  const size_t nb = (static_cast<size_t>(num_tokens) + block - 1) / block;
  return nb * nb * heads * sizeof(float);
}

extern "C" int nob200_sol_select(int num_tokens, int num_protected_blocks, const void* query, const void* pooled_key,
                                 const void* stats, void* output, int heads, float tau, int block,
                                 int topk_blocks, void* workspace, size_t workspace_bytes, void* stream) {
  NOB_REQUIRE(num_tokens > 0 && heads > 0, "sol_select: sizes must be positive");
  NOB_REQUIRE(block == 64 || block == 128, "sol_select: block must be 64 or 128 (got %d)", block);
  NOB_REQUIRE(query && pooled_key && output, "sol_select: NULL tensor");
  NOB_REQUIRE(heads <= 65535, "sol_select: heads exceed the grid limit");
  const int nb = (num_tokens + block - 1) / block;
  NOB_REQUIRE(num_protected_blocks >= 0 && num_protected_blocks <= nb,
              "sol_select: num_protected_blocks %d outside [0, %d]", num_protected_blocks, nb);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid((nb + kQbPerCta - 1) / kQbPerCta, heads);
  if (topk_blocks <= 0) {
    NOB_REQUIRE(stats, "sol_select: threshold routing needs the stats tensor");
    sol_select_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(query),
                                           static_cast<const __nv_bfloat16*>(pooled_key),
                                           static_cast<const float*>(stats), static_cast<uint8_t*>(output), nullptr,
                                           num_tokens, heads, block, nb, num_protected_blocks, tau);
    return check_launch("sol_select");
  }
  NOB_REQUIRE(nb <= kTopkMax, "sol_select: top-k routing supports at most %d blocks (got %d)", kTopkMax, nb);
  const size_t need = nob200_sol_select_workspace_bytes(num_tokens, heads, block, topk_blocks);
  NOB_REQUIRE(workspace && workspace_bytes >= need, "sol_select: top-k routing needs %zu B of workspace, %zu B given",
              need, workspace_bytes);
  // statistics are not read by top-k routing
  sol_select_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(query),
                                         static_cast<const __nv_bfloat16*>(pooled_key),
                                         static_cast<const float*>(stats), nullptr,
                                         static_cast<float*>(workspace), num_tokens, heads, block, nb,
                                         num_protected_blocks, tau);
  int rc = check_launch("sol_select(scores)");
  if (rc) return rc;
  const int keep = topk_blocks < nb ? topk_blocks : nb;
  sol_topk_kernel<<<dim3(nb, heads), 256, 0, s>>>(static_cast<const float*>(workspace), static_cast<uint8_t*>(output),
                                                  heads, nb, num_protected_blocks, keep);
  return check_launch("sol_select(topk)");
}
