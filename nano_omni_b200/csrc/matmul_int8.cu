// INT8 and BF16 GEMMs with a fused epilogue for sm_100a: the projections on either side of attention and
// their LoRA side products.
//
// Replaces the reference program matmul_int8 (src/nano_omni/kernels/matmul/matmul_int8.py:53-160, arithmetic of its
// ref_program :209-240):
//   acc[m, n]  = sum_k input[m, k] * weight[n, k]                  (int8 x int8 -> int32)
//   value      = ((float(acc) * weight_scale[n]) * input_scale[m]) [+ bias[n]] [+ residual[m, n]]
//   value      = silu(value) if use_silu;  value *= multiply[m, n] if given;  output[m, n] = bf16(value)
// input int8 [M, K], weight int8 [N, K] (both K-major), output / residual / multiply bf16 [M, N], bias bf16 [N],
// weight_scale f32 [N, 1], input_scale f32 [M].
// The BF16 form replaces matmul_bf16 (src/nano_omni/kernels/matmul/matmul_bf16.py:29-160, ref_program :183-207):
// bf16 operands, fp32 accumulation, value = acc * output_scale, then the same bias / residual / SiLU / multiply.
//
// Persistent CTAs, one per SM, walk the output tiles of 128 x 256 (N fastest, so that the CTAs in flight share A
// panels in L2).  Warp 0: TMA producer, K in chunks of 128 bytes through a 4-stage ring (A 16 KiB + B 32 KiB per
// stage, 128-byte swizzle, no multicast).  Warp 1: tcgen05 issuer, kind::i8 MMAs of 128 x 256 x 32 (kind::f16 MMAs of
// 128 x 256 x 16 for bf16: the same 32 bytes of K per instruction) into one of two
// 256-column 32-bit accumulators in TMEM, so that the MMAs of the next tile run while warps 2-9 drain the previous
// one: a thread owns one row of one 128-column half, requests its residual / multiply operands, reads 64 columns
// with tcgen05.ld and applies the epilogue in the ref_program's order with separately rounded fp32 operations.
// Every wait is bounded.
#include <cuda.h>

#include "common.cuh"
#include "tensor_map.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

constexpr int kBM = 128, kBN = 256, kBK = 128;  // bytes along K: 128 int8 or 64 bf16 elements
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK, kBBytes = kBN * kBK;
constexpr int kThreads = 320;  // producer, issuer, eight epilogue warps (two per TMEM lane quarter)
constexpr uint32_t kTmemCols = 512;

struct __align__(1024) GemmShared {
  uint8_t a[kStages][kABytes];
  uint8_t b[kStages][kBBytes];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
};

struct GemmParams {
  const float* weight_scale;
  const float* input_scale;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* multiply;
  __nv_bfloat16* output;
  int m, n, k, use_silu;  // k in bytes of a row
  float output_scale;     // bf16 form only
  uint32_t* status;
};

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
matmul_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  GemmShared& S = *reinterpret_cast<GemmShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &S.abort;
  uint32_t* status = P.status;
  const int m_tiles = (P.m + kBM - 1) / kBM, n_tiles = (P.n + kBN - 1) / kBN;
  const int num_tiles = m_tiles * n_tiles;
  const int k_chunks = (P.k + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&S.full[s], 1);
      mbar_init(&S.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&S.acc_full[b], 1);
      mbar_init(&S.acc_empty[b], 8);
    }
    S.abort = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&S.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = S.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      int issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile / n_tiles) * kBM, n0 = (tile % n_tiles) * kBN;
        for (int kc = 0; kc < k_chunks; ++kc, ++issued) {
          const int st = issued % kStages;
          if (issued >= kStages) {
            ok = mbar_wait(&S.empty[st], ((issued / kStages) - 1) & 1, abort_flag, status, kWaitTimeoutRing);
            if (!ok) break;
          }
          mbar_expect_tx(&S.full[st], kABytes + kBBytes);
          constexpr int kElementsPerChunk = BF16 ? kBK / 2 : kBK;
          tma_load_3d(S.a[st], &map_a, &S.full[st], kc * kElementsPerChunk, m0, 0);
          tma_load_3d(S.b[st], &map_b, &S.full[st], kc * kElementsPerChunk, n0, 0);
        }
      }
      if (*abort_flag) {  // gave up: let the copies in flight land before the CTA exits
        for (int i = (issued > kStages ? issued - kStages : 0); i < issued; ++i) {
          uint64_t* bar = &S.full[i % kStages];
          const uint32_t parity = (i / kStages) & 1;
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(bar, parity); ++spin) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- tcgen05 issuer
    if (lane == 0) {
      constexpr uint32_t idesc = BF16 ? umma_idesc(kDF32, kFmtBF16, kFmtBF16, 0, 0, kBM, kBN)
                                      : umma_idesc(kDS32, kFmtS8, kFmtS8, 0, 0, kBM, kBN);
      const uint64_t desc = umma_smem_desc(0, 16, 1024, kSwizzle128B);
      const uint64_t a0 = desc + (smem_u32(S.a[0]) >> 4), b0 = desc + (smem_u32(S.b[0]) >> 4);
      int taken = 0, round = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++round) {
        const int buf = round & 1;
        if (round >= 2) {  // the epilogue must have drained this accumulator (its (round / 2)-th use)
          ok = mbar_wait(&S.acc_empty[buf], ((round >> 1) - 1) & 1, abort_flag, status, kWaitTimeoutSoftmax);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t d = tmem + buf * kBN;
        for (int kc = 0; kc < k_chunks; ++kc, ++taken) {
          const int st = taken % kStages;
          ok = mbar_wait(&S.full[st], (taken / kStages) & 1, abort_flag, status, kWaitTimeoutLoad);
          if (!ok) break;
          tc_fence_after();
          const uint64_t a = a0 + st * (kABytes >> 4), b = b0 + st * (kBBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss<BF16 ? 0 : 1>(d, a + 2 * kk, b + 2 * kk, idesc, (kc > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&S.empty[st]);
        }
        if (ok) tc_commit(&S.acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;         // TMEM lanes [32 quarter, 32 quarter + 32)
    const int column_half = (warp - 2) >> 2;  // warps 2-5 drain columns 0-127 of the tile, warps 6-9 columns 128-255
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    int round = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++round) {
      const int buf = round & 1;
      const int m0 = (tile / n_tiles) * kBM, n0 = (tile % n_tiles) * kBN;
      const int row = m0 + row_in_tile;
      const bool live = row < P.m;
      const float in_scale = (!BF16 && live) ? P.input_scale[row] : 0.f;
      ok = __all_sync(0xffffffffu, mbar_wait(&S.acc_full[buf], (round >> 1) & 1, abort_flag, status, kWaitTimeoutMma));
      if (!ok) break;
      tc_fence_after();
      const size_t row_offset = static_cast<size_t>(live ? row : 0) * P.n;
#pragma unroll 1
      for (int c = column_half * (kBN / 128); c < (column_half + 1) * (kBN / 128); ++c) {
        // 64 columns per step.  Residual and multiply operands are requested before the accumulator is read, all at
        // once: their latency, not their bandwidth, bounds the epilogue of a short-K product.
        const int col0 = n0 + 64 * c;
        uint4 res[8], mul[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const bool in = live && col0 + 8 * g < P.n;
          res[g] = (in && P.residual) ? *reinterpret_cast<const uint4*>(P.residual + row_offset + col0 + 8 * g)
                                      : make_uint4(0, 0, 0, 0);
          mul[g] = (in && P.multiply) ? *reinterpret_cast<const uint4*>(P.multiply + row_offset + col0 + 8 * g)
                                      : make_uint4(0, 0, 0, 0);
        }
        uint32_t acc[64];
        __syncwarp();  // lanes that skipped the stores of the previous step rejoin before the aligned TMEM load
        tmem_ld32(tmem + lane_base + buf * kBN + 64 * c, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
        tmem_ld32(tmem + lane_base + buf * kBN + 64 * c + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
        tc_wait_ld();
        if (c == (column_half + 1) * (kBN / 128) - 1) {
          // the accumulator is in registers: the issuer may start the tile after next on it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&S.acc_empty[buf]);
        }
        if (!live || col0 >= P.n) continue;
#pragma unroll
        for (int g = 0; g < 8; ++g) {  // 8 columns = 16 bytes of bf16 at a time
          const int col = col0 + 8 * g;
          if (col >= P.n) break;
          float v[8];
          if constexpr (BF16) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__uint_as_float(acc[8 * g + i]), P.output_scale);
          } else {
            const float4 w0 = *reinterpret_cast<const float4*>(P.weight_scale + col);
            const float4 w1 = *reinterpret_cast<const float4*>(P.weight_scale + col + 4);
            const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
              v[i] = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int>(acc[8 * g + i])), ws[i]), in_scale);
          }
          if (P.bias) {
            const uint4 raw = *reinterpret_cast<const uint4*>(P.bias + col);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              v[2 * i] = __fadd_rn(v[2 * i], bf16_lo(w[i]));
              v[2 * i + 1] = __fadd_rn(v[2 * i + 1], bf16_hi(w[i]));
            }
          }
          if (P.residual) {
            const uint32_t w[4] = {res[g].x, res[g].y, res[g].z, res[g].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              v[2 * i] = __fadd_rn(v[2 * i], bf16_lo(w[i]));
              v[2 * i + 1] = __fadd_rn(v[2 * i + 1], bf16_hi(w[i]));
            }
          }
          if (P.use_silu) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fdividef(v[i], 1.0f + __expf(-v[i]));
          }
          if (P.multiply) {
            const uint32_t w[4] = {mul[g].x, mul[g].y, mul[g].z, mul[g].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              v[2 * i] = __fmul_rn(v[2 * i], bf16_lo(w[i]));
              v[2 * i + 1] = __fmul_rn(v[2 * i + 1], bf16_hi(w[i]));
            }
          }
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            o[i] = *reinterpret_cast<const uint32_t*>(&pair);
          }
          *reinterpret_cast<uint4*>(P.output + row_offset + col) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace
}  // namespace nob200

namespace nob200 {
namespace {

template <bool BF16>
int launch_matmul(const char* name, int num_tokens, const void* input, const void* weight, int n, int k,
                  GemmParams params, void* stream) {
  const int element = BF16 ? 2 : 1;
  CUtensorMap ma, mb;
  const CUtensorMapDataType dtype = BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const uint64_t pitch = static_cast<uint64_t>(k) * element;
  int rc;
  if ((rc = make_tensor_map_3d(&ma, dtype, input, k, num_tokens, 1, pitch, pitch * num_tokens, kBK / element, kBM, 1)))
    return rc;
  if ((rc = make_tensor_map_3d(&mb, dtype, weight, k, n, 1, pitch, pitch * n, kBK / element, kBN, 1))) return rc;
  params.m = num_tokens;
  params.n = n;
  params.k = k * element;
  params.status = status_word_device_ptr();
  if (!params.status) return fail(kCudaError, "%s: no current CUDA device", name);

  auto kernel = matmul_kernel<BF16>;
  const size_t smem = sizeof(GemmShared) + 1024;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess)
    return fail(kCudaError, "%s: cannot reserve %zu B of shared memory: %s", name, smem, cudaGetErrorString(err));
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const long long tiles = static_cast<long long>((num_tokens + kBM - 1) / kBM) * ((n + kBN - 1) / kBN);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(ma, mb, params);
  return check_launch(name);
}

}  // namespace
}  // namespace nob200

extern "C" int nob200_matmul_int8(int num_tokens, const void* input, const void* weight, const void* bias,
                                  const void* residual, const void* multiply, void* output, const void* weight_scale,
                                  const void* input_scale, int n, int k, int use_silu, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(num_tokens > 0 && n > 0 && k > 0, "matmul_int8: sizes must be positive");
  NOB_REQUIRE(input && weight && output && weight_scale && input_scale, "matmul_int8: NULL tensor");
  NOB_REQUIRE(k % 16 == 0, "matmul_int8: k (%d) must be a multiple of 16 (row pitch of the TMA tiles)", k);
  NOB_REQUIRE(n % 8 == 0, "matmul_int8: n (%d) must be a multiple of 8 (16-byte rows of the bf16 epilogue)", n);
  GemmParams params = {};
  params.weight_scale = static_cast<const float*>(weight_scale);
  params.input_scale = static_cast<const float*>(input_scale);
  params.bias = static_cast<const __nv_bfloat16*>(bias);
  params.residual = static_cast<const __nv_bfloat16*>(residual);
  params.multiply = static_cast<const __nv_bfloat16*>(multiply);
  params.output = static_cast<__nv_bfloat16*>(output);
  params.use_silu = use_silu != 0;
  return launch_matmul<false>("matmul_int8", num_tokens, input, weight, n, k, params, stream);
}

extern "C" int nob200_matmul_bf16(int num_tokens, const void* input, const void* weight, const void* bias,
                                  const void* residual, const void* multiply, void* output, float output_scale, int n,
                                  int k, int use_silu, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(num_tokens > 0 && n > 0 && k > 0, "matmul_bf16: sizes must be positive");
  NOB_REQUIRE(input && weight && output, "matmul_bf16: NULL tensor");
  NOB_REQUIRE(k % 8 == 0, "matmul_bf16: k (%d) must be a multiple of 8 (row pitch of the TMA tiles)", k);
  NOB_REQUIRE(n % 8 == 0, "matmul_bf16: n (%d) must be a multiple of 8 (16-byte rows of the bf16 epilogue)", n);
  GemmParams params = {};
  params.bias = static_cast<const __nv_bfloat16*>(bias);
  params.residual = static_cast<const __nv_bfloat16*>(residual);
  params.multiply = static_cast<const __nv_bfloat16*>(multiply);
  params.output = static_cast<__nv_bfloat16*>(output);
  params.output_scale = output_scale;
  params.use_silu = use_silu != 0;
  return launch_matmul<true>("matmul_bf16", num_tokens, input, weight, n, k, params, stream);
}
