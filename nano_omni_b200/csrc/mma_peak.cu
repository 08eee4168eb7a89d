// Issue-rate peak of tcgen05.mma on this GPU for the operand kinds the attention kernels use, and for the block-scaled
// fp4 kind they do not use: the denominator for "fraction of the tensor peak" at int8, fp8 and nvfp4, for which no
// library figure is at hand.  One CTA per SM; one thread
// issues `count` MMAs of 128 x 128 x K (both operands K-major in shared memory, 128-byte swizzle, accumulator in
// TMEM), four accumulators round robin, then commits and waits (bounded).  Operand bytes are zero: the rate does not
// depend on the data.  The nvfp4 kind (e2m1 x e2m1 with one ue4m3 scale per 16 elements, K = 64 per MMA) takes its
// scale factors from TMEM columns 384 (A) and 400 (B), which nobody writes: any byte is a valid ue4m3 scale or a NaN,
// and the results are never read.  No counterpart in the reference.
#include <cuda.h>

#include "common.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

struct __align__(1024) PeakShared {
  uint8_t a[16384];  // 128 rows x 128 bytes
  uint8_t b[16384];
  uint64_t done;
  uint32_t tmem_base;
  uint32_t abort;
};

template <int KIND>  // 0: bf16 (K = 16 per MMA), 1: int8 (K = 32), 2: e4m3 (K = 32), 3: nvfp4 block-scaled (K = 64)
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int count, long long* cycles, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  PeakShared& S = *reinterpret_cast<PeakShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  volatile uint32_t* abort_flag = &S.abort;
  if (threadIdx.x == 0) {
    mbar_init(&S.done, 1);
    S.abort = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < 16384 / 4; i += 128) {
    reinterpret_cast<uint32_t*>(S.a)[i] = 0u;
    reinterpret_cast<uint32_t*>(S.b)[i] = 0u;
  }
  if (warp == 0) {
    tmem_alloc(&S.tmem_base, 512);
    tmem_relinquish();
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = S.tmem_base;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = KIND == 0   ? umma_idesc(kDF32, kFmtBF16, kFmtBF16, 0, 0, 128, 128)
                               : KIND == 1 ? umma_idesc(kDS32, kFmtS8, kFmtS8, 0, 0, 128, 128)
                                           : umma_idesc(kDF32, kFmtE4M3, kFmtE4M3, 0, 0, 128, 128);
    const uint64_t da = umma_smem_desc(smem_u32(S.a), 16, 1024, kSwizzle128B);
    const uint64_t db = umma_smem_desc(smem_u32(S.b), 16, 1024, kSwizzle128B);
    // block-scaled instruction descriptor: a/b format e2m1 (1) in bits 7-9 / 10-12, N >> 3 in bits 17-22,
    // scale format ue4m3 (0) in bit 23, M >> 4 in bits 24-28, scale-factor ids 0, K = 64 (bit 31 clear)
    constexpr uint32_t idesc_fp4 = (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
    const long long t0 = clock64();
    for (int it = 0; it < count; it += 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {  // 32-byte K steps
        if constexpr (KIND == 3) {
          asm volatile(
              "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(
                  tmem + 128 * (i % 3)),
              "l"(da + 2 * i), "l"(db + 2 * i), "r"(idesc_fp4), "r"(1u), "r"(tmem + 384), "r"(tmem + 400)
              : "memory");
        } else {
          umma_ss<KIND>(tmem + 128 * i, da + 2 * i, db + 2 * i, idesc, 1);
        }
      }
    }
    tc_commit(&S.done);
    const bool ok = mbar_wait(&S.done, 0, abort_flag, status, kWaitTimeoutMma);
    const long long t1 = clock64();
    cycles[blockIdx.x] = ok ? t1 - t0 : -1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace
}  // namespace nob200

namespace nob200 {
namespace {

// Issue rate of the instruction kinds the softmax warps are made of: every thread runs `iters` rounds of 16
// independent instructions of one kind; cycles[cta * 32 + warp] receives the warp's cycle count.
template <int OP>
__device__ __forceinline__ void pipe_round(float (&x)[16], uint32_t (&u)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if constexpr (OP == 0) {  // exponential on the MUFU
      asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(x[i]));
    } else if constexpr (OP == 1) {  // two fp32 -> two e4m3
      uint16_t d;
      asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(x[i]), "f"(x[(i + 1) & 15]));
      u[i] ^= d;
    } else if constexpr (OP == 2) {  // two fp32 -> two e2m1
      uint16_t d;
      asm volatile("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n\tcvt.u16.u8 %0, b;\n\t}"
                   : "=h"(d)
                   : "f"(x[i]), "f"(x[(i + 1) & 15]));
      u[i] ^= d;
    } else if constexpr (OP == 3) {  // two fp32 -> two bf16
      uint32_t d;
      asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(x[i]), "f"(x[(i + 1) & 15]));
      u[i] ^= d;
    } else if constexpr (OP == 4) {  // fused multiply-add
      asm volatile("fma.rn.f32 %0, %0, %0, %0;" : "+f"(x[i]));
    } else if constexpr (OP == 5) {  // three-input maximum
      asm volatile("max.f32 %0, %0, %1, %2;" : "+f"(x[i]) : "f"(x[(i + 1) & 15]), "f"(x[(i + 2) & 15]));
    } else {  // integer add
      asm volatile("add.u32 %0, %0, %1;" : "+r"(u[i]) : "r"(u[(i + 1) & 15]));
    }
  }
}

template <int OP>
__global__ void pipe_rate_kernel(int iters, long long* cycles, float* sink) {
  float x[16];
  uint32_t u[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] = 0.001f * (threadIdx.x + i), u[i] = threadIdx.x * 17 + i;
  __syncthreads();
  const long long t0 = clock64();
  for (int j = 0; j < iters; ++j) pipe_round<OP>(x, u);
  const long long t1 = clock64();
  float s = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) s += x[i] + u[i];
  if (s == 1.2345f) sink[threadIdx.x] = s;  // keeps the results alive
  if ((threadIdx.x & 31) == 0) cycles[blockIdx.x * 32 + (threadIdx.x >> 5)] = t1 - t0;
}

}  // namespace
}  // namespace nob200

extern "C" int nob200_pipe_issue_rate(int op, int warps, int iters, int ctas, long long* cycles, float* sink,
                                      void* stream) {
  using namespace nob200;
  NOB_REQUIRE(op >= 0 && op <= 6, "pipe_issue_rate: op %d (0 ex2, 1 cvt e4m3x2, 2 cvt e2m1x2, 3 cvt bf16x2, 4 fma, "
              "5 max3, 6 integer add)", op);
  NOB_REQUIRE(warps > 0 && warps <= 32 && iters > 0 && ctas > 0 && ctas <= 65535, "pipe_issue_rate: bad sizes");
  NOB_REQUIRE(cycles && sink, "pipe_issue_rate: NULL result (cycles: ctas x 32 words, sink: 1024 floats)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = warps * 32;
  switch (op) {
    case 0: pipe_rate_kernel<0><<<ctas, threads, 0, s>>>(iters, cycles, sink); break;
    case 1: pipe_rate_kernel<1><<<ctas, threads, 0, s>>>(iters, cycles, sink); break;
    case 2: pipe_rate_kernel<2><<<ctas, threads, 0, s>>>(iters, cycles, sink); break;
    case 3: pipe_rate_kernel<3><<<ctas, threads, 0, s>>>(iters, cycles, sink); break;
    case 4: pipe_rate_kernel<4><<<ctas, threads, 0, s>>>(iters, cycles, sink); break;
    case 5: pipe_rate_kernel<5><<<ctas, threads, 0, s>>>(iters, cycles, sink); break;
    default: pipe_rate_kernel<6><<<ctas, threads, 0, s>>>(iters, cycles, sink); break;
  }
  return check_launch("pipe_issue_rate");
}

extern "C" int nob200_mma_issue_rate(int kind, int count, int ctas, long long* cycles, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(kind >= 0 && kind <= 3, "mma_issue_rate: kind %d (0 bf16, 1 int8, 2 e4m3, 3 nvfp4 block-scaled)", kind);
  NOB_REQUIRE(count > 0 && count % 4 == 0 && count <= (1 << 22), "mma_issue_rate: count must be a multiple of 4 up to 2^22");
  NOB_REQUIRE(ctas > 0 && ctas <= 65535 && cycles, "mma_issue_rate: bad grid or NULL result");
  uint32_t* status = status_word_device_ptr();
  if (!status) return fail(kCudaError, "mma_issue_rate: no current CUDA device");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(PeakShared) + 1024;  // below the 48 KB default limit
  if (kind == 0) mma_peak_kernel<0><<<ctas, 128, smem, s>>>(count, cycles, status);
  if (kind == 1) mma_peak_kernel<1><<<ctas, 128, smem, s>>>(count, cycles, status);
  if (kind == 2) mma_peak_kernel<2><<<ctas, 128, smem, s>>>(count, cycles, status);
  if (kind == 3) mma_peak_kernel<3><<<ctas, 128, smem, s>>>(count, cycles, status);
  return check_launch("mma_issue_rate");
}
