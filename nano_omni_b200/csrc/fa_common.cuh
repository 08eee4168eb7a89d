// Device helpers shared by the attention kernels: register reallocation between warpgroups,
// exp2 on the MUFU and on the FMA pipe, bf16 packing and packed fp32x2 arithmetic.
#pragma once

#include "common.cuh"

namespace nob200 {

template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// ---- packed fp32x2 arithmetic (two lanes of a 64-bit register pair)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x for a pair on the FMA pipe: x = n + r with n = round(x), r in [-0.5, 0.5];
// 2^r by a degree-3 polynomial (relative error 7.5e-5, below bf16 resolution),
// n added into the exponent field.  x is clamped at -126 (result ~1e-38).
__device__ __forceinline__ void exp2_poly_pair(uint64_t x, float& y0, float& y1) {
  const uint64_t magic = pack2(12582912.f, 12582912.f);
  const uint64_t neg_magic = pack2(-12582912.f, -12582912.f);
  float x0, x1;
  unpack2(x, x0, x1);
  x = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t t = add2(x, magic);
  const uint64_t n = add2(t, neg_magic);
  const uint64_t r = fma2(n, pack2(-1.f, -1.f), x);
  uint64_t p = fma2(pack2(0.0551716648042202f, 0.0551716648042202f), r, pack2(0.2426111251115799f, 0.2426111251115799f));
  p = fma2(p, r, pack2(0.6932609677314758f, 0.6932609677314758f));
  p = fma2(p, r, pack2(0.9999280571937561f, 0.9999280571937561f));
  float t0, t1, p0, p1;
  unpack2(t, t0, t1);
  unpack2(p, p0, p1);
  y0 = __uint_as_float(__float_as_uint(p0) + (__float_as_uint(t0) << 23));
  y1 = __uint_as_float(__float_as_uint(p1) + (__float_as_uint(t1) << 23));
}

// ---- waits of the attention kernels (all 32 lanes of a converged warp call them; the result is warp-uniform)
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Gives up (warp-uniformly) when the CTA's abort flag is up or `start` lies more than the wait budget back; the
// first warp to give up raises the flag and records `bit` in the status word.
__device__ __forceinline__ bool warp_gives_up(uint64_t& start, volatile uint32_t* abort_flag, uint32_t* status,
                                              uint32_t bit) {
  const uint64_t now = global_timer_ns();
  if (start == 0) start = now;
  if (!__any_sync(0xffffffffu, *abort_flag != 0 || now - start > kWaitBudgetNs)) return false;
  if ((threadIdx.x & 31) == 0 && *abort_flag == 0) {
    *abort_flag = 1;
    atomicOr(status, bit);
  }
  return true;
}
// Polls mbarrier.test_wait.  For waits on the kernel's critical hand-overs: a warp suspended in try_wait was seen
// to resume hundreds of cycles after the phase completed, and the slowest warp of a tile sets the tile's pace.
__device__ __forceinline__ bool warp_poll(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status, uint32_t bit) {
  uint64_t start = 0;
  for (uint32_t spins = 1; !__all_sync(0xffffffffu, mbar_test(bar, parity)); ++spins) {
    if ((spins & 0x3FF) == 0 && warp_gives_up(start, abort_flag, status, bit)) return false;
  }
  return true;
}
// Suspends in mbarrier.try_wait.  For waits with slack: a polling warp takes issue slots from the softmax warps of
// its scheduler.
__device__ __forceinline__ bool warp_rest(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status, uint32_t bit) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, status, bit));
}
// Waits until a shared-memory counter written by another warp of the CTA has reached `target`.
__device__ __forceinline__ bool warp_wait_counter(const uint32_t* counter, uint32_t target,
                                                  volatile uint32_t* abort_flag, uint32_t* status, uint32_t bit) {
  uint64_t start = 0;
  for (uint32_t spins = 1; !__all_sync(0xffffffffu, *reinterpret_cast<const volatile uint32_t*>(counter) >= target);
       ++spins) {
    __nanosleep(64);
    if ((spins & 0x3FF) == 0 && warp_gives_up(start, abort_flag, status, bit)) return false;
  }
  return true;
}
// One lane of a converged warp.  The issuing warps run all 32 lanes through warp-uniform control flow and put only
// the tcgen05 instructions themselves under this predicate: the compiler then keeps descriptors and addresses in
// uniform registers, which is where tcgen05.mma reads them from.  With a single active lane (`if (lane == 0)`)
// they live in ordinary registers and every MMA pays moves into uniform registers: about 100 instead of 64 cycles
// per MMA for the issuing thread.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

// Where output rows go.  tokens_per_rank == 0: all rows to peer[0] (the local output tensor).
// tokens_per_rank > 0: row `token` belongs to rank token / tokens_per_rank and is stored straight into
// that rank's output tensor (a peer pointer over NVLink) at its local row index: the head->sequence
// reshard of the multi-GPU path happens in the epilogue, without a collective.
constexpr int kMaxWorld = 8;
struct OutRoute {
  __nv_bfloat16* peer[kMaxWorld];
  int tokens_per_rank;
  __device__ __forceinline__ __nv_bfloat16* row(int token, int total_heads, int head) const {
    if (tokens_per_rank == 0) return peer[0] + (static_cast<size_t>(token) * total_heads + head) * 128;
    const int owner = token / tokens_per_rank;
    return peer[owner] + (static_cast<size_t>(token - owner * tokens_per_rank) * total_heads + head) * 128;
  }
};

// A scatter epilogue stores into other ranks' tensors only while no cross-rank barrier has timed out: after a
// timeout this rank's input was incomplete and its rows must not overwrite the peers' outputs.
__device__ __forceinline__ bool route_open(const OutRoute& route, const uint32_t* status) {
  if (route.tokens_per_rank == 0) return true;
  uint32_t word;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(word) : "l"(status));
  return (word & kWaitTimeoutPeer) == 0;
}

// Merge of key-split shares (normalised bf16 partial outputs [split][token][head][128] and their log-sum-exp in log2
// units) into the routed output; defined beside the bf16 attention kernel.
int launch_merge_splits(const __nv_bfloat16* partial_out, const float* partial_lse, const OutRoute& route, int num_tokens,
                        int heads, int total_heads, int head_offset, int splits, void* stream);

}  // namespace nob200
