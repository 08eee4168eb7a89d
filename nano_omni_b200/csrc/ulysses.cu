// Head-group packing for the sequence<->head reshard around attention (Ulysses).
// The reference is single-GPU (device 0 is hard-wired, src/nano_omni/core/runtime/execution.py:68,86);
// these kernels have no counterpart there.  They are HBM-bound 16-byte copies:
//   pack:   src [tokens, heads, 128] -> dst [world, tokens, heads/world, 128]
//           (slab p is what rank p receives: this rank's tokens, head group p)
//   unpack: src [world, tokens, heads/world, 128] -> dst [tokens, heads, 128]
//           (slab p came from rank p: this rank's tokens, head group p)
#include <algorithm>

#include "common.cuh"
#include "../../include/nano_omni_b200.h"

namespace nob200 {
namespace {

// one thread per 16-byte piece (8 bf16); a (token, head) row of 128 channels has 16 pieces
template <bool PACK>
__global__ void __launch_bounds__(256)
ulysses_move_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int tokens, int heads, int world,
                    long long pieces) {
  const int group = heads / world;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < pieces; i += 256ll * gridDim.x) {
    const int piece = static_cast<int>(i & 15);
    const long long row = i >> 4;  // token * heads + head
    const int head = static_cast<int>(row % heads);
    const long long token = row / heads;
    const int p = head / group, hh = head % group;
    const long long slab = ((static_cast<long long>(p) * tokens + token) * group + hh) * 16 + piece;
    if (PACK) {
      dst[slab] = src[i];
    } else {
      dst[i] = src[slab];
    }
  }
}

int launch(bool pack, const void* src, void* dst, int tokens, int heads, int world, void* stream) {
  NOB_REQUIRE(tokens > 0 && heads > 0 && world > 0, "ulysses: sizes must be positive");
  NOB_REQUIRE(heads % world == 0, "ulysses: heads (%d) must be divisible by the world size (%d)", heads, world);
  NOB_REQUIRE(src && dst, "ulysses: NULL tensor");
  const long long pieces = static_cast<long long>(tokens) * heads * 16;
  const int blocks = static_cast<int>(std::min<long long>((pieces + 255) / 256, 148 * 16));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pack)
    ulysses_move_kernel<true><<<blocks, 256, 0, s>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), tokens,
                                                     heads, world, pieces);
  else
    ulysses_move_kernel<false><<<blocks, 256, 0, s>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst),
                                                      tokens, heads, world, pieces);
  return check_launch(pack ? "ulysses_pack_heads" : "ulysses_unpack_heads");
}

}  // namespace
}  // namespace nob200

extern "C" int nob200_ulysses_pack_heads(const void* src, void* dst, int tokens, int heads, int world, void* stream) {
  return nob200::launch(true, src, dst, tokens, heads, world, stream);
}
extern "C" int nob200_ulysses_unpack_heads(const void* src, void* dst, int tokens, int heads, int world,
                                           void* stream) {
  return nob200::launch(false, src, dst, tokens, heads, world, stream);
}
