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

constexpr int kMaxWorld = 8;

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

// ---- reshard over peer memory (NVLink): no send buffers, no library collective
// push: every rank writes slab [rank] of each peer's receive buffer directly with 16-byte stores.
//   receive buffer of rank p: [3 tensors][world sources][tokens][heads/world][128]
struct PushParams {
  const uint4* src[3];   // Q, K, V of this rank: [tokens, heads, 128]
  uint4* dst[kMaxWorld]; // base of each rank's receive buffer (dst[rank] is the local one)
  int tokens, heads, world, rank;
  int head_begin, group_heads;  // of every rank's heads / world heads, the group that is pushed
};

// receive buffer of rank p for a head group: [3 tensors][world sources][tokens][group_heads][128]
__global__ void __launch_bounds__(256) ulysses_push_kernel(const PushParams P) {
  const int per_rank = P.heads / P.world;
  const int tensor = blockIdx.z;
  const int row_heads = P.world * P.group_heads;  // heads of one token that this launch moves
  const long long pieces = static_cast<long long>(P.tokens) * row_heads * 16;
  const uint4* __restrict__ src = P.src[tensor];
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < pieces; i += 256ll * gridDim.x) {
    const int piece = static_cast<int>(i & 15);
    const long long row = i >> 4;
    const int slot = static_cast<int>(row % row_heads);
    const long long token = row / row_heads;
    const int p = slot / P.group_heads, hh = slot % P.group_heads;
    const long long from = (token * P.heads + p * per_rank + P.head_begin + hh) * 16 + piece;
    const long long slab = (static_cast<long long>(tensor) * P.world + P.rank) * P.tokens + token;
    P.dst[p][(slab * P.group_heads + hh) * 16 + piece] = src[from];
  }
}

// push of head-major byte tensors (quantised operands and their scales): the source holds, for each of `heads` heads,
// `rows` rows of `row_bytes` bytes; head p * heads / world + hh goes to rank p as head hh, row by row, at
// dst[p] + hh * head_stride + row * pitch + offset.
struct PushBlocksParams {
  const uint4* src;
  uint4* dst[kMaxWorld];
  int heads, world, rows;
  long long row_pieces, head_pieces, pitch_pieces, offset_pieces;  // in 16-byte pieces
};

__global__ void __launch_bounds__(256) ulysses_push_blocks_kernel(const PushBlocksParams P) {
  const int per_rank = P.heads / P.world;
  const long long pieces = static_cast<long long>(P.heads) * P.rows * P.row_pieces;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < pieces; i += 256ll * gridDim.x) {
    const long long piece = i % P.row_pieces;
    const long long line = i / P.row_pieces;  // head * rows + row
    const int row = static_cast<int>(line % P.rows);
    const int head = static_cast<int>(line / P.rows);
    const int p = head / per_rank, hh = head % per_rank;
    P.dst[p][hh * P.head_pieces + row * P.pitch_pieces + P.offset_pieces + piece] = P.src[i];
  }
}

// reverse reshard of an attended head slice: src bf16 [num_tokens, local_heads, 128] of this rank's heads; row `token`
// goes to its owner token / (num_tokens / world) at dst[owner][token % ..][rank * local_heads + hh].  Nothing is stored
// once a cross-rank barrier has timed out (the input was incomplete).
struct PushOutputParams {
  const uint4* src;
  uint4* dst[kMaxWorld];
  int num_tokens, local_heads, total_heads, world, rank;
  const uint32_t* status;
};

__global__ void __launch_bounds__(256) ulysses_push_output_kernel(const PushOutputParams P) {
  uint32_t word;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(word) : "l"(P.status));
  if (word & kWaitTimeoutPeer) return;
  const int per_rank = P.num_tokens / P.world;
  const long long pieces = static_cast<long long>(P.num_tokens) * P.local_heads * 16;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < pieces; i += 256ll * gridDim.x) {
    const int piece = static_cast<int>(i & 15);
    const long long line = i >> 4;  // token * local_heads + hh
    const int hh = static_cast<int>(line % P.local_heads);
    const int token = static_cast<int>(line / P.local_heads);
    const int owner = token / per_rank, local = token % per_rank;
    P.dst[owner][((static_cast<long long>(local) * P.total_heads) + P.rank * P.local_heads + hh) * 16 + piece] = P.src[i];
  }
}

// Barrier between the ranks' streams: every rank stores `epoch` into slot [rank] of every peer's flag
// array (release, system scope: the pushes issued earlier on this stream are visible first), then waits
// until all of its own slots have reached `epoch`.  The wait is bounded; on expiry a status bit is set.
struct BarrierParams {
  uint32_t* flags[kMaxWorld];  // flag array (kMaxWorld words) of every rank
  int world, rank;
  uint32_t epoch;
  uint32_t* status;
  uint64_t budget_ns;  // how long to wait for the peers before giving up
};

// Process-wide wait budget of the cross-rank barrier (nob200_set_wait_budget_ns); 2 s unless set.
static uint64_t g_peer_wait_budget_ns = kWaitBudgetNs;

__global__ void ulysses_barrier_kernel(const BarrierParams P) {
  const int peer = threadIdx.x;
  if (peer >= P.world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(P.flags[peer] + P.rank), "r"(P.epoch) : "memory");
  const uint32_t* mine = P.flags[P.rank] + peer;
  const uint64_t start = global_timer_ns();
  for (uint32_t spins = 0;; ++spins) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (static_cast<int32_t>(seen - P.epoch) >= 0) break;
    if ((spins & 0x3FF) == 0x3FF && global_timer_ns() - start > P.budget_ns) {
      atomicOr(P.status, kWaitTimeoutPeer);
      break;
    }
  }
}

}  // namespace
}  // namespace nob200

extern "C" int nob200_ulysses_push_head_group(const void* query, const void* key, const void* value,
                                              void* const* peer_buffers, int tokens, int heads, int world, int rank,
                                              int head_begin, int group_heads, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(tokens > 0 && heads > 0 && world > 0 && world <= kMaxWorld, "ulysses_push_heads: bad sizes");
  NOB_REQUIRE(heads % world == 0, "ulysses_push_heads: heads (%d) must be divisible by the world size (%d)", heads, world);
  NOB_REQUIRE(rank >= 0 && rank < world, "ulysses_push_heads: rank %d outside [0, %d)", rank, world);
  NOB_REQUIRE(head_begin >= 0 && group_heads > 0 && head_begin + group_heads <= heads / world,
              "ulysses_push_heads: head group [%d, %d) outside the %d heads of a rank", head_begin,
              head_begin + group_heads, heads / world);
  NOB_REQUIRE(query && key && value && peer_buffers, "ulysses_push_heads: NULL tensor");
  PushParams params;
  params.src[0] = static_cast<const uint4*>(query);
  params.src[1] = static_cast<const uint4*>(key);
  params.src[2] = static_cast<const uint4*>(value);
  for (int p = 0; p < world; ++p) {
    NOB_REQUIRE(peer_buffers[p], "ulysses_push_heads: NULL buffer for rank %d", p);
    params.dst[p] = static_cast<uint4*>(peer_buffers[p]);
  }
  params.tokens = tokens, params.heads = heads, params.world = world, params.rank = rank;
  params.head_begin = head_begin, params.group_heads = group_heads;
  const long long pieces = static_cast<long long>(tokens) * world * group_heads * 16;
  const int blocks = static_cast<int>(std::min<long long>((pieces + 255) / 256, 148 * 8));
  ulysses_push_kernel<<<dim3(blocks, 1, 3), 256, 0, static_cast<cudaStream_t>(stream)>>>(params);
  return check_launch("ulysses_push_heads");
}

extern "C" int nob200_ulysses_push_heads(const void* query, const void* key, const void* value,
                                         void* const* peer_buffers, int tokens, int heads, int world, int rank,
                                         void* stream) {
  NOB_REQUIRE(world > 0 && heads % world == 0, "ulysses_push_heads: heads (%d) must be divisible by the world size (%d)",
              heads, world);
  return nob200_ulysses_push_head_group(query, key, value, peer_buffers, tokens, heads, world, rank, 0, heads / world,
                                        stream);
}

extern "C" int nob200_ulysses_push_blocks(const void* source, void* const* peer_destinations, int heads, int world,
                                          int rows, long long row_bytes, long long destination_head_stride,
                                          long long destination_pitch, long long destination_offset, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(heads > 0 && rows > 0 && row_bytes > 0 && world > 0 && world <= kMaxWorld, "ulysses_push_blocks: bad sizes");
  NOB_REQUIRE(heads % world == 0, "ulysses_push_blocks: heads (%d) must be divisible by the world size (%d)", heads, world);
  NOB_REQUIRE(row_bytes % 16 == 0 && destination_head_stride % 16 == 0 && destination_pitch % 16 == 0 &&
                  destination_offset % 16 == 0,
              "ulysses_push_blocks: row bytes, head stride, pitch and offset must be multiples of 16");
  NOB_REQUIRE(destination_offset >= 0 && destination_pitch >= row_bytes &&
                  destination_head_stride >= (rows - 1) * destination_pitch + row_bytes,
              "ulysses_push_blocks: rows of %lld bytes overlap at pitch %lld / head stride %lld", row_bytes,
              destination_pitch, destination_head_stride);
  NOB_REQUIRE(source && peer_destinations, "ulysses_push_blocks: NULL tensor");
  PushBlocksParams params;
  params.src = static_cast<const uint4*>(source);
  for (int p = 0; p < world; ++p) {
    NOB_REQUIRE(peer_destinations[p] && reinterpret_cast<uintptr_t>(peer_destinations[p]) % 16 == 0,
                "ulysses_push_blocks: destination of rank %d is NULL or not 16-byte aligned", p);
    params.dst[p] = static_cast<uint4*>(peer_destinations[p]);
  }
  params.heads = heads, params.world = world, params.rows = rows;
  params.row_pieces = row_bytes / 16, params.head_pieces = destination_head_stride / 16;
  params.pitch_pieces = destination_pitch / 16, params.offset_pieces = destination_offset / 16;
  const long long pieces = static_cast<long long>(heads) * rows * params.row_pieces;
  const int blocks = static_cast<int>(std::min<long long>((pieces + 255) / 256, 148 * 8));
  ulysses_push_blocks_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(params);
  return check_launch("ulysses_push_blocks");
}

extern "C" int nob200_ulysses_push_output(const void* source, void* const* peer_outputs, int num_tokens, int local_heads,
                                          int total_heads, int world, int rank, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(num_tokens > 0 && local_heads > 0 && world > 0 && world <= kMaxWorld, "ulysses_push_output: bad sizes");
  NOB_REQUIRE(num_tokens % world == 0, "ulysses_push_output: tokens (%d) must be divisible by the world size (%d)",
              num_tokens, world);
  NOB_REQUIRE(rank >= 0 && rank < world && (rank + 1) * local_heads <= total_heads,
              "ulysses_push_output: heads [%d, %d) outside the %d heads of the output", rank * local_heads,
              (rank + 1) * local_heads, total_heads);
  NOB_REQUIRE(source && peer_outputs, "ulysses_push_output: NULL tensor");
  PushOutputParams params;
  params.src = static_cast<const uint4*>(source);
  for (int p = 0; p < world; ++p) {
    NOB_REQUIRE(peer_outputs[p], "ulysses_push_output: NULL output of rank %d", p);
    params.dst[p] = static_cast<uint4*>(peer_outputs[p]);
  }
  params.num_tokens = num_tokens, params.local_heads = local_heads, params.total_heads = total_heads;
  params.world = world, params.rank = rank;
  params.status = status_word_device_ptr();
  if (!params.status) return fail(kCudaError, "ulysses_push_output: no current CUDA device");
  const long long pieces = static_cast<long long>(num_tokens) * local_heads * 16;
  const int blocks = static_cast<int>(std::min<long long>((pieces + 255) / 256, 148 * 8));
  ulysses_push_output_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(params);
  return check_launch("ulysses_push_output");
}

extern "C" int nob200_ulysses_barrier(void* const* peer_flags, int world, int rank, unsigned epoch, void* stream) {
  using namespace nob200;
  NOB_REQUIRE(world > 0 && world <= kMaxWorld && rank >= 0 && rank < world, "ulysses_barrier: bad world/rank");
  NOB_REQUIRE(peer_flags, "ulysses_barrier: NULL flag table");
  BarrierParams params;
  for (int p = 0; p < world; ++p) {
    NOB_REQUIRE(peer_flags[p], "ulysses_barrier: NULL flag array for rank %d", p);
    params.flags[p] = static_cast<uint32_t*>(peer_flags[p]);
  }
  params.world = world, params.rank = rank, params.epoch = epoch;
  params.status = status_word_device_ptr();
  if (!params.status) return fail(kCudaError, "ulysses_barrier: no current CUDA device");
  params.budget_ns = g_peer_wait_budget_ns;
  ulysses_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(params);
  return check_launch("ulysses_barrier");
}

extern "C" int nob200_set_wait_budget_ns(unsigned long long nanoseconds) {
  using namespace nob200;
  NOB_REQUIRE(nanoseconds >= 1000ull && nanoseconds <= 60ull * 1000000000ull,
              "set_wait_budget_ns: %llu ns outside [1 us, 60 s]", nanoseconds);
  g_peer_wait_budget_ns = nanoseconds;
  return kOk;
}

extern "C" int nob200_ulysses_pack_heads(const void* src, void* dst, int tokens, int heads, int world, void* stream) {
  return nob200::launch(true, src, dst, tokens, heads, world, stream);
}
extern "C" int nob200_ulysses_unpack_heads(const void* src, void* dst, int tokens, int heads, int world,
                                           void* stream) {
  return nob200::launch(false, src, dst, tokens, heads, world, stream);
}
