/*
 * C ABI of libnano_omni_b200.so: sm_100a kernels for the MiniMax-H3 DiT attention
 * path of nano-omni.  One entry point per reference kernel `name`; arguments come
 * in the order the reference launches them (dynamic scalars first, then every
 * tensor in Arguments field order - src/nano_omni/core/kernel.py:208-222), followed
 * by the integers the reference bakes in at compile time (Workload fields) and the
 * CUDA stream.
 *
 * Conventions
 *  - every pointer is a device pointer to a contiguous row-major tensor, 16-byte
 *    aligned; `stream` is a cudaStream_t / CUstream passed as void*;
 *  - entry points only enqueue work: no host synchronisation, no allocation;
 *    scratch memory, where needed, is passed in by the caller (`workspace`), who
 *    sizes it with the matching *_workspace_bytes function;
 *  - return value 0 = enqueued; negative = rejected before launch (-1 invalid
 *    argument, -2 CUDA error, -3 unsupported); nob200_last_error() gives the text
 *    for the calling thread;
 *  - device-side waits are bounded; a kernel whose wait gave up returns early and
 *    ORs a bit into a per-device status word, read (and cleared) with
 *    nob200_read_status().
 */
#ifndef NANO_OMNI_B200_H_
#define NANO_OMNI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NOB200_ABI_VERSION 1

int nob200_abi_version(void);
const char* nob200_last_error(void);
/* Synchronises `stream`, stores the status word of the current device in *out and clears it. */
int nob200_read_status(uint32_t* out, void* stream);

/*
 * dense_bf16_attention_d128 - replaces DenseBf16AttentionKernel
 * (src/nano_omni/kernels/attention/dense_bf16.py:46-268).
 * query/key/value bf16 [num_tokens, heads, 128]; output bf16 [num_tokens, total_heads, 128],
 * heads written at [head_offset, head_offset+heads).  Non-causal, scale 1/sqrt(128).
 */
int nob200_dense_bf16_attention_d128(int num_tokens, int head_offset, const void* query, const void* key,
                                     const void* value, void* output, int heads, int total_heads, void* stream);

/*
 * The same attention with the key tiles divided into kv_splits contiguous shares per (256 query rows, head),
 * each share on its own CTA, merged by a second kernel through their log-sum-exp.  No counterpart in the
 * reference; it exists to fill all 148 SMs when rows/256 * heads is small or just above a multiple of 148
 * (few heads per GPU after the sequence<->head reshard).  workspace holds the bf16 partial outputs and
 * fp32 log-sum-exps.  kv_splits = 1 is nob200_dense_bf16_attention_d128.
 */
size_t nob200_dense_bf16_attention_d128_splitkv_workspace_bytes(int num_tokens, int heads, int kv_splits);
int nob200_dense_bf16_attention_d128_splitkv(int num_tokens, int head_offset, const void* query, const void* key,
                                             const void* value, void* output, int heads, int total_heads,
                                             int kv_splits, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The same attention with the head->sequence reshard of the multi-GPU path fused into its epilogue
 * (no counterpart in the reference, which is single-GPU): this rank holds all `num_tokens` tokens of `heads`
 * heads; output row `token` belongs to rank token / (num_tokens / world) and is written straight into
 * peer_outputs[that rank] - a pointer to that rank's bf16 [num_tokens / world, total_heads, 128] tensor,
 * mapped into this process (peer memory over NVLink) - at its local row and head_offset.  Plain 16-byte
 * stores; the caller orders them against the consumers with nob200_ulysses_barrier.
 */
int nob200_dense_bf16_attention_d128_scatter(int num_tokens, int head_offset, const void* query, const void* key,
                                             const void* value, void* const* peer_outputs, int world, int heads,
                                             int total_heads, int kv_splits, void* workspace, size_t workspace_bytes,
                                             void* stream);

/*
 * dense_int8_fp8_d128 - replaces DenseInt8Fp8AttentionKernel
 * (src/nano_omni/kernels/attention/int8_fp8/dense.py:21-481).
 * query int8 [heads, ceil32(num_query_tokens), 128] with query_scale f32 [heads, rows/32];
 * key int8 [heads, ceil64(num_kv_tokens), 128] with key_scale f32 [heads, rows/64];
 * value e4m3 [heads, 128, ceil64(num_kv_tokens)] (layout of int8_fp8_quantize_value) with
 * value_scale f32 [heads, 128]; output bf16 [num_query_tokens, heads*128].
 * P is rounded to e4m3 before the PV product, which accumulates in fp32.
 */
int nob200_dense_int8_fp8_d128(int num_kv_tokens, int num_query_tokens, const void* query, const void* key,
                               const void* value, const void* query_scale, const void* key_scale,
                               const void* value_scale, void* output, int heads, void* stream);

/*
 * dense_nvfp4_attention_d128 - replaces DenseNvfp4Kernel
 * (src/nano_omni/kernels/attention/dense_nvfp4.py:54-676).
 * query/key packed e2m1 u8 [heads, P, 64] with ue4m3 scales [heads, P, 8]; value packed u8
 * [heads, 128, Pk/2] with scales [heads, 128, Pk/16] (layouts of nvfp4_prepare; P = tokens padded to 128);
 * output bf16 [num_query_tokens, total_heads, 128] at head_offset.
 * Both contractions run as block-scaled fp4 tensor-core instructions (e2m1 codes, one ue4m3 scale per 16 along the
 * contraction).  Probabilities are rounded as the reference rounds them (dense_nvfp4.py:617-668): per 16 keys of a
 * row the scale is e4m3(max / 6) and the codes are e2m1(p / (max / 6)), p carrying the factor 2688; the row sum is
 * taken from the unrounded p.  num_query_tokens and num_kv_tokens may differ (a query slice against all keys).
 * `workspace` / `workspace_bytes` are kept for callers of the earlier signature and ignored (pass NULL, 0);
 * _workspace_bytes returns 0.
 */
size_t nob200_dense_nvfp4_attention_d128_workspace_bytes(int num_query_tokens, int num_kv_tokens, int heads);
int nob200_dense_nvfp4_attention_d128(int num_query_tokens, int num_kv_tokens, int head_offset, const void* query,
                                      const void* key, const void* value, const void* query_scales,
                                      const void* key_scales, const void* value_scales, void* output, int heads,
                                      int total_heads, void* workspace, size_t workspace_bytes, void* stream);
/* packed e2m1 + ue4m3 scales (layouts of nvfp4_prepare) -> bf16 [num_tokens, heads, 128]; exact. */
int nob200_nvfp4_expand(int num_tokens, const void* quantized, const void* scales, void* output, int heads,
                        int transpose, void* stream);

/*
 * token_group_mean - replaces TokenGroupMeanKernel
 * (src/nano_omni/kernels/normalization/token_group_mean.py:51-189).
 * input bf16 [num_tokens, columns]; output f32 [ceil(num_tokens/tokens_per_block), columns].
 * fp32 sums in a fixed order: chunks of 128 tokens summed in token order, chunk sums added
 * in chunk order.  Needs workspace when tokens_per_block > 128.
 */
size_t nob200_token_group_mean_workspace_bytes(int num_tokens, int columns, int tokens_per_block);
int nob200_token_group_mean(int num_tokens, const void* input, void* output, int columns, int tokens_per_block,
                            int include_padding, void* workspace, size_t workspace_bytes, void* stream);

/*
 * token_group_mean_static - the same column mean for callers that cannot provide scratch.
 * No counterpart in the reference.  It is for code that runs where device memory can no longer be
 * obtained: a kernel sequence whose memory plan was fixed before execution started (nano-omni lays out
 * one workspace arena per model and its submit threads may neither allocate nor synchronise), or a
 * host that forbids cudaMalloc on its hot path because the call stalls every stream of the device.
 * The partial sums live in an array built into the library, NOB200_STATIC_MEAN_SCRATCH_BYTES (4 MiB)
 * per GPU for as long as the process runs; a shape that needs more is rejected with -1 and a message
 * naming both sizes (scratch need = groups * ceil(tokens_per_block/128) * columns * 4 bytes; groups of
 * up to 128 tokens need none).  The function calls no cudaMalloc, cudaFree or allocating library routine.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 * first call outside any stream capture.  All calls on a device share the one array, which keeps the
 * previous call's partial sums (nothing has to start at zero: each call overwrites all that it reads),
 * so two calls whose kernels may overlap on the GPU - different streams without an ordering between
 * them - race on it; results equal nob200_token_group_mean bit for bit otherwise.
 */
#define NOB200_STATIC_MEAN_SCRATCH_BYTES (4u << 20)
int nob200_token_group_mean_static(int num_tokens, const void* input, void* output, int columns,
                                   int tokens_per_block, int include_padding, void* stream);

/*
 * int8_fp8_quantize_qk - replaces Int8Fp8QuantizeQKKernel
 * (src/nano_omni/kernels/attention/int8_fp8/quantize_qk.py:18-201).
 * source bf16 [num_tokens, heads*128]; statistics f32 [1, heads*128] (read when center != 0);
 * quantized int8 [heads, padded_tokens, 128]; scales f32 [heads, padded_tokens/tokens_per_block].
 * tokens_per_block in {32, 64, 128}.  `hadamard` != 0 applies a normalised 128-point
 * Walsh-Hadamard rotation over the channels of each head before the absmax; it has no
 * counterpart in the reference (0 reproduces the reference).
 */
int nob200_int8_fp8_quantize_qk(int num_tokens, const void* source, const void* statistics, void* quantized,
                                void* scales, int heads, int tokens_per_block, int center, int hadamard,
                                void* stream);

/*
 * int8_fp8_value_scale - replaces Int8Fp8ValueScaleKernel
 * (src/nano_omni/kernels/attention/int8_fp8/value_scale.py:18-123).
 * source bf16 [num_tokens, heads*128]; scales f32 [heads, 128] = max(max_t |V| / 2.25, 1e-10).
 */
int nob200_int8_fp8_value_scale(int num_tokens, const void* source, void* scales, int heads, void* stream);

/*
 * int8_fp8_quantize_value - replaces Int8Fp8QuantizeValueKernel
 * (src/nano_omni/kernels/attention/int8_fp8/quantize_value.py:20-152).
 * source bf16 [num_tokens, heads*128]; scale f32 [heads, 128];
 * output e4m3 [heads, 128, ceil(num_tokens/64)*64], channel-major, tokens of each group of 16
 * stored in the order [0,1,8,9,2,3,10,11,4,5,12,13,6,7,14,15].
 */
int nob200_int8_fp8_quantize_value(int num_tokens, const void* source, const void* scale, void* output, int heads,
                                   void* stream);

/*
 * nvfp4_prepare - replaces Nvfp4PrepareKernel
 * (src/nano_omni/kernels/attention/nvfp4_prepare.py:37-214).
 * source bf16 [num_tokens, heads*128]; mean f32 [heads, 128] or NULL (no centring);
 * transpose == 0: quantized u8 [heads, P, 64], scales ue4m3 [heads, P, 8]   (P = tokens padded to 128)
 * transpose != 0: quantized u8 [heads, 128, P/2], scales ue4m3 [heads, 128, P/16]
 * scales are stored in 512-byte atoms of 128 rows x 4 groups.
 * `hadamard` as above.  global_scale == 0 reproduces the reference attention quantiser;
 * global_scale > 0 follows the reference's global-scale NVFP4 arithmetic
 * (src/nano_omni/kernels/quantization/quantize_fp4.py:221-262).
 */
int nob200_nvfp4_prepare(int num_tokens, const void* source, const void* mean, void* quantized, void* scales,
                         int heads, int transpose, int hadamard, float global_scale, void* stream);

/*
 * sol_pool - replaces SolPoolKernel, SolInt8Fp8PoolKernel and SolNvfp4PoolKernel
 * (src/nano_omni/kernels/attention/sol/pool.py:29-114, int8_fp8/sol_pool.py:25-119, nvfp4/sol_pool.py:34-125).
 * key/value bf16 [num_tokens, heads, 128]; key_mean f32 [heads, 128] or NULL;
 * output bf16 [2 or 3, heads, blocks, 128]: K block mean, (K block mean - key_mean when key_mean is given),
 * V block sum.  block is 64 (reference) or 128.  Sums run over tokens in index order.
 */
int nob200_sol_pool(int num_tokens, const void* key, const void* value, const void* key_mean, void* output,
                    int heads, int block, void* stream);

/*
 * sol_stats - replaces SolStatsKernel (src/nano_omni/kernels/attention/sol/stats.py:28-103).
 * pooled bf16 [planes, heads, num_blocks, 128] (plane 0 is read); output f32 [heads, 2, 128] = mean and
 * clamped variance of the block means, summed over blocks in index order.
 */
int nob200_sol_stats(const void* pooled, void* output, int heads, int num_blocks, void* stream);

/*
 * sol_nvfp4_select - replaces SolNvfp4SelectKernel (src/nano_omni/kernels/attention/nvfp4/sol_select.py:42-201),
 * the routing mask shared by the int8 and nvfp4 sol paths.
 * query bf16 [num_tokens, heads, 128]; pooled_key bf16 [heads, blocks, 128]; stats f32 [heads, 2, 128];
 * output u8 [blocks, heads, blocks]: 1 where key block < num_protected_blocks, or score > threshold, or
 * |query block - key block| <= 1.  Scores are evaluated in fp32 in a fixed order (see sol_route.cu).
 * topk_blocks > 0 (no counterpart in the reference) replaces the threshold and the neighbour rule by
 * "the topk_blocks highest-scoring unprotected key blocks, ties to the lower index, plus the protected
 * blocks"; it needs nob200_sol_select_workspace_bytes(...) of workspace and at most 2048 blocks.
 */
size_t nob200_sol_select_workspace_bytes(int num_tokens, int heads, int block, int topk_blocks);
int nob200_sol_select(int num_tokens, int num_protected_blocks, const void* query, const void* pooled_key,
                      const void* stats, void* output, int heads, float tau, int block, int topk_blocks,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * sol_attention_d128 - the attention stage of SolAttentionKernel
 * (src/nano_omni/kernels/attention/sol_attention.py:53-432): exact attention over the key blocks selected
 * in `mask`, one pooled pseudo-key (weight = block length) for every other block, one online softmax.
 * The reference evaluates its routing rule inside the kernel; here the rule is evaluated by
 * nob200_sol_select into `mask` (u8 [blocks, heads, blocks]) first, which the caller keeps in op scratch.
 * query/key/value bf16 [num_tokens, heads, 128]; pooled bf16 [pooled_planes, heads, blocks, 128] from
 * nob200_sol_pool (plane 0 = key block means, last plane = value block sums); output bf16
 * [num_tokens, total_heads, 128] at head_offset.  block is 64 or 128 and must match pool and select.
 */
int nob200_sol_attention_d128(int num_tokens, int head_offset, const void* query, const void* key, const void* value,
                              const void* pooled, const void* mask, void* output, int heads, int total_heads,
                              int block, int pooled_planes, void* stream);

/* sol_attention_d128 with output rows stored into their owners' tensors on other GPUs (see
 * nob200_dense_bf16_attention_d128_scatter). */
int nob200_sol_attention_d128_scatter(int num_tokens, int head_offset, const void* query, const void* key,
                                      const void* value, const void* pooled, const void* mask,
                                      void* const* peer_outputs, int world, int heads, int total_heads, int block,
                                      int pooled_planes, void* stream);

/*
 * Exact stage of the int8-fp8 sol path.
 * Replaces SolInt8Fp8AttentionKernel / program sol_int8_fp8_attention_d128
 * (src/nano_omni/kernels/attention/int8_fp8/sol.py:27-225; Arguments :14-26: query, key, value, query_scale,
 * key_scale, value_scale, selected, output, state, num_tokens, head_offset, tau, num_protected_blocks - the last two
 * only size the reference's cost model and have no effect on the result, so they are not parameters here).
 * Operands as nob200_dense_int8_fp8_d128; selected u8 [blocks, heads, blocks] over 64-token blocks.
 * output bf16 [num_tokens, total_heads, 128] at head_offset: the UN-normalised numerator sum_k p_k v_k with
 * p_k = exp((q.k - rowmax) / sqrt(128)); state f32 [num_tokens, total_heads, 2] = (rowmax in raw dequantised q.k
 * units, sum_k p_k).  A row whose block selects nothing gets zeros and (-inf, 0).
 */
int nob200_sol_int8_fp8_attention_d128(int num_tokens, int head_offset, const void* query, const void* key,
                                       const void* value, const void* query_scale, const void* key_scale,
                                       const void* value_scale, const void* selected, void* output, void* state,
                                       int heads, int total_heads, void* stream);

/*
 * Exact stage of the nvfp4 sol path.
 * Replaces SolNvfp4Kernel / program sol_nvfp4_attention_d128 (src/nano_omni/kernels/attention/sol_nvfp4.py:30-813;
 * Arguments: query, key, value, query_scales, key_scales, value_scales, selected, output, state, num_query_tokens,
 * num_kv_tokens, head_offset, tau, num_protected_blocks).  Operands as nob200_dense_nvfp4_attention_d128; key block 0
 * always attends (sol_nvfp4.py:793-796).  output/state as nob200_sol_int8_fp8_attention_d128.  Same block-scaled
 * fp4 kernel and probability rounding (sol_nvfp4.py:764-813) as the dense entry point; each tile of 128 query rows
 * walks only the key blocks its own two query blocks select.  `workspace` is ignored (NULL, 0); _workspace_bytes
 * returns 0.
 */
size_t nob200_sol_nvfp4_attention_d128_workspace_bytes(int num_query_tokens, int num_kv_tokens, int heads);
int nob200_sol_nvfp4_attention_d128(int num_query_tokens, int num_kv_tokens, int head_offset, const void* query,
                                    const void* key, const void* value, const void* query_scales,
                                    const void* key_scales, const void* value_scales, const void* selected,
                                    void* output, void* state, int heads, int total_heads, void* workspace,
                                    size_t workspace_bytes, void* stream);

/* The same exact stage on bf16 operands [num_tokens, heads, 128] (the second half of the call above; no reference
 * counterpart of its own).  block is 64 or 128; force_first_block != 0 attends key block 0 whatever `selected` says. */
int nob200_sol_exact_state_bf16_d128(int num_tokens, int head_offset, const void* query, const void* key,
                                     const void* value, const void* selected, void* output, void* state, int heads,
                                     int total_heads, int block, int force_first_block, void* stream);

/*
 * Merge of the pooled pseudo-keys into an exact stage's numerator and state, and normalisation.
 * Replaces SolNvfp4FinalizeKernel / program sol_nvfp4_finalize
 * (src/nano_omni/kernels/attention/nvfp4/sol_finalize.py:38-270; Arguments: query, pooled, selected, exact, state,
 * output, head_offset).  query bf16 [num_tokens, heads, 128]; pooled bf16 [3, heads, blocks, 128] (plane 1 = centred
 * key block means, plane 2 = value block sums); exact/output bf16 [num_tokens, total_heads, 128], state f32
 * [num_tokens, total_heads, 2], all at head_offset.  Every unselected block kb adds one pseudo-key with logit
 * q . pooled[1][kb] (raw units, compared with state's maximum), weight = its token count, value pooled[2][kb].
 * output may be the same tensor as exact (the reference op binds them so: ops/minimax_h3/sol_int8_fp8_attention.py:117).
 * block (64 in the reference, or 128) must match the exact stage and the router.
 */
int nob200_sol_nvfp4_finalize(int num_tokens, int head_offset, const void* query, const void* pooled,
                              const void* selected, const void* exact, const void* state, void* output, int heads,
                              int total_heads, int block, void* stream);

/* sol_nvfp4_finalize for the multi-GPU path: exact / state are this rank's local tensors [num_tokens, heads, 128|2]
 * (head_offset does not apply to them); output rows go into their owners' tensors [num_tokens / world, total_heads,
 * 128] at head_offset (see nob200_dense_bf16_attention_d128_scatter). */
int nob200_sol_nvfp4_finalize_scatter(int num_tokens, int head_offset, const void* query, const void* pooled,
                                      const void* selected, const void* exact, const void* state,
                                      void* const* peer_outputs, int world, int heads, int total_heads, int block,
                                      void* stream);

/*
 * Variants for operands quantised as the benchmark specification states them (no reference counterpart: the
 * reference quantises Q per 32 and K per 64 tokens without rotation and has no global NVFP4 scale in attention).
 * _blocks: int8 Q / K with one scale per query_block (32, 64, 128) / key_block (64, 128) tokens; the Q and K row
 * counts are padded to those blocks, V as before to 64 tokens.
 * _global: NVFP4 operands whose stored block scales were divided by a global scale per tensor
 * (nob200_nvfp4_prepare with global_scale > 0): value = e2m1 * ue4m3 * global.
 * nob200_nvfp4_expand_scaled: the expansion to bf16 with that multiplier.
 * nob200_hadamard128_rows: the normalised 128-point Walsh-Hadamard transform of the quantisers on bf16 rows
 * [num_rows, 128] (its own inverse; in place allowed): attention on rotated Q and K needs nothing more (the rotation
 * cancels in q.k), attention on rotated V returns rotated rows, which this brings back.  _heads: the same on heads
 * [head_offset, head_offset + heads) of a tensor [tokens, total_heads, 128].
 */
int nob200_dense_int8_fp8_d128_blocks(int num_kv_tokens, int num_query_tokens, const void* query, const void* key,
                                      const void* value, const void* query_scale, const void* key_scale,
                                      const void* value_scale, void* output, int heads, int query_block, int key_block,
                                      void* stream);

/*
 * The same with the key tiles divided over `kv_splits` CTAs per (256 query rows, head), merged through their
 * log-sum-exp: for query slices (few query rows against all keys) whose CTAs would leave the last wave of SMs short.
 * `workspace`: nob200_dense_bf16_attention_d128_splitkv_workspace_bytes(num_query_tokens, heads, kv_splits) bytes
 * (NULL / 0 for kv_splits == 1, which is nob200_dense_int8_fp8_d128_blocks).
 */
int nob200_dense_int8_fp8_d128_splitkv(int num_kv_tokens, int num_query_tokens, const void* query, const void* key,
                                       const void* value, const void* query_scale, const void* key_scale,
                                       const void* value_scale, void* output, int heads, int query_block,
                                       int key_block, int kv_splits, void* workspace, size_t workspace_bytes,
                                       void* stream);
int nob200_dense_nvfp4_attention_d128_global(int num_query_tokens, int num_kv_tokens, int head_offset,
                                             const void* query, const void* key, const void* value,
                                             const void* query_scales, const void* key_scales,
                                             const void* value_scales, float query_global, float key_global,
                                             float value_global, void* output, int heads, int total_heads,
                                             void* workspace, size_t workspace_bytes, void* stream);
int nob200_nvfp4_expand_scaled(int num_tokens, const void* quantized, const void* scales, void* output, int heads,
                               int transpose, float multiplier, void* stream);
int nob200_hadamard128_rows(long long num_rows, const void* input, void* output, void* stream);
int nob200_hadamard128_heads(int tokens, int head_offset, const void* input, void* output, int heads, int total_heads,
                             void* stream);

/*
 * INT8 GEMM with the scaled fused epilogue of the projections around attention.
 * Replaces MatmulInt8Kernel / program matmul_int8 (src/nano_omni/kernels/matmul/matmul_int8.py:53-240; Arguments:
 * input, weight, bias, residual, multiply, output, weight_scale, input_scale, use_silu):
 *   output[m, n] = bf16( f( float(sum_k input[m,k] * weight[n,k]) * weight_scale[n] * input_scale[m]
 *                           [+ bias[n]] [+ residual[m,n]] ) [* multiply[m,n]] ),   f = silu if use_silu else identity.
 * input int8 [num_tokens, k], weight int8 [n, k], bias bf16 [n] or NULL, residual / multiply bf16 [num_tokens, n] or
 * NULL, weight_scale f32 [n, 1], input_scale f32 [num_tokens].  k must be a multiple of 16, n of 8.
 */
int nob200_matmul_int8(int num_tokens, const void* input, const void* weight, const void* bias, const void* residual,
                       const void* multiply, void* output, const void* weight_scale, const void* input_scale, int n,
                       int k, int use_silu, void* stream);

/*
 * BF16 GEMM with the same fused epilogue: the bf16 projections and the LoRA side products of a projection
 * (compress: input x down^T; update: compressed x up^T * strength + residual).
 * Replaces MatmulBf16Kernel / program matmul_bf16 (src/nano_omni/kernels/matmul/matmul_bf16.py:29-207; Arguments:
 * input, weight, bias, residual, multiply, output, output_scale, use_silu):
 *   output[m, n] = bf16( f( (sum_k input[m,k] * weight[n,k]) * output_scale [+ bias[n]] [+ residual[m,n]] )
 *                        [* multiply[m,n]] ),   fp32 accumulation, f = silu if use_silu else identity.
 * input bf16 [num_tokens, k], weight bf16 [n, k], the rest as for nob200_matmul_int8.  k and n must be multiples of 8.
 */
int nob200_matmul_bf16(int num_tokens, const void* input, const void* weight, const void* bias, const void* residual,
                       const void* multiply, void* output, float output_scale, int n, int k, int use_silu,
                       void* stream);

/*
 * Row-wise int8 of the projection inputs.  rotation_group 0 replaces Int8RowwiseKernel / program int8_rowwise
 * (src/nano_omni/kernels/quantization/int8_rowwise.py:18-116); rotation_group 256 replaces ConvRotInt8Kernel / program
 * convrot_int8 (src/nano_omni/kernels/quantization/convrot_int8.py:41-161; Arguments: input, output, scales, group):
 * every group of 256 columns is rotated by the Kronecker power of the reference's 4 x 4 base matrix over 16, rounded to
 * bf16, and the row is quantised with one scale max(amax / 127, 1e-30) to int8 in [-127, 127].
 * input bf16 [num_tokens, columns], output int8 [num_tokens, columns], scales f32 [num_tokens] - the `input` and
 * `input_scale` operands of nob200_matmul_int8.  columns a multiple of 8 (of 256 with rotation).
 */
int nob200_int8_rowwise(int num_tokens, const void* input, void* output, void* scales, int columns, int rotation_group,
                        void* stream);

/*
 * Measurement aid (no reference counterpart): `ctas` CTAs each issue `count` tcgen05.mma of 128 x 128 x K from shared
 * memory (kind 0: bf16, K = 16; 1: int8, K = 32; 2: e4m3, K = 32; 3: block-scaled nvfp4,
 * K = 64, scale factors from unwritten TMEM columns) and store the SM cycles from first issue to
 * completion in cycles[cta] (device memory, -1 if a bounded wait gave up).  `python -m nano_omni_b200.peaks` turns this
 * into the tensor-pipe peak per operand kind.
 */
int nob200_mma_issue_rate(int kind, int count, int ctas, long long* cycles, void* stream);
/*
 * Measurement aid (no reference counterpart): issue rate of the instruction kinds the softmax warps consist of.
 * `ctas` CTAs of `warps` warps each run `iters` rounds of 16 independent instructions of kind `op` (0 ex2.approx,
 * 1 cvt to e4m3x2, 2 cvt to e2m1x2, 3 cvt to bf16x2, 4 fma, 5 three-input max, 6 integer add); cycles[cta * 32 + warp]
 * receives each warp's SM cycles, `sink` (1024 floats) keeps the results alive.  `python -m nano_omni_b200.peaks --pipes`
 * turns this into lanes per clock and SM.
 */
int nob200_pipe_issue_rate(int op, int warps, int iters, int ctas, long long* cycles, float* sink, void* stream);

/*
 * Q and K normalised and rotated in place by one launch (same arithmetic per row as nob200_h3_head_norm_rope, RoPE
 * always on).  Replaces H3QkNormRopeKernel / program h3_qk_norm_rope
 * (src/nano_omni/kernels/specialized/h3_qk_norm_rope.py:33-178; Arguments: query, key, query_weight, key_weight,
 * cosines, sines), the first kernel of the reference's dense bf16 operator
 * (src/nano_omni/ops/minimax_h3/dense_bf16_attention.py:66-80).
 * query, key bf16 [tokens, heads, 128]; weights bf16 [128]; cosines, sines f32 [tokens, 48].
 */
int nob200_h3_qk_norm_rope(int tokens, void* query, void* key, const void* query_weight, const void* key_weight,
                           const void* cosines, const void* sines, int heads, void* stream);

/*
 * Per-head RMS norm and split-half RoPE, the step before every attention path.
 * nob200_h3_head_norm_rope replaces H3HeadNormRopeKernel / program h3_head_norm_rope
 * (src/nano_omni/kernels/specialized/h3_head_norm_rope.py:36-97; Arguments: input, weight, cosines, sines, output):
 * input/output bf16 [tokens, heads, 128] (may be the same tensor), weight bf16 [128], cosines/sines f32
 * [tokens, 48] or both NULL (no rotation).
 * nob200_h3_query_prepare replaces H3QueryPrepareKernel / program h3_query_prepare
 * (src/nano_omni/kernels/specialized/h3_query_prepare.py:42-125; Arguments: source, weight, cosines, sines,
 * quantized, scales): the same norm and rotation on source bf16 [tokens, heads*128], rounded to bf16, then
 * symmetric int8 with one scale per (head, 32 tokens): quantized int8 [heads, ceil32(tokens), 128], scales f32
 * [heads, ceil32(tokens)/32] - the operands nob200_dense_int8_fp8_d128 takes as query and query_scale.
 * Arithmetic is IEEE fp32 in a fixed order (see norm_rope.cu), so results do not depend on the launch shape.
 */
int nob200_h3_head_norm_rope(int tokens, const void* input, const void* weight, const void* cosines,
                             const void* sines, void* output, int heads, void* stream);
int nob200_h3_query_prepare(int tokens, const void* source, const void* weight, const void* cosines,
                            const void* sines, void* quantized, void* scales, int heads, void* stream);

/*
 * Head-group packing for the sequence<->head reshard (Ulysses all-to-all) around attention.
 * No counterpart in the reference, which is single-GPU (src/nano_omni/core/runtime/execution.py:68,86).
 * pack:   src bf16 [tokens, heads, 128] -> dst [world, tokens, heads/world, 128]; slab p goes to rank p.
 * unpack: src [world, tokens, heads/world, 128] (slab p came from rank p) -> dst [tokens, heads, 128].
 */
int nob200_ulysses_pack_heads(const void* src, void* dst, int tokens, int heads, int world, void* stream);
int nob200_ulysses_unpack_heads(const void* src, void* dst, int tokens, int heads, int world, void* stream);

/*
 * The same reshard over peer memory, without send buffers or a library collective (no counterpart in the
 * reference either):
 * push:    this rank's query/key/value bf16 [tokens, heads, 128] are written straight into every rank's
 *          receive buffer peer_buffers[p], laid out [3, world, tokens, heads/world, 128] (tensor, source rank);
 * barrier: stores `epoch` into slot [rank] of every rank's flag array peer_flags[p] (8 x u32, zero-initialised,
 *          epochs increasing) and waits until all slots of its own array reached `epoch`.  The wait is bounded
 *          (2 s unless nob200_set_wait_budget_ns changed it): when it runs out the kernel sets bit 4 (value 16)
 *          of the device status word and returns.  From then on, and until nob200_read_status clears the word,
 *          the attention kernels with a scatter epilogue store nothing into other ranks' tensors: their input
 *          was incomplete.  A caller that sees the bit must treat the step's output as invalid on every rank.
 * All pointers are device addresses valid in this process (local memory or mapped peer memory).
 * nob200_set_wait_budget_ns sets the barrier's wait budget for this process, 1 us to 60 s.
 */
int nob200_ulysses_push_heads(const void* query, const void* key, const void* value, void* const* peer_buffers,
                              int tokens, int heads, int world, int rank, void* stream);
/* The same for a group of each rank's heads: heads [head_begin, head_begin + group_heads) of every rank's heads / world
 * go to receive buffers laid out [3, world, tokens, group_heads, 128], so that a caller can push one group while the
 * previous one is attended. */
int nob200_ulysses_push_head_group(const void* query, const void* key, const void* value, void* const* peer_buffers,
                                   int tokens, int heads, int world, int rank, int head_begin, int group_heads,
                                   void* stream);
int nob200_ulysses_barrier(void* const* peer_flags, int world, int rank, unsigned epoch, void* stream);
/*
 * Reshard of quantised operands (quantise before the exchange: int8 / e4m3 / e2m1 bytes and their scales cross
 * NVLink instead of bf16).  push_blocks: `source` holds, head-major, `rows` rows of `row_bytes` bytes for each of
 * `heads` heads (the layouts the quantisers write: [heads, tokens, 128] bytes, [heads, 128, tokens] bytes,
 * [heads, blocks] f32); head p * heads / world + hh is stored into peer_destinations[p] as head hh, each row at
 * hh * destination_head_stride + row * destination_pitch + destination_offset, so that a rank's token range lands
 * inside the destination's full-sequence tensor.  Sizes in bytes, multiples of 16.
 * push_output: the reverse reshard after an attention that wrote a local tensor: bf16 [num_tokens, local_heads, 128]
 * of this rank's heads; every row goes to its owner's [num_tokens / world, total_heads, 128] tensor at heads
 * rank * local_heads + hh.  Stores nothing after a barrier time-out, like the scatter epilogues.
 */
int nob200_ulysses_push_blocks(const void* source, void* const* peer_destinations, int heads, int world, int rows,
                               long long row_bytes, long long destination_head_stride, long long destination_pitch,
                               long long destination_offset, void* stream);
int nob200_ulysses_push_output(const void* source, void* const* peer_outputs, int num_tokens, int local_heads,
                               int total_heads, int world, int rank, void* stream);
int nob200_set_wait_budget_ns(unsigned long long nanoseconds);

#ifdef __cplusplus
}
#endif

#endif /* NANO_OMNI_B200_H_ */
