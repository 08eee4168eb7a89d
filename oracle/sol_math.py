"""CPU restatement of the "sol" block-sparse routing path.

TEST INFRASTRUCTURE ONLY (same rule as ``oracle/reference_math.py``): imported by
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``.

The reference computes pooling, statistics and routing scores with torch reductions
whose summation order is torch's own, and its kernel and ``ref_program`` even differ
in order (kernel: per-token bf16 MMA then mean, sol_select.py:90-107; ref: mean first,
then fp32 einsum, sol_select.py:183-197).  Block masks can only be compared bit for
bit if the order is fixed, so this module fixes one (the one the CUDA kernels use):

* sums over the tokens of a block and over blocks are sequential fp32 additions in
  index order, starting from the first element;
* dot products over the 128 channels are sequential ``acc = acc + (a*b)`` with the
  product and the sum each rounded to fp32 (no fused multiply-add);
* divisions, square roots are IEEE fp32.

Pinning: ``tests/golden/make_golden.py`` stores the reference ``ref_program`` results;
``tests/test_oracle_golden.py`` checks these functions against them - pooled tensors
to one bf16 ulp, statistics to 1e-6, masks identical except where a score lies within
1e-5 (relative) of its threshold, attention outputs to the reference tolerance.
Top-k routing over 128-token blocks (``route_topk``) restates the benchmark specification's
sentence and has no counterpart in the reference: parity unpinned.
"""

from __future__ import annotations

import math

import numpy as np
import torch

F32 = np.float32
SQRT128 = F32(math.sqrt(128.0))


def _seq_sum(x: np.ndarray, axis: int) -> np.ndarray:
    """Sequential fp32 sum along ``axis`` (index order, first element first)."""
    x = np.moveaxis(x.astype(np.float32, copy=False), axis, 0)
    acc = x[0].copy()
    for i in range(1, x.shape[0]):
        acc = acc + x[i]
    return acc


def _seq_dot(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """sum_d a[..., d] * b[..., d] with every product and partial sum rounded to fp32."""
    a = a.astype(np.float32, copy=False)
    b = b.astype(np.float32, copy=False)
    acc = a[..., 0] * b[..., 0]
    for d in range(1, a.shape[-1]):
        acc = acc + a[..., d] * b[..., d]
    return acc


def block_lengths(num_tokens: int, block: int) -> np.ndarray:
    nb = -(-num_tokens // block)
    lengths = np.full(nb, block, dtype=np.float32)
    lengths[-1] = num_tokens - (nb - 1) * block
    return lengths


def block_sums(source: torch.Tensor, block: int) -> np.ndarray:
    """fp32 sums of bf16 [tokens, heads, 128] over blocks of tokens -> [blocks, heads, 128]."""
    tokens, heads, dim = source.shape
    nb = -(-tokens // block)
    x = np.zeros((nb * block, heads, dim), dtype=np.float32)
    x[:tokens] = source.to(torch.float32).numpy()
    return _seq_sum(x.reshape(nb, block, heads, dim), 1)


def sol_pool(key: torch.Tensor, value: torch.Tensor, key_mean: torch.Tensor | None = None, block: int = 64) -> torch.Tensor:
    """Pooled planes, bf16 [2 or 3, heads, blocks, 128].

    plane 0: mean of K over the block's valid tokens; (plane 1 with ``key_mean``: that mean
    minus the global K mean [heads, 128]); last plane: SUM of V over the block.
    src/nano_omni/kernels/attention/sol/pool.py:96-114 and
    src/nano_omni/kernels/attention/int8_fp8/sol_pool.py:99-119 (identical to
    src/nano_omni/kernels/attention/nvfp4/sol_pool.py:104-125).
    """
    lengths = block_lengths(key.shape[0], block)
    kmean = (block_sums(key, block) / lengths[:, None, None]).transpose(1, 0, 2)  # [heads, blocks, 128]
    vsum = block_sums(value, block).transpose(1, 0, 2)
    planes = [kmean]
    if key_mean is not None:
        planes.append(kmean - key_mean.numpy().astype(np.float32)[:, None, :])
    planes.append(vsum)
    return torch.from_numpy(np.stack(planes)).to(torch.bfloat16)


def sol_stats(pooled: torch.Tensor) -> torch.Tensor:
    """Per (head, channel) mean and variance of the block means, f32 [heads, 2, 128].

    src/nano_omni/kernels/attention/sol/stats.py:93-103: var = max(E[x^2] - E[x]^2, 0).
    """
    kmean = pooled[0].to(torch.float32).numpy()  # [heads, blocks, 128]
    nb = F32(kmean.shape[1])
    mean = _seq_sum(kmean, 1) / nb
    second = _seq_sum(kmean * kmean, 1) / nb
    variance = np.maximum(second - mean * mean, F32(0))
    return torch.from_numpy(np.stack((mean, variance), axis=1))


def query_block_means(query: torch.Tensor, block: int = 64) -> np.ndarray:
    """fp32 [blocks, heads, 128]: mean of Q over the block's valid tokens."""
    lengths = block_lengths(query.shape[0], block)
    return block_sums(query, block) / lengths[:, None, None]


def route_scores(
    query: torch.Tensor, pooled_key: torch.Tensor, stats: torch.Tensor, tau: float, block: int = 64, query_blocks=None
):
    """(score [qb, heads, kb], threshold [qb, heads]) of the threshold router; ``query_blocks`` (indices) restricts
    the rows to those query blocks, which keeps full-size checks affordable.

    src/nano_omni/kernels/attention/nvfp4/sol_select.py:183-197:
    score = q_mean . centroid / sqrt(128);
    threshold = q_mean . mu / sqrt(128) + tau * sqrt(max(sum q_mean^2 var / 128, 0) + 1e-6).
    """
    qm = query_block_means(query, block)  # [qb, heads, 128]
    if query_blocks is not None:
        qm = qm[np.asarray(query_blocks)]
    kc = pooled_key.to(torch.float32).numpy()  # [heads, kb, 128]
    st = stats.numpy().astype(np.float32)
    score = _seq_dot(qm[:, :, None, :], kc[None, :, :, :]) / SQRT128
    mean = _seq_dot(qm, st[None, :, 0, :]) / SQRT128
    variance = _seq_dot(qm * qm, st[None, :, 1, :]) / F32(128)
    deviation = np.sqrt(np.maximum(variance, F32(0)) + F32(1e-6))
    threshold = mean + F32(tau) * deviation
    return score, threshold


def sol_select(
    query: torch.Tensor,
    pooled_key: torch.Tensor,
    stats: torch.Tensor,
    tau: float,
    num_protected_blocks: int,
    block: int = 64,
    query_blocks=None,
) -> torch.Tensor:
    """Routing mask u8 [qb, heads, kb]: protected blocks, score above threshold, or |qb - kb| <= 1.

    src/nano_omni/kernels/attention/nvfp4/sol_select.py:178-201.  ``query_blocks`` as in ``route_scores``.
    """
    score, threshold = route_scores(query, pooled_key, stats, tau, block, query_blocks)
    mask = score > threshold[:, :, None]
    mask[:, :, :num_protected_blocks] = True
    rows = np.arange(mask.shape[0]) if query_blocks is None else np.asarray(query_blocks)
    mask |= (np.abs(rows[:, None] - np.arange(mask.shape[2])[None, :]) <= 1)[:, None, :]
    return torch.from_numpy(mask.astype(np.uint8))


def route_topk(
    query: torch.Tensor, pooled_key: torch.Tensor, fraction: float, num_protected_blocks: int, block: int = 128,
    query_blocks=None,
) -> torch.Tensor:  # fmt: skip
    """Top-k routing of the benchmark's sol configuration: every query block keeps the
    k = ceil(fraction * blocks) key blocks with the highest pooled score (ties: lower block
    index first), plus all protected (text) blocks, which do not count against k.
    No counterpart in the reference: parity unpinned.
    """
    qm = query_block_means(query, block)
    if query_blocks is not None:
        qm = qm[np.asarray(query_blocks)]
    kc = pooled_key.to(torch.float32).numpy()
    score = _seq_dot(qm[:, :, None, :], kc[None, :, :, :]) / SQRT128  # [qb, heads, kb]
    nb = score.shape[2]
    k = min(nb, int(math.ceil(fraction * nb)))
    candidate = score.copy()
    candidate[:, :, :num_protected_blocks] = -np.inf
    order = np.argsort(-candidate, axis=-1, kind="stable")  # stable: ties keep the lower index first
    mask = np.zeros(score.shape, dtype=bool)
    np.put_along_axis(mask, order[:, :, :k], True, axis=-1)
    mask &= np.isfinite(candidate)
    mask[:, :, :num_protected_blocks] = True
    return torch.from_numpy(mask.astype(np.uint8))


def sol_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    pooled: torch.Tensor,
    mask: torch.Tensor,
    block: int = 64,
) -> torch.Tensor:
    """Block-sparse attention with pooled correction, fp32 [tokens, heads, 128].

    For query block qb and head h: selected key blocks (mask[qb, h, kb] != 0) attend exactly;
    every other block contributes one pseudo-key with logit q . pooled[0][h, kb] / sqrt(128),
    weight = block length in the denominator and value pooled[-1][h, kb] (sum of V) in the
    numerator.  src/nano_omni/kernels/attention/sol_attention.py:301-395 (there the mask is
    evaluated inline; passing it in lets the same function check the int8/nvfp4 variants'
    select -> exact -> finalize chain, src/nano_omni/kernels/attention/nvfp4/sol_finalize.py:212-270).
    """
    tokens, heads, _ = query.shape
    nb = -(-tokens // block)
    q = query.to(torch.float32)
    k = key.to(torch.float32)
    v = value.to(torch.float32)
    kc = pooled[0].to(torch.float32)  # [heads, blocks, 128]
    vs = pooled[-1].to(torch.float32)
    lengths = torch.from_numpy(block_lengths(tokens, block))
    scale = 128**-0.5
    out = torch.empty(tokens, heads, 128)
    for qb in range(nb):
        rows = slice(qb * block, min((qb + 1) * block, tokens))
        for h in range(heads):
            selected = mask[qb, h].bool()
            token_selected = selected.repeat_interleave(block)[:tokens]
            qq = q[rows, h]
            exact_logits = (qq @ k[token_selected, h].T) * scale
            pooled_logits = (qq @ kc[h, ~selected].T) * scale
            logits = torch.cat((exact_logits, pooled_logits), dim=1)
            m = logits.max(dim=1, keepdim=True).values
            pe = torch.exp(exact_logits - m)
            pp = torch.exp(pooled_logits - m)
            numerator = pe @ v[token_selected, h] + pp @ vs[h, ~selected]
            denominator = pe.sum(1) + pp @ lengths[~selected]
            out[rows, h] = numerator / denominator[:, None]
    return out


# ------------------------------------------------ exact stage + finalize (quantised sol paths)
def sol_exact_generic(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    mask: torch.Tensor,
    block: int = 64,
    always_first_block: bool = False,
    round_probability=None,
    probability_scale: float = 1.0,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Online softmax over the selected key blocks only, returning the un-normalised numerator
    (in probability units) and the state (row maximum in raw q.k units, sum of probabilities).

    Restates src/nano_omni/kernels/attention/int8_fp8/sol.py:167-225 and
    src/nano_omni/kernels/attention/sol_nvfp4.py:764-813: blocks in ascending order, running
    maximum per block, probabilities relative to the running maximum, optionally rounded
    (``round_probability`` applied to ``p * probability_scale``) before the value product.
    ``query``/``key``/``value`` are fp32 [heads, tokens, 128]; ``always_first_block`` is the nvfp4
    stage's rule that key block 0 is always attended.
    """
    heads, tokens, _ = query.shape
    nb = -(-tokens // block)
    scale = 128**-0.5
    numerator_out = torch.zeros(tokens, heads, 128)
    state = torch.zeros(tokens, heads, 2)
    for qb in range(nb):
        rows = slice(qb * block, min((qb + 1) * block, tokens))
        for h in range(heads):
            n = rows.stop - rows.start
            maximum = torch.full((n,), -torch.inf)
            denominator = torch.zeros(n)
            numerator = torch.zeros(n, 128)
            for kb in range(nb):
                if not (mask[qb, h, kb] or (always_first_block and kb == 0)):
                    continue
                keys = slice(kb * block, min((kb + 1) * block, tokens))
                scores = query[h, rows] @ key[h, keys].T
                next_maximum = torch.maximum(maximum, scores.amax(1))
                correction = torch.exp((maximum - next_maximum) * scale)
                probability = torch.exp((scores - next_maximum[:, None]) * scale)
                used = probability
                if round_probability is not None:
                    used = round_probability(probability * probability_scale) / probability_scale
                numerator = numerator * correction[:, None] + used @ value[h, keys]
                denominator = denominator * correction + probability.sum(1)
                maximum = next_maximum
            numerator_out[rows, h] = numerator
            state[rows, h, 0] = maximum
            state[rows, h, 1] = denominator
    return numerator_out, state


def sol_finalize(
    query: torch.Tensor, pooled: torch.Tensor, mask: torch.Tensor, exact: torch.Tensor, state: torch.Tensor, block: int = 64
) -> torch.Tensor:
    """Merge the pooled pseudo-keys of every unselected block into (numerator, max, sum) and normalise.

    src/nano_omni/kernels/attention/nvfp4/sol_finalize.py:212-270: logit = q . pooled[1][kb] (raw units),
    weight = block length, value = pooled[2][kb] (sum of V).  ``query`` bf16/fp32 [tokens, heads, 128],
    ``exact`` [tokens, heads, 128], ``state`` [tokens, heads, 2]; returns fp32 [tokens, heads, 128].
    """
    tokens, heads, _ = query.shape
    nb = -(-tokens // block)
    q = query.to(torch.float32)
    kc = pooled[1].to(torch.float32)
    vs = pooled[2].to(torch.float32)
    lengths = torch.from_numpy(block_lengths(tokens, block))
    scale = 128**-0.5
    out = torch.empty(tokens, heads, 128)
    for qb in range(nb):
        rows = slice(qb * block, min((qb + 1) * block, tokens))
        for h in range(heads):
            unselected = mask[qb, h] == 0
            logits = q[rows, h] @ kc[h, unselected].T  # raw units
            m0 = state[rows, h, 0].to(torch.float32)
            m = torch.maximum(m0, logits.amax(1)) if logits.shape[1] else m0
            correction = torch.exp((m0 - m) * scale)
            correction = torch.where(torch.isfinite(m0), correction, torch.zeros_like(correction))
            p = torch.exp((logits - m[:, None]) * scale)
            numerator = exact[rows, h].to(torch.float32) * correction[:, None] + p @ vs[h, unselected]
            denominator = state[rows, h, 1].to(torch.float32) * correction + p @ lengths[unselected]
            out[rows, h] = numerator / denominator[:, None]
    return out


def round_e4m3(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float8_e4m3fn).to(torch.float32)


def round_nvfp4_groups(x: torch.Tensor) -> torch.Tensor:
    """e2m1 with one e4m3 scale per 16 columns, as the nvfp4 sol stage rounds probabilities
    (src/nano_omni/kernels/attention/sol_nvfp4.py:764-781)."""
    rows, cols = x.shape
    padded = -(-cols // 16) * 16
    v = torch.zeros(rows, padded)
    v[:, :cols] = x
    g = v.reshape(rows, padded // 16, 16)
    block_scale = (g.abs().amax(-1) / 6).clamp(max=448)
    encoded = block_scale.to(torch.float8_e4m3fn).to(torch.float32)
    inverse = torch.where(block_scale == 0, torch.zeros_like(block_scale), 1.0 / block_scale)
    y = g * inverse[..., None]
    from oracle.reference_math import E2M1_VALUES, e2m1_codes

    codes = e2m1_codes(y).long()
    mags = torch.tensor(E2M1_VALUES)[codes & 7]
    q = torch.where(codes >= 8, -mags, mags) * encoded[..., None]
    return q.reshape(rows, padded)[:, :cols]


def dense_attention_rounded_p(
    query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, key_tile: int = 128, probability_scale: float = 2688.0
) -> torch.Tensor:
    """Dense attention with the probabilities rounded to NVFP4 before the value product, as the reference's nvfp4
    kernels do (src/nano_omni/kernels/attention/dense_nvfp4.py:250-289; the arithmetic of its torch restatement in
    src/nano_omni/kernels/attention/sol_nvfp4.py:764-813 with every key block attended): key tiles in ascending
    order, running maximum raised with every tile, p = exp2((s - max) log2e/sqrt(128)) * 2688 rounded per 16 keys to
    e2m1 with a ue4m3 scale, row sum of the unrounded p.  ``key_tile`` is the number of keys between two updates of
    the running maximum: 64 in the reference's restatement, 128 in its dense kernel and in the CUDA kernel here.
    ``query`` [heads, Tq, 128], ``key``/``value`` [heads, Tk, 128] fp32 (dequantised operands).  Returns fp32
    [Tq, heads, 128].
    """
    heads, tq, _ = query.shape
    tk = key.shape[1]
    scale = 128**-0.5
    out = torch.empty(tq, heads, 128)
    for h in range(heads):
        maximum = torch.full((tq,), -torch.inf)
        denominator = torch.zeros(tq)
        numerator = torch.zeros(tq, 128)
        for start in range(0, tk, key_tile):
            keys = slice(start, min(start + key_tile, tk))
            scores = query[h] @ key[h, keys].T
            next_maximum = torch.maximum(maximum, scores.amax(1))
            correction = torch.exp((maximum - next_maximum) * scale)
            probability = torch.exp((scores - next_maximum[:, None]) * scale)
            used = round_nvfp4_groups(probability * probability_scale) / probability_scale
            numerator = numerator * correction[:, None] + used @ value[h, keys]
            denominator = denominator * correction + probability.sum(1)
            maximum = next_maximum
        out[:, h] = numerator / denominator[:, None]
    return out
