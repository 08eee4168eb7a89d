"""Fused sol block-sparse attention (router + masked exact tiles + pooled pseudo-keys) on the GPU.

Checked against the CPU restatement of the reference's SolAttentionKernel.ref_program
(oracle/sol_math.py, pinned to the reference fixtures) with the reference's tolerance
rtol 0.02 / atol 0.01, and against the reference's own outputs stored in the fixtures.
"""

import pytest
import torch

from oracle import sol_math as sm
from tests.conftest import bf16
from tests.gpu_util import desc, randn_bf16, run
from tests.test_gpu_sol_route import gpu_pool, gpu_stats, structured_keys

pytestmark = pytest.mark.gpu


def sol_attend(q, k, v, pooled, stats, tau, protected, block=64, topk=0.0, total_heads=None, head_offset=0):
    from nano_omni_b200.core import DType
    from nano_omni_b200.kernels.sol import SolAttentionArguments, SolAttentionKernel

    T, h, _ = q.shape
    nb = -(-T // block)
    H = total_heads or h
    out = torch.full((T, H, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    mask = torch.full((nb, h, nb), 9, dtype=torch.uint8, device="cuda")
    ws = torch.empty(nb * nb * h * 4, dtype=torch.uint8, device="cuda") if topk > 0 else None
    run(
        SolAttentionKernel(
            SolAttentionArguments(
                desc(q), desc(k), desc(v), desc(pooled), desc(stats), desc(out), tau, head_offset, protected,
                desc(mask), block, topk, desc(ws, DType.U8) if ws is not None else None,
            )
        )
    )
    return out, mask


@pytest.mark.parametrize("T", [64, 65, 130, 300, 1000, 2100])
@pytest.mark.parametrize("block", [64, 128])
def test_threshold_routing_matches_oracle(T, block):
    h = 2
    q = randn_bf16(60 + T, T, h, 128)
    k = structured_keys(61 + T, T, h, block)
    v = randn_bf16(62 + T, T, h, 128)
    pooled = gpu_pool(k, v, None, block)
    stats = gpu_stats(pooled)
    nb = -(-T // block)
    protected = min(1, nb)
    out, mask = sol_attend(q, k, v, pooled, stats, 1.0, protected, block)
    want_mask = sm.sol_select(q.cpu(), pooled[0].cpu(), stats.cpu(), 1.0, protected, block)
    assert torch.equal(mask.cpu(), want_mask)
    want = sm.sol_attention(q.cpu(), k.cpu(), v.cpu(), pooled.cpu(), want_mask, block)
    got = out.cpu().float()
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, rtol=0.02, atol=0.01)


def test_topk_routing_with_128_blocks_and_head_offset():
    """The benchmark's routing: 128x128 blocks, top 25 % of key blocks plus the protected text blocks."""
    T, h, H = 2048, 2, 5
    block = 128
    q = randn_bf16(70, T, h, 128)
    k = structured_keys(71, T, h, block)
    v = randn_bf16(72, T, h, 128)
    pooled = gpu_pool(k, v, None, block)
    stats = gpu_stats(pooled)
    out, mask = sol_attend(q, k, v, pooled, stats, 1.0, 2, block, topk=0.25, total_heads=H, head_offset=3)
    want_mask = sm.route_topk(q.cpu(), pooled[0].cpu(), 0.25, 2, block)
    assert torch.equal(mask.cpu(), want_mask)
    want = sm.sol_attention(q.cpu(), k.cpu(), v.cpu(), pooled.cpu(), want_mask, block)
    torch.testing.assert_close(out[:, 3:5].cpu().float(), want, rtol=0.02, atol=0.01)
    assert torch.isnan(out[:, :3]).all()


def test_all_blocks_selected_equals_dense():
    """tau very negative selects every block: the result must equal dense attention."""
    from oracle import reference_math as rm

    T, h = 700, 2
    q, k, v = (randn_bf16(80 + i, T, h, 128) for i in range(3))
    pooled = gpu_pool(k, v, None, 64)
    stats = gpu_stats(pooled)
    out, mask = sol_attend(q, k, v, pooled, stats, -1e9, 0, 64)
    assert (mask == 1).all()
    want = rm.dense_attention_fp32(q.cpu(), k.cpu(), v.cpu())
    assert (out.cpu().float() - want).abs().max() <= 2e-2


@pytest.mark.parametrize("T,h", [(300, 2), (1000, 2)])
def test_against_reference_fixtures(golden_sol, T, h):
    tag = f"T{T}_h{h}"
    q, k, v = (bf16(golden_sol[f"{n}_{tag}"]).cuda() for n in "qkv")
    protected = int(golden_sol[f"protected_{tag}"])
    pooled = bf16(golden_sol[f"pooled_{tag}"]).cuda()
    stats = torch.from_numpy(golden_sol[f"stats_{tag}"]).cuda()
    out, _ = sol_attend(q, k, v, pooled, stats, 1.0, protected, 64)
    want = bf16(golden_sol[f"sol_out_{tag}"]).float()
    torch.testing.assert_close(out.cpu().float(), want, rtol=0.02, atol=0.01)


def test_full_size_threshold_mask_bit_exact():
    """The reference's routing (64-token blocks, threshold rule) at S = 131072: the GPU mask of sampled query blocks
    against the oracle for every key block and head, bit for bit, with the pooled planes and statistics the GPU
    kernels produced (those are bit-exact against the oracle at small sizes)."""
    from tests.test_gpu_sol_route import gpu_select

    T, h, block, protected = 131072, 2, 64, 8
    nb = T // block
    q = randn_bf16(94, T, h, 128)
    k = randn_bf16(95, T, h, 128)
    pooled = gpu_pool(k, k, None, block)
    stats = gpu_stats(pooled)
    mask = gpu_select(q, pooled[0].contiguous(), stats, 1.0, protected, block)
    assert mask.shape == (nb, h, nb)
    sampled = [0, 9, 1031, nb - 1]
    want = sm.sol_select(q.cpu(), pooled[0].cpu(), stats.cpu(), 1.0, protected, block, query_blocks=sampled)
    assert torch.equal(mask[sampled].cpu(), want)
    selected = mask[:, :, protected:].float().mean().item()
    assert 0.10 < selected < 0.22  # about Phi(-1) = 15.9 % of the unprotected blocks, plus the diagonal band


def test_full_size_properties():
    """S = 131072, 128-token blocks, top 25 %: size-independent checks at the benchmark's sol shape (4 of its 24 heads).

    V of ones makes every value, and every pooled value sum divided by its block length, equal to one, so the
    merged softmax must return one in every channel whatever the routing.  With V = the token's block index the
    output of a row is a convex combination of block indices: inside [0, blocks - 1], and sampled rows are
    compared with the oracle computed from the kernel's own mask."""
    T, h, block = 131072, 4, 128
    nb = T // block
    q = randn_bf16(90, T, h, 128)
    k = randn_bf16(91, T, h, 128)
    ones = torch.ones(T, h, 128, dtype=torch.bfloat16, device="cuda")
    pooled = gpu_pool(k, ones, None, block)
    stats = gpu_stats(pooled)
    out, mask = sol_attend(q, k, ones, pooled, stats, 1.0, 4, block, topk=0.25)
    assert (mask[:, :, 4:].sum(-1) == 256).all() and (mask[:, :, :4] == 1).all()
    # the mask itself, bit for bit against the oracle, for sampled query blocks x every key block x every head
    sampled = [0, 5, 517, nb - 1]
    want_mask = sm.route_topk(q.cpu(), pooled[0].cpu(), 0.25, 4, block, query_blocks=sampled)
    assert torch.equal(mask[sampled].cpu(), want_mask)
    got = out.float()
    assert torch.isfinite(got).all()
    assert (got - 1.0).abs().max() <= 2**-7
    del out, ones, got
    index = (torch.arange(T, device="cuda") // block).float()
    v = (index / 8)[:, None, None].expand(T, h, 128).to(torch.bfloat16).contiguous()  # multiples of 1/8 up to 128: exact
    pooled = gpu_pool(k, v, None, block)
    out, mask2 = sol_attend(q, k, v, pooled, gpu_stats(pooled), 1.0, 4, block, topk=0.25)
    assert torch.equal(mask, mask2)
    got = out.float()
    assert got.min() >= 0 and got.max() <= (nb - 1) / 8 + 2**-4
    # every channel of a row carries the same value
    assert (got - got[..., :1]).abs().max() <= 2**-5 * got.abs().max()
    # sampled query blocks against the oracle restricted to those rows (all keys are needed)
    rows = torch.cat([torch.arange(b * block, b * block + block) for b in (0, 517, nb - 1)])
    qb = rows // block
    kc, vc, pc = k.cpu().float(), v.cpu().float(), pooled.cpu().float()
    for head in (0, 3):
        scores = (q[rows.cuda(), head].cpu().float() @ kc[:, head].T) / 128**0.5  # [rows, T]
        pooled_scores = (q[rows.cuda(), head].cpu().float() @ pc[0, head].T) / 128**0.5  # [rows, nb]
        selected = mask[qb, head].cpu().bool()  # [rows, nb]
        exact = torch.where(selected.repeat_interleave(block, dim=1), scores, torch.full_like(scores, -torch.inf))
        approx = torch.where(selected, torch.full_like(pooled_scores, -torch.inf), pooled_scores)
        top = torch.maximum(exact.amax(1), approx.amax(1))[:, None]
        pe, pa = torch.exp(exact - top), torch.exp(approx - top)
        numerator = pe @ vc[:, head, 0] + pa @ pc[1, head, :, 0]
        denominator = pe.sum(1) + pa.sum(1) * block
        want = numerator / denominator
        torch.testing.assert_close(got[rows.cuda(), head, 0].cpu(), want, rtol=0.02, atol=0.02)
