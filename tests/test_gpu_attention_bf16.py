"""Dense bf16 attention on the GPU against the fp32 CPU oracle (max-abs <= 2e-2)."""

import pytest
import torch

from oracle import reference_math as rm
from tests.conftest import bf16
from tests.gpu_util import desc, randn_bf16, run

pytestmark = pytest.mark.gpu

TOLERANCE = 2e-2  # max-abs against fp32 math, the bound the bf16 path is held to


def _attend(q, k, v, total_heads=None, head_offset=0):
    from nano_omni_b200.kernels.dense_bf16 import DenseBf16AttentionArguments, DenseBf16AttentionKernel

    T, h, _ = q.shape
    total_heads = total_heads or h
    out = torch.full((T, total_heads, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    run(DenseBf16AttentionKernel(DenseBf16AttentionArguments(desc(q), desc(k), desc(v), desc(out), head_offset)))
    return out


@pytest.mark.parametrize("T", [1, 63, 64, 65, 128, 130, 256, 257, 500, 1000])
def test_small_and_ragged_sizes(T):
    h = 2
    q, k, v = (randn_bf16(10 * T + i, T, h, 128) for i in range(3))
    got = _attend(q, k, v).cpu().float()
    want = rm.dense_attention_fp32(q.cpu(), k.cpu(), v.cpu())
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= TOLERANCE


def test_head_offset_writes_only_its_slice():
    T, h, H = 300, 2, 5
    q, k, v = (randn_bf16(7 + i, T, h, 128) for i in range(3))
    out = _attend(q, k, v, total_heads=H, head_offset=2).cpu().float()
    want = rm.dense_attention_fp32(q.cpu(), k.cpu(), v.cpu())
    assert (out[:, 2:4] - want).abs().max() <= TOLERANCE
    assert torch.isnan(out[:, :2]).all() and torch.isnan(out[:, 4:]).all()


def test_config0_seq4096_heads4():
    """Benchmark configuration 0: batch 1, 4 heads, seq 4096, seed 0, checked against fp32 SDPA on CPU."""
    torch.manual_seed(0)
    q, k, v = (torch.randn(4096, 4, 128).bfloat16().cuda() for _ in range(3))
    got = _attend(q, k, v).cpu().float()
    want = rm.dense_attention_fp32(q.cpu(), k.cpu(), v.cpu())
    assert (got - want).abs().max() <= TOLERANCE
    assert rm.cosine(got, want) > 0.999


def test_outlier_channel_and_large_logits():
    """One K channel x16 (the outlier recipe of the DiT-scale config) and scaled-up Q: sharp softmax,
    the running maximum moves by more than the lazy-rescale threshold."""
    T, h = 2048, 2
    q, k, v = (randn_bf16(50 + i, T, h, 128) for i in range(3))
    k[..., 5] *= 16
    q = (q.float() * 3).bfloat16()
    got = _attend(q, k, v).cpu().float()
    want = rm.dense_attention_fp32(q.cpu(), k.cpu(), v.cpu())
    assert (got - want).abs().max() <= TOLERANCE


def test_matches_reference_golden(golden):
    q, k, v = (bf16(golden[f"att_{n}"]).cuda() for n in "qkv")
    got = _attend(q, k, v).cpu().float()
    want = bf16(golden["att_bf16_out"])[:, 1:3].float()
    torch.testing.assert_close(got, want, rtol=0.02, atol=0.01)


def test_full_size_rows_sum_property():
    """DiT-scale shape (24 heads x 32768 tokens): V = all-ones channel block makes every output
    row equal to 1 in those channels whatever the softmax, and a sampled set of rows is checked
    against the fp32 oracle."""
    T, h = 32768, 24
    torch.manual_seed(1)
    q = torch.randn(T, h, 128).bfloat16().cuda()
    k = torch.randn(T, h, 128).bfloat16().cuda()
    v = torch.randn(T, h, 128).bfloat16()
    v[..., :8] = 1.0
    v = v.cuda()
    got = _attend(q, k, v)
    assert (got[..., :8].float() - 1.0).abs().max() <= 1e-2
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 4095, 20000, 32767])
    heads = [0, 11, 23]
    # rows of Q against all keys: small enough for the CPU oracle
    qs = q[rows][:, heads].cpu().float().transpose(0, 1)
    ks = k[:, heads].cpu().float().transpose(0, 1)
    vs = v[:, heads].cpu().float().transpose(0, 1)
    want = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs).transpose(0, 1)
    assert (got[rows][:, heads].cpu().float() - want).abs().max() <= TOLERANCE


@pytest.mark.parametrize("T,splits", [(2048, 2), (2100, 3), (5000, 5)])
def test_split_kv_matches_single_pass(T, splits):
    """Key tiles divided over several CTAs and merged through the log-sum-exp: same result as one pass."""
    from nano_omni_b200.core import DType
    from nano_omni_b200.kernels.dense_bf16 import (
        DenseBf16AttentionArguments,
        DenseBf16AttentionConfig,
        DenseBf16AttentionKernel,
        splitkv_workspace_bytes,
    )

    h, H = 2, 3
    q, k, v = (randn_bf16(300 + T + i, T, h, 128) for i in range(3))
    k[..., 7] *= 8
    out = torch.full((T, H, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(splitkv_workspace_bytes(T, h, splits), dtype=torch.uint8, device="cuda")
    args = DenseBf16AttentionArguments(desc(q), desc(k), desc(v), desc(out), 1, desc(ws, DType.U8))
    run(DenseBf16AttentionKernel(args, DenseBf16AttentionConfig(kv_splits=splits)))
    want = rm.dense_attention_fp32(q.cpu(), k.cpu(), v.cpu())
    assert (out[:, 1:3].cpu().float() - want).abs().max() <= TOLERANCE
    assert torch.isnan(out[:, 0]).all()
    single = _attend(q, k, v)
    # the shares are rounded to bf16 before the merge: up to two bf16 steps from the single pass
    torch.testing.assert_close(out[:, 1:3].float(), single.float(), rtol=2.0**-6, atol=1e-2)


def test_choose_kv_splits_fills_the_gpu():
    from nano_omni_b200.kernels.dense_bf16 import choose_kv_splits

    assert choose_kv_splits(32768, 24) == 1   # 3072 CTAs: 20.8 waves already
    assert choose_kv_splits(32768, 3) > 1     # 384 CTAs = 2.6 waves
