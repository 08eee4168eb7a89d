"""The sol-path oracle against the reference's own ref_program outputs (tests/golden/sol_path.npz).

The reference sums in torch's order, the oracle in a fixed sequential order, so pooled bf16
values may differ by one ulp in rare elements, statistics in the last fp32 bits, and a mask
entry only where a routing score sits on its threshold.
"""

import numpy as np
import pytest
import torch

from oracle import sol_math as sm
from tests.conftest import bf16

CASES = [(300, 2), (1000, 2)]


def _bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    ia = a.view(torch.int16).to(torch.int32)
    ib = b.view(torch.int16).to(torch.int32)
    # map sign-magnitude to a monotone integer line
    ia = torch.where(ia < 0, -(ia & 0x7FFF), ia)
    ib = torch.where(ib < 0, -(ib & 0x7FFF), ib)
    return (ia - ib).abs()


@pytest.mark.parametrize("T,h", CASES)
def test_pool_within_one_ulp(golden_sol, T, h):
    tag = f"T{T}_h{h}"
    k, v = bf16(golden_sol[f"k_{tag}"]), bf16(golden_sol[f"v_{tag}"])
    want2 = bf16(golden_sol[f"pooled_{tag}"])
    got2 = sm.sol_pool(k, v)
    assert got2.shape == want2.shape
    d = _bf16_ulp_distance(got2, want2)
    assert d.max() <= 1 and (d > 0).float().mean() < 1e-3
    kmean = torch.from_numpy(golden_sol[f"kmean_{tag}"])
    want3 = bf16(golden_sol[f"pooled3_{tag}"])
    got3 = sm.sol_pool(k, v, kmean)
    d = _bf16_ulp_distance(got3, want3)
    assert d.max() <= 1 and (d > 0).float().mean() < 1e-3


@pytest.mark.parametrize("T,h", CASES)
def test_stats_close(golden_sol, T, h):
    tag = f"T{T}_h{h}"
    pooled = bf16(golden_sol[f"pooled_{tag}"])
    want = torch.from_numpy(golden_sol[f"stats_{tag}"])
    got = sm.sol_stats(pooled)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("T,h", CASES)
def test_mask_equals_reference_away_from_threshold(golden_sol, T, h):
    tag = f"T{T}_h{h}"
    q = bf16(golden_sol[f"q_{tag}"])
    pooled = bf16(golden_sol[f"pooled_{tag}"])
    stats = torch.from_numpy(golden_sol[f"stats_{tag}"])
    protected = int(golden_sol[f"protected_{tag}"])
    want = torch.from_numpy(golden_sol[f"mask_{tag}"])
    got = sm.sol_select(q, pooled[0], stats, 1.0, protected)
    score, threshold = sm.route_scores(q, pooled[0], stats, 1.0)
    margin = np.abs(score - threshold[:, :, None]) / (np.abs(threshold[:, :, None]) + 1e-6)
    differs = (got != want).numpy()
    assert not (differs & (margin > 1e-5)).any()
    assert differs.mean() < 1e-3
    # the routing is not trivial on this fixture: some blocks beyond the mandatory ones are kept, some dropped
    assert 0.05 < got.float().mean() < 0.95


@pytest.mark.parametrize("T,h", CASES)
def test_sol_attention_matches_reference(golden_sol, T, h):
    tag = f"T{T}_h{h}"
    q, k, v = (bf16(golden_sol[f"{n}_{tag}"]) for n in "qkv")
    pooled = bf16(golden_sol[f"pooled_{tag}"])
    mask = torch.from_numpy(golden_sol[f"mask_{tag}"])
    want = bf16(golden_sol[f"sol_out_{tag}"]).float()
    got = sm.sol_attention(q, k, v, pooled, mask)
    torch.testing.assert_close(got, want, rtol=0.02, atol=0.01)


def test_selector_known_answer_zero_variance_epsilon():
    """Known answer of the reference's own test (tests/test_sol_attention_state.py:73-105):
    with zero statistics the threshold is sqrt(1e-6); a route just below stays off, just above turns on."""
    q = torch.ones(256, 1, 128, dtype=torch.bfloat16)
    pooled = torch.zeros(1, 4, 128, dtype=torch.bfloat16)
    pooled[:, 2] = 0.00004
    pooled[:, 3] = 0.0002
    stats = torch.zeros(1, 2, 128)
    mask = sm.sol_select(q, pooled, stats, 1.0, 0)
    assert int(mask[0, 0, 2]) == 0
    assert int(mask[0, 0, 3]) == 1


def test_topk_keeps_k_plus_protected():
    g = torch.Generator().manual_seed(4)
    T, h = 1024, 2
    q = torch.randn(T, h, 128, generator=g).bfloat16()
    k = torch.randn(T, h, 128, generator=g).bfloat16()
    pooled = sm.sol_pool(k, k, block=128)
    mask = sm.route_topk(q, pooled[0], 0.25, 1, block=128)
    nb = 8
    assert mask.shape == (nb, h, nb)
    assert (mask[:, :, 0] == 1).all()
    assert (mask[:, :, 1:].sum(-1) == 2).all()  # ceil(0.25 * 8) = 2 unprotected blocks per row


# ------------------------------------------------ quantised sol: exact stage (numerator + state) and finalize
QTAG = "T300_h2"


def _quantised_operands(golden, golden_sol, kind):
    """Operands of the exact stage, rebuilt by the oracle quantisers from the fixture's bf16 inputs."""
    from oracle import reference_math as rm

    T, h = 300, 2
    q, k, v = (bf16(golden_sol[f"{n}_{QTAG}"]).reshape(T, h * 128) for n in "qkv")
    kmean = torch.from_numpy(golden_sol[f"q_kmean_{QTAG}"])
    if kind == "int8":
        q8, qs = rm.int8_fp8_quantize_qk(q, kmean, h, 32, False)
        k8, ks = rm.int8_fp8_quantize_qk(k, kmean, h, 64, True)
        vs = rm.int8_fp8_value_scale(v, h)
        v8 = rm.int8_fp8_quantize_value(v, vs, h)
        return rm.int8_fp8_dequantize(q8, k8, v8, qs, ks, vs, T, T)
    q4 = rm.nvfp4_prepare(q, None, h, False)
    k4 = rm.nvfp4_prepare(k, kmean.reshape(h, 128), h, False)
    v4 = rm.nvfp4_prepare(v, None, h, True)
    return (
        rm.nvfp4_dequantize(*q4)[:, :T],
        rm.nvfp4_dequantize(*k4)[:, :T],
        rm.nvfp4_dequantize(*v4).transpose(1, 2)[:, :T],
    )


@pytest.mark.parametrize("kind", ["int8", "nvfp4"])
def test_exact_stage_and_state_match_reference(golden, golden_sol, kind):
    q, k, v = _quantised_operands(golden, golden_sol, kind)
    mask = torch.from_numpy(golden_sol[f"q_mask_{QTAG}"])
    prefix = "i8" if kind == "int8" else "f4"
    want_exact = bf16(golden_sol[f"{prefix}_exact_{QTAG}"]).float()
    want_state = torch.from_numpy(golden_sol[f"{prefix}_state_{QTAG}"])
    if kind == "int8":
        numerator, state = sm.sol_exact_generic(q, k, v, mask, round_probability=sm.round_e4m3, probability_scale=448.0)
    else:
        numerator, state = sm.sol_exact_generic(
            q, k, v, mask, always_first_block=True, round_probability=sm.round_nvfp4_groups, probability_scale=2688.0
        )
    torch.testing.assert_close(state, want_state, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(numerator, want_exact, rtol=2**-6, atol=2e-2)


@pytest.mark.parametrize("prefix", ["i8", "f4"])
def test_finalize_matches_reference(golden_sol, prefix):
    q = bf16(golden_sol[f"q_{QTAG}"])
    pooled = bf16(golden_sol[f"q_pooled3_{QTAG}"])
    mask = torch.from_numpy(golden_sol[f"q_mask_{QTAG}"])
    exact = bf16(golden_sol[f"{prefix}_exact_{QTAG}"])
    state = torch.from_numpy(golden_sol[f"{prefix}_state_{QTAG}"])
    want = bf16(golden_sol[f"{prefix}_final_{QTAG}"]).float()
    got = sm.sol_finalize(q, pooled, mask, exact, state)
    torch.testing.assert_close(got, want, rtol=2**-7, atol=2e-3)
