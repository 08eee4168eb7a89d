"""The norm + RoPE oracle against the reference's ref_program outputs (tests/golden/norm_rope.npz).

The reference sums the squares in torch's order (and differently in its two ref_programs); the oracle uses the
fixed order of the CUDA kernel.  A different last bit of the inverse RMS moves a result across a bf16 rounding
boundary in a few elements per thousand: bf16 outputs may differ by one ulp there, int8 values by one step.
"""

import pytest
import torch

from oracle import reference_math as rm
from tests.conftest import bf16


def _ulps(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    ia, ib = a.view(torch.int16).to(torch.int32), b.view(torch.int16).to(torch.int32)
    ia = torch.where(ia < 0, -(ia & 0x7FFF), ia)
    ib = torch.where(ib < 0, -(ib & 0x7FFF), ib)
    return (ia - ib).abs()


@pytest.mark.parametrize("rope", [False, True])
def test_head_norm_rope(golden_norm_rope, rope):
    g = golden_norm_rope
    source, weight = bf16(g["source"]), bf16(g["weight"])
    cosines = torch.from_numpy(g["cosines"]) if rope else None
    sines = torch.from_numpy(g["sines"]) if rope else None
    got = rm.h3_head_norm_rope(source, weight, cosines, sines)
    want = bf16(g[f"head_norm_rope_{int(rope)}"])
    d = _ulps(got, want)
    assert d.max() <= 1 and (d > 0).float().mean() < 5e-3


@pytest.mark.parametrize("rope", [False, True])
def test_query_prepare(golden_norm_rope, rope):
    g = golden_norm_rope
    source, weight = bf16(g["source"]), bf16(g["weight"])
    T, h, _ = source.shape
    cosines = torch.from_numpy(g["cosines"]) if rope else None
    sines = torch.from_numpy(g["sines"]) if rope else None
    q, s = rm.h3_query_prepare(source.reshape(T, h * 128), weight, cosines, sines, h)
    want_q, want_s = torch.from_numpy(g[f"query_q_{int(rope)}"]), torch.from_numpy(g[f"query_s_{int(rope)}"])
    torch.testing.assert_close(s, want_s, rtol=2**-7, atol=0)
    d = (q.int() - want_q.int()).abs()
    assert d.max() <= 1 and (d > 0).float().mean() < 2e-2
    same_scale = (s == want_s)[:, :, None, None].expand(h, s.shape[1], 32, 128).reshape(h, -1, 128)
    assert (d[same_scale] > 0).float().mean() < 5e-3


def test_rowwise_int8_and_group_rotation(golden_norm_rope):
    """int8_rowwise is plain arithmetic: equal.  convrot_int8 multiplies by the 256 x 256 rotation in the GEMM's order,
    the oracle runs four radix-4 stages: a different last bit can move a value across a bf16 rounding boundary."""
    g = golden_norm_rope
    source = bf16(g["rowwise_src"])
    q, s = rm.int8_rowwise(source)
    assert torch.equal(q, torch.from_numpy(g["rowwise_q"])) and torch.equal(s, torch.from_numpy(g["rowwise_s"]))
    q, s = rm.int8_rowwise(source, 256)
    want_q, want_s = torch.from_numpy(g["convrot_q"]), torch.from_numpy(g["convrot_s"])
    torch.testing.assert_close(s, want_s, rtol=2**-7, atol=0)
    d = (q.int() - want_q.int()).abs()
    assert d.max() <= 1 and (d[(s == want_s)] > 0).float().mean() < 5e-3
