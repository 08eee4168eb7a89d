"""The GEMM oracles against the reference's ref_program outputs (tests/golden/matmul.npz).

int8: the reference accumulates exactly (torch._int_mm) and applies the scales in the order the oracle follows, so
outputs without SiLU are equal bit for bit.  bf16: the reference accumulates in fp32 in torch's order, the oracle in
float64; both round the same fp32-level value to bf16, so they differ by at most one bf16 step in rare elements.
"""

import pytest
import torch

from oracle import reference_math as rm
from tests.conftest import bf16

CASES = {"plain": (False, False, False, False), "bias_res": (True, True, False, False), "all": (True, True, True, True)}


def operands(g, case):
    b, r, m, silu = CASES[case]
    return (bf16(g["bias"]) if b else None, bf16(g["residual"]) if r else None, bf16(g["multiply"]) if m else None, silu)


def steps_apart(a, b):
    ia, ib = a.view(torch.int16).int(), b.view(torch.int16).int()
    return (torch.where(ia < 0, -(ia & 0x7FFF), ia) - torch.where(ib < 0, -(ib & 0x7FFF), ib)).abs()


@pytest.mark.parametrize("case", list(CASES))
def test_matmul_int8(golden_matmul, case):
    g = golden_matmul
    b, r, m, silu = operands(g, case)
    got = rm.matmul_int8(torch.from_numpy(g["x8"]), torch.from_numpy(g["w8"]), torch.from_numpy(g["ws"]),
                         torch.from_numpy(g["xs"]), b, r, m, silu)  # fmt: skip
    want = bf16(g[f"int8_{case}"])
    if silu:
        assert steps_apart(got, want).max() <= 1
    else:
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("case", list(CASES))
def test_matmul_bf16(golden_matmul, case):
    g = golden_matmul
    b, r, m, silu = operands(g, case)
    got = rm.matmul_bf16(bf16(g["xb"]), bf16(g["wb"]), b, r, m, 0.75, silu)
    want = bf16(g[f"bf16_{case}"])
    d = steps_apart(got, want)
    assert d.max() <= 1 and (d > 0).float().mean() < 0.02
