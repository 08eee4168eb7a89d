"""BF16 GEMM with the fused epilogue and the projection operator (LoRA chain, int8 path) on the GPU against the CPU
restatement of the reference ref_programs.

The tensor cores accumulate fp32 in their own order, so the bf16 GEMM is compared with a float64-accumulated oracle
at a tolerance of a few bf16 ulps of the result (rtol 2^-7) plus an absolute term for cancelled sums.  The int8
projection without LoRA is exact; with LoRA the residual that enters the int8 GEMM carries the bf16 GEMM's rounding.
"""

import pytest
import torch

from oracle import reference_math as rm
from tests.gpu_util import desc, run

pytestmark = pytest.mark.gpu


def operands(M, N, K, seed, bias, residual, multiply):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * K**-0.5).bfloat16()
    b = (torch.randn(N, generator=g) * 0.5).bfloat16() if bias else None
    r = torch.randn(M, N, generator=g).bfloat16() if residual else None
    m = torch.randn(M, N, generator=g).bfloat16() if multiply else None
    return x, w, b, r, m


def gemm(x, w, b, r, m, scale, use_silu):
    from nano_omni_b200.kernels.matmul import MatmulBf16Arguments, MatmulBf16Kernel

    out = torch.full((x.shape[0], w.shape[0]), float("nan"), dtype=torch.bfloat16, device="cuda")
    d = lambda t: desc(t.cuda()) if t is not None else None  # noqa: E731
    run(MatmulBf16Kernel(MatmulBf16Arguments(d(x), d(w), d(b), d(r), d(m), desc(out), scale, use_silu)))
    return out.cpu()


@pytest.mark.parametrize(
    "M,N,K", [(1, 8, 8), (17, 8, 24), (130, 264, 72), (128, 256, 64), (129, 512, 320), (1000, 1792, 256), (300, 32, 5376), (300, 280, 32)]
)
@pytest.mark.parametrize(
    "bias,residual,multiply,silu,scale", [(False, False, False, False, 1.0), (True, True, False, False, 0.25), (True, True, True, True, 1.0)]
)
def test_matches_oracle(M, N, K, bias, residual, multiply, silu, scale):
    x, w, b, r, m = operands(M, N, K, 9100 + M + N + K, bias, residual, multiply)
    got = gemm(x, w, b, r, m, scale, silu)
    want = rm.matmul_bf16(x, w, b, r, m, scale, silu)
    assert torch.isfinite(got.float()).all()
    torch.testing.assert_close(got.float(), want.float(), rtol=2**-7, atol=2e-3)


def test_exact_for_exactly_representable_sums():
    """Small integers: every product and partial sum is exact in fp32, so the result must equal the oracle's."""
    g = torch.Generator().manual_seed(9190)
    x = torch.randint(-4, 5, (257, 192), generator=g).bfloat16()
    w = torch.randint(-4, 5, (264, 192), generator=g).bfloat16()
    got = gemm(x, w, None, None, None, 1.0, False)
    want = rm.matmul_bf16(x, w)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_many_tiles_per_cta():
    x, w, b, r, m = operands(4096, 2560, 192, 9191, True, False, False)
    got = gemm(x, w, b, r, m, 1.0, False)
    torch.testing.assert_close(got.float(), rm.matmul_bf16(x, w, b).float(), rtol=2**-7, atol=2e-3)


def linear_case(M, N, K, rank, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    ws = torch.rand(N, 1, generator=g) * 2e-4 + 1e-5
    bias = (torch.randn(N, generator=g) * 0.5).bfloat16()
    residual = torch.randn(M, N, generator=g).bfloat16()
    loras = tuple(
        ((torch.randn(rank, K, generator=g) * K**-0.5).bfloat16(), (torch.randn(N, rank, generator=g) * rank**-0.5).bfloat16(), s)
        for s in (0.75, -0.5)
    )
    return x, w, ws, bias, residual, loras


def run_linear(x, w, ws, bias, residual, loras, rotation_group):
    from nano_omni_b200.ops import Linear

    d = lambda t: desc(t.cuda())  # noqa: E731
    out = torch.full((x.shape[0], w.shape[0]), float("nan"), dtype=torch.bfloat16, device="cuda")
    op = Linear(
        d(x), d(w), weight_scale=d(ws), bias=d(bias), residual=d(residual),
        loras=tuple((d(a), d(b), s) for a, b, s in loras), rotation_group=rotation_group,
    ).to(desc(out))  # fmt: skip
    calls, need = op.prepare()
    scratch = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
    op.run(scratch)
    torch.cuda.synchronize()
    return out.cpu(), [c.name for c in calls]


@pytest.mark.parametrize("rotation_group", [0, 256])
def test_int8_projection_without_lora_is_exact(rotation_group):
    x, w, ws, bias, residual, _ = linear_case(300, 520, 768, 32, 9200 + rotation_group)
    got, names = run_linear(x, w, ws, bias, residual, (), rotation_group)
    assert names == ["convrot_int8" if rotation_group else "int8_rowwise", "matmul_int8"]
    want = rm.linear_int8(x, w, ws, bias=bias, residual=residual, rotation_group=rotation_group)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_int8_projection_with_two_loras():
    x, w, ws, bias, residual, loras = linear_case(300, 520, 768, 32, 9210)
    got, names = run_linear(x, w, ws, bias, residual, loras, 256)
    assert names == ["matmul_bf16"] * 4 + ["convrot_int8", "matmul_int8"]
    want = rm.linear_int8(x, w, ws, bias=bias, residual=residual, loras=loras, rotation_group=256)
    torch.testing.assert_close(got.float(), want.float(), rtol=2**-6, atol=3e-2)
    # the LoRA terms are really in: without them the result differs visibly
    plain = rm.linear_int8(x, w, ws, bias=bias, residual=residual, rotation_group=256)
    assert (got.float() - plain.float()).abs().mean() > 0.2


@pytest.mark.parametrize("case", ["plain", "bias_res", "all"])
def test_both_gemms_against_reference_fixtures(golden_matmul, case):
    """Outputs of the reference's ref_programs (tests/golden/matmul.npz): int8 equal bit for bit without SiLU, bf16
    within one bf16 step (fp32 accumulation order)."""
    from nano_omni_b200.kernels.matmul import MatmulInt8Arguments, MatmulInt8Kernel
    from tests.conftest import bf16

    g = golden_matmul
    use_b, use_r, use_m, silu = {"plain": (0, 0, 0, False), "bias_res": (1, 1, 0, False), "all": (1, 1, 1, True)}[case]
    b = bf16(g["bias"]) if use_b else None
    r = bf16(g["residual"]) if use_r else None
    m = bf16(g["multiply"]) if use_m else None

    def steps(a, c):
        ia, ib = a.view(torch.int16).int(), c.view(torch.int16).int()
        return (torch.where(ia < 0, -(ia & 0x7FFF), ia) - torch.where(ib < 0, -(ib & 0x7FFF), ib)).abs()

    got = gemm(bf16(g["xb"]), bf16(g["wb"]), b, r, m, 0.75, silu)
    d = steps(got, bf16(g[f"bf16_{case}"]))
    assert d.max() <= (2 if silu else 1) and (d > 0).float().mean() < 0.03

    x8, w8 = torch.from_numpy(g["x8"]), torch.from_numpy(g["w8"])
    ws, xs = torch.from_numpy(g["ws"]), torch.from_numpy(g["xs"])
    out = torch.full((x8.shape[0], w8.shape[0]), float("nan"), dtype=torch.bfloat16, device="cuda")
    dd = lambda t: desc(t.cuda()) if t is not None else None  # noqa: E731
    run(MatmulInt8Kernel(MatmulInt8Arguments(dd(x8), dd(w8), dd(b), dd(r), dd(m), desc(out), dd(ws), dd(xs), silu)))
    want = bf16(g[f"int8_{case}"])
    if silu:
        assert steps(out.cpu(), want).max() <= 2
    else:
        assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))
