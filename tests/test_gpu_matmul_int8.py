"""INT8 GEMM with the fused epilogue on the GPU against the CPU restatement of the reference ref_program
(exact integer accumulation; fp32 epilogue in the same order with separately rounded operations, so results
without SiLU are equal bit for bit)."""

import pytest
import torch

from oracle import reference_math as rm
from tests.gpu_util import desc, run

pytestmark = pytest.mark.gpu


def case(M, N, K, seed, bias, residual, multiply):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    ws = torch.rand(N, 1, generator=g) * 2e-4 + 1e-5
    xs = torch.rand(M, generator=g) * 0.05 + 0.001
    b = (torch.randn(N, generator=g) * 0.5).bfloat16() if bias else None
    r = torch.randn(M, N, generator=g).bfloat16() if residual else None
    m = torch.randn(M, N, generator=g).bfloat16() if multiply else None
    return x, w, ws, xs, b, r, m


def gemm(x, w, ws, xs, b, r, m, use_silu):
    from nano_omni_b200.kernels.matmul import MatmulInt8Arguments, MatmulInt8Kernel

    M, N = x.shape[0], w.shape[0]
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    d = lambda t: desc(t.cuda()) if t is not None else None  # noqa: E731
    run(MatmulInt8Kernel(MatmulInt8Arguments(d(x), d(w), d(b), d(r), d(m), desc(out), d(ws), d(xs), use_silu)))
    return out.cpu()


@pytest.mark.parametrize(
    "M,N,K", [(1, 8, 16), (17, 8, 48), (130, 264, 144), (128, 256, 128), (129, 512, 640), (1000, 1792, 512), (300, 280, 5376)]
)
@pytest.mark.parametrize("bias,residual,multiply,silu", [(False, False, False, False), (True, True, False, False), (True, True, True, True)])
def test_matches_oracle(M, N, K, bias, residual, multiply, silu):
    operands = case(M, N, K, 9000 + M + N + K, bias, residual, multiply)
    got = gemm(*operands, silu)
    x, w, ws, xs, b, r, m = operands
    want = rm.matmul_int8(x, w, ws, xs, b, r, m, silu)
    assert torch.isfinite(got.float()).all()
    if silu:
        torch.testing.assert_close(got.float(), want.float(), rtol=2**-7, atol=1e-3)
    else:
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_many_tiles_per_cta_and_both_accumulators():
    """More tiles than SMs: every CTA walks several tiles and alternates between the two accumulators."""
    M, N, K = 4096, 2560, 384  # 32 x 10 tiles
    operands = case(M, N, K, 9900, True, False, False)
    got = gemm(*operands, False)
    x, w, ws, xs, b, r, m = operands
    want = rm.matmul_int8(x, w, ws, xs, b, r, m, False)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_extreme_operands_do_not_overflow():
    """All operands at the int8 extreme with the reference's largest K: |acc| = 5376 * 127^2 < 2^31."""
    M, N, K = 64, 64, 5376
    x = torch.full((M, K), 127, dtype=torch.int8)
    w = torch.full((N, K), -127, dtype=torch.int8)
    ws, xs = torch.full((N, 1), 1e-6), torch.full((M,), 1.0)
    got = gemm(x, w, ws, xs, None, None, None, False)
    want = rm.matmul_int8(x, w, ws, xs)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
