"""Norm + RoPE kernels on the GPU: bit-exact against the CPU restatement (same fixed summation order), and within
the rounding-boundary allowance against the reference's ref_program outputs."""

import pytest
import torch

from oracle import reference_math as rm
from tests.conftest import bf16
from tests.gpu_util import desc, run

pytestmark = pytest.mark.gpu


def inputs(T, h, seed):
    g = torch.Generator().manual_seed(seed)
    source = (torch.randn(T, h, 128, generator=g) * 3).bfloat16()
    source[:, :, 7] *= 12  # an outlier channel
    weight = (1 + 0.2 * torch.randn(128, generator=g)).bfloat16()
    angle = torch.rand(T, 48, generator=g) * 6.2831853
    return source, weight, torch.cos(angle).contiguous(), torch.sin(angle).contiguous()


def head_norm_rope(source, weight, cosines, sines, in_place=False):
    from nano_omni_b200.kernels.norm_rope import H3HeadNormRopeArguments, H3HeadNormRopeKernel

    src = source.cuda()
    out = src if in_place else torch.full_like(src, float("nan"))
    c = desc(cosines.cuda()) if cosines is not None else None
    s = desc(sines.cuda()) if sines is not None else None
    run(H3HeadNormRopeKernel(H3HeadNormRopeArguments(desc(src), desc(weight.cuda()), c, s, desc(out))))
    return out.cpu()


def query_prepare(source2d, weight, cosines, sines, h):
    from nano_omni_b200.kernels.norm_rope import H3QueryPrepareArguments, H3QueryPrepareKernel

    T = source2d.shape[0]
    rows = -(-T // 32) * 32
    q = torch.full((h, rows, 128), 99, dtype=torch.int8, device="cuda")
    s = torch.full((h, rows // 32), float("nan"), device="cuda")
    c = desc(cosines.cuda()) if cosines is not None else None
    sn = desc(sines.cuda()) if sines is not None else None
    run(H3QueryPrepareKernel(H3QueryPrepareArguments(desc(source2d.cuda()), desc(weight.cuda()), c, sn, desc(q), desc(s))))
    return q.cpu(), s.cpu()


@pytest.mark.parametrize("T", [1, 31, 32, 33, 130, 1000])
@pytest.mark.parametrize("rope", [False, True])
def test_bit_exact_against_oracle(T, rope):
    h = 3
    source, weight, cosines, sines = inputs(T, h, 8000 + T)
    c, s = (cosines, sines) if rope else (None, None)
    want = rm.h3_head_norm_rope(source, weight, c, s)
    got = head_norm_rope(source, weight, c, s)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    again = head_norm_rope(source, weight, c, s, in_place=True)
    assert torch.equal(again.view(torch.int16), want.view(torch.int16))
    want_q, want_s = rm.h3_query_prepare(source.reshape(T, h * 128), weight, c, s, h)
    got_q, got_s = query_prepare(source.reshape(T, h * 128), weight, c, s, h)
    assert torch.equal(got_s, want_s)
    assert torch.equal(got_q, want_q)


def test_result_does_not_depend_on_the_launch_shape():
    """The same rows inside a larger problem (another grid) give the same bytes."""
    h = 2
    source, weight, cosines, sines = inputs(5000, h, 8100)
    whole = head_norm_rope(source, weight, cosines, sines)
    part = head_norm_rope(source[:300].contiguous(), weight, cosines[:300].contiguous(), sines[:300].contiguous())
    assert torch.equal(whole[:300].view(torch.int16), part.view(torch.int16))


def test_against_reference_fixtures(golden_norm_rope):
    g = golden_norm_rope
    source, weight = bf16(g["source"]), bf16(g["weight"])
    T, h, _ = source.shape
    cosines, sines = torch.from_numpy(g["cosines"]), torch.from_numpy(g["sines"])
    for rope in (False, True):
        c, s = (cosines, sines) if rope else (None, None)
        got = head_norm_rope(source, weight, c, s)
        want = bf16(g[f"head_norm_rope_{int(rope)}"])
        ia, ib = got.view(torch.int16).int(), want.view(torch.int16).int()
        d = (torch.where(ia < 0, -(ia & 0x7FFF), ia) - torch.where(ib < 0, -(ib & 0x7FFF), ib)).abs()
        assert d.max() <= 1 and (d > 0).float().mean() < 5e-3
        q, sc = query_prepare(source.reshape(T, h * 128), weight, c, s, h)
        torch.testing.assert_close(sc, torch.from_numpy(g[f"query_s_{int(rope)}"]), rtol=2**-7, atol=0)
        dq = (q.int() - torch.from_numpy(g[f"query_q_{int(rope)}"]).int()).abs()
        assert dq.max() <= 1 and (dq > 0).float().mean() < 2e-2


def test_query_prepare_feeds_the_int8_attention():
    """norm + RoPE + quantise in one kernel equals head_norm_rope followed by the int8 Q quantiser."""
    from nano_omni_b200.kernels.quantize import Int8Fp8QuantizeQKArguments, Int8Fp8QuantizeQKKernel

    T, h = 777, 4
    source, weight, cosines, sines = inputs(T, h, 8200)
    fused_q, fused_s = query_prepare(source.reshape(T, h * 128), weight, cosines, sines, h)
    rotated = head_norm_rope(source, weight, cosines, sines).reshape(T, h * 128).cuda()
    rows = -(-T // 32) * 32
    q = torch.empty(h, rows, 128, dtype=torch.int8, device="cuda")
    s = torch.empty(h, rows // 32, device="cuda")
    unused = torch.zeros(1, h * 128, device="cuda")
    run(Int8Fp8QuantizeQKKernel(Int8Fp8QuantizeQKArguments(desc(rotated), desc(unused), desc(q), desc(s), h, 32, False)))
    assert torch.equal(fused_q, q.cpu()) and torch.equal(fused_s, s.cpu())


def rowwise(source, group):
    from nano_omni_b200.kernels.matmul import (
        ConvRotInt8Arguments,
        ConvRotInt8Kernel,
        Int8RowwiseArguments,
        Int8RowwiseKernel,
    )

    rows, columns = source.shape
    q = torch.full((rows, columns), 99, dtype=torch.int8, device="cuda")
    s = torch.full((rows,), float("nan"), device="cuda")
    if group:
        run(ConvRotInt8Kernel(ConvRotInt8Arguments(desc(source.cuda()), desc(q), desc(s), group)))
    else:
        run(Int8RowwiseKernel(Int8RowwiseArguments(desc(source.cuda()), desc(q), desc(s))))
    return q.cpu(), s.cpu()


@pytest.mark.parametrize("rows,columns", [(1, 256), (37, 768), (200, 5376), (9, 14336)])
@pytest.mark.parametrize("group", [0, 256])
def test_rowwise_int8_bit_exact(rows, columns, group):
    g = torch.Generator().manual_seed(8300 + rows + columns)
    source = (torch.randn(rows, columns, generator=g) * 1.7).bfloat16()
    source[:, 17] *= 11
    if rows > 1:
        source[1] = 0  # an all-zero row: scale 1e-30, zeros out
    want_q, want_s = rm.int8_rowwise(source, group)
    got_q, got_s = rowwise(source, group)
    assert torch.equal(got_s, want_s)
    assert torch.equal(got_q, want_q)


def test_rowwise_without_rotation_on_ragged_width():
    source = (torch.randn(33, 264, generator=torch.Generator().manual_seed(8400)) * 3).bfloat16()  # 256 + 8 columns
    want_q, want_s = rm.int8_rowwise(source, 0)
    got_q, got_s = rowwise(source, 0)
    assert torch.equal(got_s, want_s) and torch.equal(got_q, want_q)


def test_rowwise_quantiser_feeds_the_gemm():
    """Rotated int8 activations x int8 weights rotated the same way reproduce the unrotated product (the rotation is
    orthonormal), up to the two quantisations."""
    from nano_omni_b200.kernels.matmul import MatmulInt8Arguments, MatmulInt8Kernel

    M, N, K = 300, 512, 768
    g = torch.Generator().manual_seed(8500)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    xq, xs = rowwise(x, 256)
    wq, ws = rowwise(w, 256)  # weights go through the same rotation so that it cancels in the product
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    run(
        MatmulInt8Kernel(
            MatmulInt8Arguments(
                desc(xq.cuda()), desc(wq.cuda()), None, None, None, desc(out), desc(ws.reshape(N, 1).cuda()), desc(xs.cuda()), False
            )
        )
    )
    want = x.float() @ w.float().T
    assert rm.cosine(out.cpu().float(), want) >= 0.999


def qk_norm_rope(query, key, query_weight, key_weight, cosines, sines):
    from nano_omni_b200.kernels.norm_rope import H3QkNormRopeArguments, H3QkNormRopeKernel

    q, k = query.cuda(), key.cuda()
    d = lambda t: desc(t.cuda())  # noqa: E731
    run(H3QkNormRopeKernel(H3QkNormRopeArguments(desc(q), desc(k), d(query_weight), d(key_weight), d(cosines), d(sines))))
    return q.cpu(), k.cpu()


@pytest.mark.parametrize("T,h", [(1, 1), (33, 3), (130, 24), (2048, 5)])
def test_qk_pair_in_place_bit_exact(T, h):
    """The fused Q/K launch is the head kernel applied to each tensor in place
    (reference ref_program: h3_qk_norm_rope.py:178-192)."""
    query, query_weight, cosines, sines = inputs(T, h, 8100 + T)
    key, key_weight, _, _ = inputs(T, h, 8200 + T)
    got_q, got_k = qk_norm_rope(query, key, query_weight, key_weight, cosines, sines)
    want_q = rm.h3_head_norm_rope(query, query_weight, cosines, sines)
    want_k = rm.h3_head_norm_rope(key, key_weight, cosines, sines)
    assert torch.equal(got_q.view(torch.int16), want_q.view(torch.int16))
    assert torch.equal(got_k.view(torch.int16), want_k.view(torch.int16))
    # and equal to the single-tensor kernel
    assert torch.equal(got_k.view(torch.int16), head_norm_rope(key, key_weight, cosines, sines).view(torch.int16))


def test_qk_pair_against_reference_fixture(golden_norm_rope):
    g = golden_norm_rope
    source, weight = bf16(g["source"]), bf16(g["weight"])
    cosines, sines = torch.from_numpy(g["cosines"]), torch.from_numpy(g["sines"])
    got_q, got_k = qk_norm_rope(source, source.clone(), weight, weight, cosines, sines)
    want = bf16(g["head_norm_rope_1"])
    for got in (got_q, got_k):
        ia, ib = got.view(torch.int16).int(), want.view(torch.int16).int()
        d = (torch.where(ia < 0, -(ia & 0x7FFF), ia) - torch.where(ib < 0, -(ib & 0x7FFF), ib)).abs()
        assert d.max() <= 1 and (d > 0).float().mean() < 5e-3


def test_rowwise_rotation_on_rows_wider_than_16384_columns():
    """The width of the DiT's feed-forward activations (4 x 5376): the reference splits this case into a rotation
    kernel and int8_rowwise (ops/matmul/sequence.py:96-116); one fused launch gives the same bytes."""
    from nano_omni_b200.kernels.matmul import ConvRotInt8Arguments, ConvRotInt8Kernel

    rows, columns = 19, 21504
    g = torch.Generator().manual_seed(8300)
    x = (torch.randn(rows, columns, generator=g) * 1.3).bfloat16()
    q = torch.full((rows, columns), 99, dtype=torch.int8, device="cuda")
    s = torch.full((rows,), float("nan"), device="cuda")
    run(ConvRotInt8Kernel(ConvRotInt8Arguments(desc(x.cuda()), desc(q), desc(s), 256)))
    want_q, want_s = rm.int8_rowwise(x, 256)
    assert torch.equal(s.cpu(), want_s) and torch.equal(q.cpu(), want_q)
