"""The CPU oracle must reproduce the reference's own ref_program outputs.

Fixtures in tests/golden/dense_path.npz were produced by running the unmodified
reference on CPU (tests/golden/make_golden.py).  Byte/integer results and fp32
scales are compared exactly; the column mean is compared to 1 ulp-scale
tolerance because the reference leaves its summation order to torch.
"""

import numpy as np
import pytest
import torch

from oracle import reference_math as rm
from tests.conftest import bf16, e4m3

CASES = [(130, 2), (500, 3)]


@pytest.mark.parametrize("T,h", CASES)
def test_token_group_mean_close_to_reference(golden, T, h):
    src = bf16(golden[f"src_T{T}_h{h}"])
    for tpb, pad in ((T, False), (64, False), (64, True)):
        want = torch.from_numpy(golden[f"mean_T{T}_h{h}_tpb{tpb}_pad{int(pad)}"])
        got = rm.token_group_mean(src, tpb, pad)
        assert got.shape == want.shape
        # different (but fixed) summation order than torch: a few ulps of the largest partial sum
        torch.testing.assert_close(got, want, rtol=0, atol=2e-5)


@pytest.mark.parametrize("T,h", CASES)
@pytest.mark.parametrize("tpb,center", [(32, False), (64, True), (128, True)])
def test_int8_qk_bit_exact(golden, T, h, tpb, center):
    tag = f"T{T}_h{h}"
    src = bf16(golden[f"src_{tag}"])
    mean = torch.from_numpy(golden[f"mean_{tag}_tpb{T}_pad0"])
    q, s = rm.int8_fp8_quantize_qk(src, mean, h, tpb, center)
    assert np.array_equal(q.numpy(), golden[f"qk_q_{tag}_tpb{tpb}_c{int(center)}"])
    assert np.array_equal(s.numpy(), golden[f"qk_s_{tag}_tpb{tpb}_c{int(center)}"])


@pytest.mark.parametrize("T,h", CASES)
def test_value_scale_and_fp8_bit_exact(golden, T, h):
    tag = f"T{T}_h{h}"
    src = bf16(golden[f"src_{tag}"])
    vs = rm.int8_fp8_value_scale(src, h)
    assert np.array_equal(vs.numpy(), golden[f"vscale_{tag}"])
    v8 = rm.int8_fp8_quantize_value(src, vs, h)
    assert np.array_equal(v8.view(torch.uint8).numpy(), golden[f"v8_{tag}"])


@pytest.mark.parametrize("T,h", CASES)
@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("center", [False, True])
def test_nvfp4_prepare_bit_exact(golden, T, h, transpose, center):
    tag = f"T{T}_h{h}"
    src = bf16(golden[f"src_{tag}"])
    mean = torch.from_numpy(golden[f"mean_{tag}_tpb{T}_pad0"]).reshape(h, 128)
    packed, sf = rm.nvfp4_prepare(src, mean if center else None, h, transpose)
    key = f"{tag}_t{int(transpose)}_c{int(center)}"
    assert np.array_equal(packed.numpy(), golden[f"fp4_q_{key}"])
    assert np.array_equal(sf.numpy(), golden[f"fp4_s_{key}"])


def test_nvfp4_global_scale_bit_exact(golden):
    src = bf16(golden["gfp4_src"])
    packed, sf = rm.nvfp4_prepare(src, None, 1, False, global_scale=0.75)
    assert np.array_equal(packed[0, :130].numpy(), golden["gfp4_q"])
    # the linear-layer quantiser pads scale rows to 128 like the attention one (256 rows here)
    assert np.array_equal(sf[0].numpy(), golden["gfp4_s"])


def test_dense_bf16_attention_matches_reference(golden):
    q, k, v = (bf16(golden[f"att_{n}"]) for n in "qkv")
    want = bf16(golden["att_bf16_out"])[:, 1:3]
    got = rm.dense_bf16_attention(q, k, v)
    assert torch.equal(got, want)
    fp32 = rm.dense_attention_fp32(q, k, v)
    assert (fp32 - want.float()).abs().max() < 2e-2


def _reference_quantised_inputs(golden):
    T, h = 200, 2
    q, k, v = (bf16(golden[f"att_{n}"]).reshape(T, h * 128) for n in "qkv")
    return T, h, q, k, v


def test_dense_int8_fp8_attention_matches_reference(golden):
    T, h, q, k, v = _reference_quantised_inputs(golden)
    kmean = rm.token_group_mean(k, T, False)
    # the reference fixture used torch's summation order for the mean; stay within what that allows
    q8, qs = rm.int8_fp8_quantize_qk(q, None, h, 32, False)
    k8, ks = rm.int8_fp8_quantize_qk(k, kmean, h, 64, True)
    vs = rm.int8_fp8_value_scale(v, h)
    v8 = rm.int8_fp8_quantize_value(v, vs, h)
    got = rm.dense_int8_fp8_attention(q8, k8, v8, qs, ks, vs, T, T)
    want = bf16(golden["att_int8_out"])
    assert rm.cosine(got, want) > 0.99999
    torch.testing.assert_close(got.float(), want.float(), rtol=0.02, atol=0.01)


def test_dense_nvfp4_attention_matches_reference(golden):
    T, h, q, k, v = _reference_quantised_inputs(golden)
    kmean = rm.token_group_mean(k, T, False).reshape(h, 128)
    q4, qsf = rm.nvfp4_prepare(q, None, h, False)
    k4, ksf = rm.nvfp4_prepare(k, kmean, h, False)
    v4, vsf = rm.nvfp4_prepare(v, None, h, True)
    got = rm.dense_nvfp4_attention(q4, k4, v4, qsf, ksf, vsf, T, T)
    want = bf16(golden["att_nvfp4_out"])
    assert rm.cosine(got, want) > 0.9999
    torch.testing.assert_close(got.float(), want.float(), rtol=0.03, atol=0.03)


def test_nvfp4_roundtrip_and_swizzle():
    g = torch.Generator().manual_seed(5)
    src = torch.randn(256, 2 * 128, generator=g).bfloat16()
    packed, sf = rm.nvfp4_prepare(src, None, 2, False)
    assert torch.equal(rm.swizzle_scales(rm.unswizzle_scales(sf)), sf)
    back = rm.nvfp4_dequantize(packed, sf)  # [heads, rows, 128]
    err = (back.permute(1, 0, 2).reshape(256, 256) - src.float()).abs().max()
    assert err < 1.1  # e2m1 step near amax is amax/6 * 2 / 2


def test_hadamard_is_orthonormal_and_involutive():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(7, 128, generator=g)
    y = rm.hadamard128(x)
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(rm.hadamard128(y), x, rtol=1e-5, atol=1e-5)
    # Sylvester matrix: first output is the scaled sum, second alternates signs
    torch.testing.assert_close(y[:, 0], x.sum(-1) * float(rm.INV_SQRT_128), rtol=1e-5, atol=1e-5)
    signs = torch.tensor([1.0, -1.0]).repeat(64)
    torch.testing.assert_close(y[:, 1], (x * signs).sum(-1) * float(rm.INV_SQRT_128), rtol=1e-5, atol=1e-5)
