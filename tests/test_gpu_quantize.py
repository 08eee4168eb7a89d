"""Bit-exact parity of the quantiser kernels with the CPU oracle (through the C ABI)."""

import numpy as np
import pytest
import torch

from oracle import reference_math as rm
from tests.conftest import bf16
from tests.gpu_util import desc, randn_bf16, run

pytestmark = pytest.mark.gpu

SIZES = [1, 63, 64, 65, 130, 500, 4096]


def _mean(src, tpb, pad):
    from nano_omni_b200.core import DType
    from nano_omni_b200.kernels.quantize import TokenGroupMeanArguments, TokenGroupMeanKernel, TokenGroupMeanWorkload

    T, C = src.shape
    nb = -(-T // tpb)
    out = torch.full((nb, C), float("nan"), device="cuda")
    need = TokenGroupMeanKernel.workspace_bytes(
        TokenGroupMeanWorkload(num_tokens=T, columns=C, tokens_per_block=tpb, include_padding=pad)
    )
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    run(TokenGroupMeanKernel(TokenGroupMeanArguments(desc(src), desc(out), tpb, pad, desc(ws, DType.U8) if need else None)))
    return out


@pytest.mark.parametrize("T", SIZES)
def test_token_group_mean_bit_exact(T):
    h = 2
    src = randn_bf16(T, T, h * 128, outlier=True)
    for tpb, pad in ((T, False), (64, False), (64, True), (300, False)):
        got = _mean(src, tpb, pad).cpu()
        want = rm.token_group_mean(src.cpu(), tpb, pad)
        assert torch.equal(got, want), f"T={T} tpb={tpb} pad={pad}"


def test_token_group_mean_long_group_and_ragged_columns():
    """More chunk sums per group than the finishing kernel stages at once (256), and a column count that is no
    multiple of the 32 columns a finishing CTA owns."""
    T, C = 40000, 132
    src = randn_bf16(T, T, C, outlier=True)
    for tpb, pad in ((T, False), (33000, True)):
        got = _mean(src, tpb, pad).cpu()
        want = rm.token_group_mean(src.cpu(), tpb, pad)
        assert torch.equal(got, want), f"tpb={tpb} pad={pad}"


@pytest.mark.parametrize("T", SIZES)
@pytest.mark.parametrize("tpb,center,hadamard", [(32, False, False), (64, True, False), (128, True, False), (32, False, True), (128, True, True)])
def test_int8_qk_bit_exact(T, tpb, center, hadamard):
    from nano_omni_b200.kernels.quantize import Int8Fp8QuantizeQKArguments, Int8Fp8QuantizeQKKernel

    h = 3
    src = randn_bf16(100 + T, T, h * 128, outlier=True)
    mean = rm.token_group_mean(src.cpu(), T, False)
    padded = -(-T // tpb) * tpb
    q = torch.full((h, padded, 128), 77, dtype=torch.int8, device="cuda")
    s = torch.full((h, padded // tpb), float("nan"), device="cuda")
    run(
        Int8Fp8QuantizeQKKernel(
            Int8Fp8QuantizeQKArguments(desc(src), desc(mean.cuda()), desc(q), desc(s), h, tpb, center, hadamard)
        )
    )
    want_q, want_s = rm.int8_fp8_quantize_qk(src.cpu(), mean, h, tpb, center, hadamard)
    assert torch.equal(s.cpu(), want_s)
    assert torch.equal(q.cpu(), want_q)


@pytest.mark.parametrize("T", SIZES)
def test_value_scale_and_fp8_bit_exact(T):
    from nano_omni_b200.kernels.quantize import (
        Int8Fp8QuantizeValueArguments,
        Int8Fp8QuantizeValueKernel,
        Int8Fp8ValueScaleArguments,
        Int8Fp8ValueScaleKernel,
    )

    h = 3
    src = randn_bf16(200 + T, T, h * 128, outlier=True)
    vs = torch.full((h, 128), float("nan"), device="cuda")
    run(Int8Fp8ValueScaleKernel(Int8Fp8ValueScaleArguments(desc(src), desc(vs), h)))
    want_vs = rm.int8_fp8_value_scale(src.cpu(), h)
    assert torch.equal(vs.cpu(), want_vs)
    padded = -(-T // 64) * 64
    v8 = torch.full((h, 128, padded), 0x55, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    run(Int8Fp8QuantizeValueKernel(Int8Fp8QuantizeValueArguments(desc(src), desc(vs), desc(v8), h)))
    want = rm.int8_fp8_quantize_value(src.cpu(), want_vs, h)
    assert torch.equal(v8.cpu().view(torch.uint8), want.view(torch.uint8))


@pytest.mark.parametrize("T", SIZES)
@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("center,hadamard,gscale", [(False, False, 0.0), (True, False, 0.0), (True, True, 0.0), (False, False, 0.75)])
def test_nvfp4_prepare_bit_exact(T, transpose, center, hadamard, gscale):
    from nano_omni_b200.core import DType
    from nano_omni_b200.kernels.quantize import Nvfp4PrepareArguments, Nvfp4PrepareKernel

    h = 2
    src = randn_bf16(300 + T, T, h * 128, outlier=True)
    mean = rm.token_group_mean(src.cpu(), T, False).reshape(h, 128) if center else None
    padded = -(-T // 128) * 128
    rows, cols = (128, padded) if transpose else (padded, 128)
    packed = torch.full((h, rows, cols // 2), 0xAA, dtype=torch.uint8, device="cuda")
    sf = torch.full((h, rows, cols // 16), 0xAA, dtype=torch.uint8, device="cuda")
    run(
        Nvfp4PrepareKernel(
            Nvfp4PrepareArguments(
                desc(src),
                desc(mean.cuda()) if center else None,
                desc(packed),
                desc(sf, DType.FP8_UE4M3),
                h,
                transpose,
                hadamard,
                gscale,
            )
        )
    )
    want_p, want_s = rm.nvfp4_prepare(src.cpu(), mean, h, transpose, hadamard, gscale)
    assert torch.equal(sf.cpu(), want_s)
    assert torch.equal(packed.cpu(), want_p)


def test_quantisers_match_reference_golden(golden):
    """Same kernels against the fixtures produced by the reference's own ref_programs."""
    from nano_omni_b200.core import DType
    from nano_omni_b200.kernels.quantize import (
        Int8Fp8QuantizeQKArguments,
        Int8Fp8QuantizeQKKernel,
        Int8Fp8QuantizeValueArguments,
        Int8Fp8QuantizeValueKernel,
        Int8Fp8ValueScaleArguments,
        Int8Fp8ValueScaleKernel,
        Nvfp4PrepareArguments,
        Nvfp4PrepareKernel,
    )

    for T, h in ((130, 2), (500, 3)):
        tag = f"T{T}_h{h}"
        src = bf16(golden[f"src_{tag}"]).cuda()
        mean = torch.from_numpy(golden[f"mean_{tag}_tpb{T}_pad0"]).cuda()
        for tpb, center in ((32, False), (64, True), (128, True)):
            padded = -(-T // tpb) * tpb
            q = torch.empty((h, padded, 128), dtype=torch.int8, device="cuda")
            s = torch.empty((h, padded // tpb), device="cuda")
            run(Int8Fp8QuantizeQKKernel(Int8Fp8QuantizeQKArguments(desc(src), desc(mean), desc(q), desc(s), h, tpb, center)))
            assert np.array_equal(q.cpu().numpy(), golden[f"qk_q_{tag}_tpb{tpb}_c{int(center)}"])
            assert np.array_equal(s.cpu().numpy(), golden[f"qk_s_{tag}_tpb{tpb}_c{int(center)}"])
        vs = torch.empty((h, 128), device="cuda")
        run(Int8Fp8ValueScaleKernel(Int8Fp8ValueScaleArguments(desc(src), desc(vs), h)))
        assert np.array_equal(vs.cpu().numpy(), golden[f"vscale_{tag}"])
        v8 = torch.empty((h, 128, -(-T // 64) * 64), dtype=torch.uint8, device="cuda")
        run(Int8Fp8QuantizeValueKernel(Int8Fp8QuantizeValueArguments(desc(src), desc(vs), desc(v8, DType.FP8_E4M3), h)))
        assert np.array_equal(v8.cpu().numpy(), golden[f"v8_{tag}"])
        padded = -(-T // 128) * 128
        mean_h = mean.reshape(h, 128).contiguous()
        for transpose in (False, True):
            for center in (False, True):
                rows, cols = (128, padded) if transpose else (padded, 128)
                packed = torch.empty((h, rows, cols // 2), dtype=torch.uint8, device="cuda")
                sf = torch.empty((h, rows, cols // 16), dtype=torch.uint8, device="cuda")
                run(
                    Nvfp4PrepareKernel(
                        Nvfp4PrepareArguments(
                            desc(src), desc(mean_h) if center else None, desc(packed), desc(sf, DType.FP8_UE4M3), h, transpose
                        )
                    )
                )
                key = f"{tag}_t{int(transpose)}_c{int(center)}"
                assert np.array_equal(packed.cpu().numpy(), golden[f"fp4_q_{key}"])
                assert np.array_equal(sf.cpu().numpy(), golden[f"fp4_s_{key}"])
