"""Dense int8-fp8 attention on the GPU against the reference's dequantise-and-attend oracle.

Operands are produced by this library's quantiser kernels (bit-exact with the reference
quantisers, see test_gpu_quantize.py).  Bars:
* cosine >= 0.999 against the oracle of src/nano_omni/kernels/attention/int8_fp8/dense.py:394-437
  on N(0,1) inputs, plus max-abs <= 0.06: P is rounded to e4m3 (relative step 2^-4) exactly as the
  reference kernel does (dense.py:196-221), which the oracle does not model, so with few keys and
  |V| ~ 1 single outputs move by up to a few hundredths;
* the reference checker's own tolerance rtol 0.02 / atol 0.01 (src/nano_omni/core/kernel.py:128-129)
  on the reference checker's own input recipe, floats = randn * 0.1 (scripts/tune.py:123).
"""

import pytest
import torch

from oracle import reference_math as rm
from tests.conftest import bf16
from tests.gpu_util import desc, randn_bf16, run

pytestmark = pytest.mark.gpu

COSINE = 0.999
MAX_ABS = 0.06


def quantise(q, k, v, h):
    """bf16 [T, h*128] -> the seven tensors the attention kernel consumes (via the GPU quantisers)."""
    from nano_omni_b200.core import DType
    from nano_omni_b200.kernels.quantize import (
        Int8Fp8QuantizeQKArguments,
        Int8Fp8QuantizeQKKernel,
        Int8Fp8QuantizeValueArguments,
        Int8Fp8QuantizeValueKernel,
        Int8Fp8ValueScaleArguments,
        Int8Fp8ValueScaleKernel,
    )

    Tq, Tk = q.shape[0], k.shape[0]
    kmean = rm.token_group_mean(k.cpu(), Tk, False).cuda()
    q8 = torch.empty(h, -(-Tq // 32) * 32, 128, dtype=torch.int8, device="cuda")
    qs = torch.empty(h, -(-Tq // 32), device="cuda")
    k8 = torch.empty(h, -(-Tk // 64) * 64, 128, dtype=torch.int8, device="cuda")
    ks = torch.empty(h, -(-Tk // 64), device="cuda")
    vs = torch.empty(h, 128, device="cuda")
    v8 = torch.empty(h, 128, -(-Tk // 64) * 64, dtype=torch.uint8, device="cuda")
    run(Int8Fp8QuantizeQKKernel(Int8Fp8QuantizeQKArguments(desc(q), desc(kmean), desc(q8), desc(qs), h, 32, False)))
    run(Int8Fp8QuantizeQKKernel(Int8Fp8QuantizeQKArguments(desc(k), desc(kmean), desc(k8), desc(ks), h, 64, True)))
    run(Int8Fp8ValueScaleKernel(Int8Fp8ValueScaleArguments(desc(v), desc(vs), h)))
    run(Int8Fp8QuantizeValueKernel(Int8Fp8QuantizeValueArguments(desc(v), desc(vs), desc(v8, DType.FP8_E4M3), h)))
    return q8, k8, v8.view(torch.float8_e4m3fn), qs, ks, vs


def attend(ops, Tq, Tk, h):
    from nano_omni_b200.kernels.dense_int8_fp8 import DenseInt8Fp8AttentionArguments, DenseInt8Fp8AttentionKernel

    q8, k8, v8, qs, ks, vs = ops
    out = torch.full((Tq, h * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    run(
        DenseInt8Fp8AttentionKernel(
            DenseInt8Fp8AttentionArguments(desc(q8), desc(k8), desc(v8), desc(qs), desc(ks), desc(vs), desc(out), Tk, h, Tq)
        )
    )
    return out


def oracle(ops, Tq, Tk):
    q8, k8, v8, qs, ks, vs = (t.cpu() for t in ops)
    return rm.dense_int8_fp8_attention(q8, k8, v8, qs, ks, vs, Tq, Tk)


@pytest.mark.parametrize("T", [1, 63, 64, 65, 130, 257, 500, 1000])
def test_small_and_ragged_sizes(T):
    h = 2
    q, k, v = (randn_bf16(20 * T + i, T, h * 128) for i in range(3))
    ops = quantise(q, k, v, h)
    got = attend(ops, T, T, h).cpu().float()
    want = oracle(ops, T, T).float()
    assert torch.isfinite(got).all()
    assert rm.cosine(got, want) >= COSINE
    assert (got - want).abs().max() <= MAX_ABS


def test_query_slice_against_longer_keys():
    """Tq != Tk: the reference's production shape for dense int8 (query slices, persistent K/V)."""
    h, Tq, Tk = 3, 300, 1111
    q = randn_bf16(1, Tq, h * 128)
    k, v = randn_bf16(2, Tk, h * 128, outlier=True), randn_bf16(3, Tk, h * 128)
    ops = quantise(q, k, v, h)
    got = attend(ops, Tq, Tk, h).cpu().float()
    want = oracle(ops, Tq, Tk).float()
    assert rm.cosine(got, want) >= COSINE
    # the x16 key channel makes the softmax sharp: a row is a few keys' values, each weighted by an
    # e4m3-rounded probability (relative step 2^-4), so the bound scales with |V|
    assert (got - want).abs().max() <= 2.0**-4 * v.float().abs().max().item()


def test_config2_seq4096_heads4():
    """Benchmark configuration 2: the seed-0 tensors of the small bf16 config through the int8-fp8 path."""
    torch.manual_seed(0)
    T, h = 4096, 4
    q, k, v = (torch.randn(T, h, 128).bfloat16().reshape(T, h * 128).cuda() for _ in range(3))
    ops = quantise(q, k, v, h)
    got = attend(ops, T, T, h).cpu().float()
    want = oracle(ops, T, T).float()
    assert rm.cosine(got, want) >= COSINE
    # and the quantised path stays close to fp32 attention on the unquantised tensors
    fp32 = rm.dense_attention_fp32(*(t.cpu().reshape(T, h, 128) for t in (q, k, v))).reshape(T, h * 128)
    assert rm.cosine(got, fp32) >= 0.99


def test_reference_golden_operands(golden):
    """Operands quantised by the reference itself (fixtures) -> output compared with its ref_program output."""
    from tests.conftest import e4m3  # noqa: F401

    T, h = 200, 2
    q, k, v = (bf16(golden[f"att_{n}"]).reshape(T, h * 128).cuda() for n in "qkv")
    ops = quantise(q, k, v, h)
    got = attend(ops, T, T, h).cpu().float()
    want = bf16(golden["att_int8_out"]).float()
    assert rm.cosine(got, want) >= COSINE
    assert (got - want).abs().max() <= MAX_ABS


@pytest.mark.parametrize("T", [130, 1000])
def test_reference_checker_recipe_and_tolerance(T):
    """Inputs as the reference's checker draws them (randn * 0.1) and its rtol/atol."""
    h = 2
    g = torch.Generator().manual_seed(0)
    q, k, v = ((torch.randn(T, h * 128, generator=g) * 0.1).bfloat16().cuda() for _ in range(3))
    ops = quantise(q, k, v, h)
    got = attend(ops, T, T, h).cpu().float()
    want = oracle(ops, T, T).float()
    torch.testing.assert_close(got, want, rtol=0.02, atol=0.01)
    assert rm.cosine(got, want) >= COSINE


def test_large_scales_keep_equal_logits_equal():
    """Scales near 1 (the reference's known-answer regime, tests/test_sol_attention_state.py:231-270).

    Every key has the same logit (K = c_b with scale 1/c_b per 64-key block), so the output is the plain mean of V
    over the keys.  A conversion of the int32 scores that loses low bits of the per-block factor would weight the
    blocks unequally.
    """
    T, h = 256, 1
    c = torch.tensor([1, 2, 4, 8], dtype=torch.int8)
    q8 = torch.ones(h, T, 128, dtype=torch.int8, device="cuda")
    k8 = c.repeat_interleave(64)[None, :, None].expand(h, T, 128).contiguous().cuda()
    qs = torch.full((h, T // 32), 0.9, device="cuda")
    ks = (1.0 / c.float())[None].cuda() * 1.1
    v8 = (torch.arange(4).float() + 1).repeat_interleave(64)[None, None, :].expand(h, 128, T).contiguous()
    v8 = v8.to(torch.float8_e4m3fn).cuda()
    vs = torch.ones(h, 128, device="cuda")
    out = attend((q8, k8, v8, qs, ks, vs), T, T, h)
    torch.testing.assert_close(out.float().cpu(), torch.full((T, 128), 2.5), rtol=2e-3, atol=0)


def test_rotated_operands_with_128_token_scales():
    """Benchmark configuration 2 as stated: Q and K through the Walsh-Hadamard rotation, int8 with one scale per
    128-token block; V e4m3 per channel; P e4m3.  The rotation cancels in q.k, so the result is compared with fp32
    attention on the unrotated tensors, and with the oracle on the quantised operands."""
    from nano_omni_b200.core import DType
    from nano_omni_b200.kernels.dense_int8_fp8 import DenseInt8Fp8AttentionArguments, DenseInt8Fp8AttentionKernel
    from nano_omni_b200.kernels.quantize import (
        Int8Fp8QuantizeQKArguments,
        Int8Fp8QuantizeQKKernel,
        Int8Fp8QuantizeValueArguments,
        Int8Fp8QuantizeValueKernel,
        Int8Fp8ValueScaleArguments,
        Int8Fp8ValueScaleKernel,
    )

    T, h = 4000, 4  # not a multiple of 128: ragged last blocks
    g = torch.Generator().manual_seed(1)
    q = torch.randn(T, h, 128, generator=g).bfloat16()
    k = torch.randn(T, h, 128, generator=g)
    k[:, torch.arange(h), torch.randint(0, 128, (h,), generator=g)] *= 16  # one outlier channel per head
    k = k.bfloat16()
    v = torch.randn(T, h, 128, generator=g).bfloat16()
    flat = lambda t: t.reshape(T, h * 128).cuda()  # noqa: E731
    rows = -(-T // 128) * 128
    unused = torch.zeros(1, h * 128, device="cuda")
    q8 = torch.empty(h, rows, 128, dtype=torch.int8, device="cuda")
    k8 = torch.empty_like(q8)
    qs = torch.empty(h, rows // 128, device="cuda")
    ks = torch.empty_like(qs)
    vs = torch.empty(h, 128, device="cuda")
    v8 = torch.empty(h, 128, -(-T // 64) * 64, dtype=torch.uint8, device="cuda")
    run(Int8Fp8QuantizeQKKernel(Int8Fp8QuantizeQKArguments(desc(flat(q)), desc(unused), desc(q8), desc(qs), h, 128, False, True)))
    run(Int8Fp8QuantizeQKKernel(Int8Fp8QuantizeQKArguments(desc(flat(k)), desc(unused), desc(k8), desc(ks), h, 128, False, True)))
    run(Int8Fp8ValueScaleKernel(Int8Fp8ValueScaleArguments(desc(flat(v)), desc(vs), h)))
    run(Int8Fp8QuantizeValueKernel(Int8Fp8QuantizeValueArguments(desc(flat(v)), desc(vs), desc(v8, DType.FP8_E4M3), h)))
    out = torch.full((T, h * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    run(
        DenseInt8Fp8AttentionKernel(
            DenseInt8Fp8AttentionArguments(
                desc(q8), desc(k8), desc(v8, DType.FP8_E4M3), desc(qs), desc(ks), desc(vs), desc(out), T, h, T, 128, 128
            )
        )
    )
    got = out.cpu().float().reshape(T, h, 128)
    assert torch.isfinite(got).all()
    # oracle: dequantise with the 128-token scales (still in the rotated basis for Q and K) and attend in fp32
    dq = (q8.cpu().float().reshape(h, -1, 128, 128) * qs.cpu()[:, :, None, None]).reshape(h, -1, 128)[:, :T]
    dk = (k8.cpu().float().reshape(h, -1, 128, 128) * ks.cpu()[:, :, None, None]).reshape(h, -1, 128)[:, :T]
    order = rm.unpermute_value_tokens(v8.shape[2])[:T]
    dv = v8.view(torch.float8_e4m3fn).cpu().float()[:, :, order].transpose(1, 2) * vs.cpu()[:, None, :]
    want = torch.nn.functional.scaled_dot_product_attention(dq, dk, dv).transpose(0, 1)
    assert rm.cosine(got, want) >= COSINE
    fp32 = rm.dense_attention_fp32(q, k, v)
    assert rm.cosine(got, fp32) >= 0.998


@pytest.mark.parametrize("Tq,Tk,splits", [(300, 1111, 2), (300, 1111, 3), (129, 2048 + 37, 4), (1000, 1000, 2)])
def test_key_splits_agree_with_one_share(Tq, Tk, splits):
    """Key tiles divided over several CTAs and merged by their log-sum-exp: the same attention as one share, up to the
    bf16 rounding of the partial results (each share is normalised and stored as bf16 before the merge)."""
    from nano_omni_b200.core import DType, TensorDesc
    from nano_omni_b200.kernels.dense_bf16 import splitkv_workspace_bytes
    from nano_omni_b200.kernels.dense_int8_fp8 import (
        DenseInt8Fp8AttentionArguments,
        DenseInt8Fp8AttentionConfig,
        DenseInt8Fp8AttentionKernel,
    )

    h = 3
    q = randn_bf16(11, Tq, h * 128)
    k, v = randn_bf16(12, Tk, h * 128, outlier=True), randn_bf16(13, Tk, h * 128)
    ops = quantise(q, k, v, h)
    one = attend(ops, Tq, Tk, h).cpu().float()
    q8, k8, v8, qs, ks, vs = ops
    out = torch.full((Tq, h * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(splitkv_workspace_bytes(Tq, h, splits), dtype=torch.uint8, device="cuda")
    run(
        DenseInt8Fp8AttentionKernel(
            DenseInt8Fp8AttentionArguments(
                desc(q8), desc(k8), desc(v8), desc(qs), desc(ks), desc(vs), desc(out), Tk, h, Tq,
                workspace=TensorDesc.from_torch(scratch, DType.U8),
            ),
            DenseInt8Fp8AttentionConfig(kv_splits=splits),
        )
    )  # fmt: skip
    got = out.cpu().float()
    assert torch.isfinite(got).all()
    want = oracle(ops, Tq, Tk).float()
    assert rm.cosine(got, want) >= COSINE
    assert (got - one).abs().max() <= 2.0**-6 * v.float().abs().max().item()


def test_query_slice_operator_divides_the_keys():
    """QuerySlice picks key splits for a slice that would leave the last wave of SMs short, and the result stays that
    of the unsplit kernel (attention_slices.py:113-161 is the reference operator)."""
    from nano_omni_b200 import ops as nob_ops
    from nano_omni_b200.kernels.dense_bf16 import choose_kv_splits

    h, Tq, Tk = 37, 512, 4096
    assert choose_kv_splits(4096, 56, num_kv_tokens=60778) == 2  # 896 CTAs: 6.05 waves of 148
    splits = choose_kv_splits(Tq, h, num_kv_tokens=Tk)
    assert splits == 2  # 74 CTAs on 148 SMs
    q = randn_bf16(21, Tq, h * 128)
    k, v = randn_bf16(22, Tk, h * 128), randn_bf16(23, Tk, h * 128)
    prepared = quantise(q, k, v, h)
    _, k8, v8, _, ks, vs = prepared
    out = torch.full((Tq, h * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    op = nob_ops.QuerySlice(desc(q), desc(k8), desc(ks), desc(v8), desc(vs), total_tokens=Tk).to(desc(out))
    calls, need = op.prepare()
    assert calls[-1].config.kv_splits == splits
    scratch = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    aligned = scratch[(-scratch.data_ptr()) % 256 :]
    op.run(aligned)
    torch.cuda.synchronize()
    want = attend(prepared, Tq, Tk, h).cpu().float()
    assert (out.cpu().float() - want).abs().max() <= 2.0**-6 * v.float().abs().max().item()
