"""Planning of the attention operators on CPU: kernel order, scratch layout, bindings.

The expected kernel orders are the attention parts of the reference operators (projections, norm-RoPE and
the output projection removed): ops/minimax_h3/attention.py:73-139, dense_nvfp4_attention.py:107-150,
sol_attention.py:133-158, sol_int8_fp8_attention.py:139-228, sol_nvfp4_attention.py:135-226.
"""

import pytest

from nano_omni_b200 import ops
from nano_omni_b200.core import DType, TensorDesc, TensorKind

T, h, H, OFF = 300, 2, 4, 1

EXPECTED = {
    ("dense", "bf16"): ["dense_bf16_attention_d128"],
    ("dense", "int8_fp8"): [
        "token_group_mean", "int8_fp8_quantize_qk", "int8_fp8_value_scale", "int8_fp8_quantize_value",
        "int8_fp8_quantize_qk", "dense_int8_fp8_d128",
    ],
    ("dense", "nvfp4"): ["token_group_mean", "nvfp4_prepare", "nvfp4_prepare", "nvfp4_prepare", "dense_nvfp4_attention_d128"],
    ("sol", "bf16"): ["sol_pool", "sol_stats", "sol_attention_d128"],
    ("sol", "int8_fp8"): [
        "token_group_mean", "int8_fp8_quantize_qk", "int8_fp8_value_scale", "int8_fp8_quantize_value",
        "int8_fp8_quantize_qk", "sol_int8_fp8_pool", "sol_stats", "sol_nvfp4_select", "sol_int8_fp8_attention_d128",
        "sol_nvfp4_finalize",
    ],
    ("sol", "nvfp4"): [
        "token_group_mean", "nvfp4_prepare", "nvfp4_prepare", "nvfp4_prepare", "sol_nvfp4_pool", "sol_stats",
        "sol_nvfp4_select", "sol_nvfp4_attention_d128", "sol_nvfp4_finalize",
    ],
}  # fmt: skip


def inputs():
    return tuple(TensorDesc.from_pointer(0x10000000 * (i + 1), DType.BF16, (T, h * 128)) for i in range(3))


def make(kind, precision):
    cls = ops.ATTENTION_OPS[(kind, precision)]
    if cls is ops.DenseInt8Fp8Attention:
        return cls(*inputs()).to(TensorDesc.from_pointer(0x90000000, DType.BF16, (T, h * 128)))
    extra = {"protected_tokens": 70} if kind == "sol" else {}
    op = cls(*inputs(), total_heads=H, head_offset=OFF, **extra)
    return op.to(TensorDesc.from_pointer(0x90000000, DType.BF16, (T, H, 128)))


def scratch_regions(calls):
    found = {}
    for call in calls:
        for tensor in call.arguments.values():
            if tensor is not None and tensor.kind == TensorKind.SCRATCH:
                found[(tensor.info[1], tensor.num_bytes)] = tensor
    return sorted(found, key=lambda r: (r[0], -r[1]))  # a parent region before the views into it


@pytest.mark.parametrize("kind,precision", list(EXPECTED))
def test_kernel_order_and_scratch(kind, precision):
    op = make(kind, precision)
    calls, num_bytes = op.prepare()
    assert [type(c).name for c in calls] == EXPECTED[(kind, precision)]
    regions = scratch_regions(calls)
    # views (a plane of the pooled tensor, the mean as [heads, 128]) share their parent's bytes: merge by start
    starts = {}
    for offset, size in regions:
        base = max((s for s in starts if s <= offset < s + starts[s]), default=None)
        if base is None:
            assert offset % 256 == 0, "temporaries start on 256-byte boundaries"
            starts[offset] = size
        else:
            assert offset + size <= base + starts[base], "a view stays inside its region"
    ordered = sorted(starts.items())
    for (a, size), (b, _) in zip(ordered, ordered[1:]):
        assert a + size <= b, "scratch regions overlap"
    assert all(offset + size <= num_bytes for offset, size in regions)
    # binding resolves every scratch descriptor against the base and leaves the rest alone
    base = 0x7F0000000000
    for call in op.bind(base):
        for tensor in call.arguments.values():
            if tensor is not None:
                assert tensor.kind == TensorKind.DEVICE
                assert tensor.data_ptr() >= 0x10000000


def test_sol_quantised_ops_finalize_in_place():
    """``exact`` is the output tensor itself (ops/minimax_h3/sol_int8_fp8_attention.py:116-118)."""
    for precision in ("int8_fp8", "nvfp4"):
        op = make("sol", precision)
        calls, _ = op.prepare()
        exact_stage, finalize = calls[-2], calls[-1]
        assert exact_stage.arguments.output == op.bound_outputs[0]
        assert finalize.arguments.exact == finalize.arguments.output == op.bound_outputs[0]
        assert exact_stage.arguments.state == finalize.arguments.state
        assert exact_stage.arguments.selected == finalize.arguments.selected == calls[-3].arguments.output
        assert exact_stage.arguments.num_protected_blocks == 2  # ceil(70 / 64)
        assert exact_stage.arguments.head_offset == finalize.arguments.head_offset == OFF


def test_key_value_persist_across_query_slices():
    key, value = inputs()[1:]
    krows = -(-T // 64) * 64
    outs = (
        TensorDesc.from_pointer(0x50000000, DType.I8, (h, krows, 128)),
        TensorDesc.from_pointer(0x51000000, DType.F32, (h, krows // 64)),
        TensorDesc.from_pointer(0x52000000, DType.FP8_E4M3, (h, 128, krows)),
        TensorDesc.from_pointer(0x53000000, DType.F32, (h, 128)),
    )
    prepare = ops.PrepareKeyValue(key, value).to(*outs)
    calls, _ = prepare.prepare()
    assert [type(c).name for c in calls] == [
        "token_group_mean", "int8_fp8_quantize_qk", "int8_fp8_value_scale", "int8_fp8_quantize_value",
    ]  # fmt: skip
    assert calls[1].arguments.quantized == outs[0] and calls[3].arguments.output == outs[2]
    chunk = TensorDesc.from_pointer(0x60000000, DType.BF16, (128, h * 128))
    attended = TensorDesc.from_pointer(0x61000000, DType.BF16, (128, h * 128))
    calls, _ = ops.QuerySlice(chunk, *outs, total_tokens=T).to(attended).prepare()
    assert [type(c).name for c in calls] == ["int8_fp8_quantize_qk", "dense_int8_fp8_d128"]
    assert calls[1].arguments.num_kv_tokens == T and calls[1].arguments.num_query_tokens == 128


def test_binding_errors():
    query, key, value = inputs()
    op = ops.DenseBf16Attention(query, key, value, total_heads=H, head_offset=OFF)
    with pytest.raises(AssertionError):
        op.prepare()  # outputs not bound
    with pytest.raises(AssertionError):
        op.to(TensorDesc.from_pointer(1 << 20, DType.BF16, (T, H + 1, 128)))
    with pytest.raises(AssertionError):
        op.to(TensorDesc.from_pointer(1 << 20, DType.F32, (T, H, 128)))
    op.to(TensorDesc.from_pointer(1 << 20, DType.BF16, (T, H, 128)))
    with pytest.raises(AssertionError):
        op.to(TensorDesc.from_pointer(1 << 20, DType.BF16, (T, H, 128)))  # bound once
    with pytest.raises(AssertionError):
        ops.DenseBf16Attention(query, key, value, total_heads=H, head_offset=H - 1)  # slice does not fit
    with pytest.raises(AssertionError):
        ops.SolAttention(query, key, value, total_heads=H, protected_tokens=T + 1)


def rotation():
    return ops.Rotation(
        TensorDesc.from_pointer(0x70000000, DType.BF16, (128,)),
        TensorDesc.from_pointer(0x70001000, DType.BF16, (128,)),
        TensorDesc.from_pointer(0x70002000, DType.F32, (T, 48)),
        TensorDesc.from_pointer(0x70102000, DType.F32, (T, 48)),
    )


def test_rotation_adds_norm_rope_before_attention():
    """Q and K straight from the projections (ops/minimax_h3/attention.py:51-97, sol_attention.py:105-131)."""
    rot = rotation()
    out3 = TensorDesc.from_pointer(0x90000000, DType.BF16, (T, H, 128))
    names = lambda op: [type(c).name for c in op.prepare()[0]]  # noqa: E731
    bf16 = ops.DenseBf16Attention(*inputs(), total_heads=H, head_offset=OFF, rotation=rot).to(out3)
    assert names(bf16) == ["h3_head_norm_rope", "h3_head_norm_rope", "dense_bf16_attention_d128"]
    calls, _ = bf16.prepare()
    assert calls[0].arguments.weight == rot.query_norm and calls[1].arguments.weight == rot.key_norm
    assert calls[2].arguments.query.info == calls[0].arguments.output.info  # attention reads the rotated temporaries
    assert calls[2].arguments.key.info == calls[1].arguments.output.info
    assert calls[2].arguments.value.info == inputs()[2].info

    int8 = ops.DenseInt8Fp8Attention(*inputs(), rotation=rot).to(TensorDesc.from_pointer(0x90000000, DType.BF16, (T, h * 128)))
    assert names(int8) == [
        "h3_head_norm_rope", "token_group_mean", "int8_fp8_quantize_qk", "int8_fp8_value_scale", "int8_fp8_quantize_value",
        "h3_query_prepare", "dense_int8_fp8_d128",
    ]  # fmt: skip
    sol8 = ops.SolInt8Fp8Attention(*inputs(), total_heads=H, head_offset=OFF, protected_tokens=70, rotation=rot).to(out3)
    assert names(sol8)[:2] == ["h3_head_norm_rope", "h3_head_norm_rope"] and names(sol8)[-1] == "sol_nvfp4_finalize"
    chunk = TensorDesc.from_pointer(0x60000000, DType.BF16, (128, h * 128))
    krows = -(-T // 64) * 64
    quantised = (
        TensorDesc.from_pointer(0x50000000, DType.I8, (h, krows, 128)),
        TensorDesc.from_pointer(0x51000000, DType.F32, (h, krows // 64)),
        TensorDesc.from_pointer(0x52000000, DType.FP8_E4M3, (h, 128, krows)),
        TensorDesc.from_pointer(0x53000000, DType.F32, (h, 128)),
    )
    planes = ops.Rotation(rot.query_norm, rot.key_norm,
                          TensorDesc.from_pointer(0x70002000, DType.F32, (128, 48)),
                          TensorDesc.from_pointer(0x70102000, DType.F32, (128, 48)))  # fmt: skip
    sliced = ops.QuerySlice(chunk, *quantised, total_tokens=T, rotation=planes)
    sliced.to(TensorDesc.from_pointer(0x61000000, DType.BF16, (128, h * 128)))
    assert names(sliced) == ["h3_query_prepare", "dense_int8_fp8_d128"]


def test_linear_shares_one_prepared_input_between_sibling_projections():
    """ops/matmul/sequence.py:29-122: the activations are quantised once per (dtype, rotation group) and a LoRA
    down-projection once per weight; each projection then adds its own up-projection and GEMM."""
    from nano_omni_b200.core import ScratchLayout

    tokens, width, rank = 300, 768, 32
    sequence = ops.KernelSequence(ScratchLayout())
    x = TensorDesc.from_pointer(0x10000000, DType.BF16, (tokens, width))
    prepared = sequence.prepare(x)
    down = TensorDesc.from_pointer(0x20000000, DType.BF16, (rank, width))
    for index, n in enumerate((512, 256)):
        weight = TensorDesc.from_pointer(0x30000000 + index * 0x1000000, DType.I8, (n, width))
        scale = TensorDesc.from_pointer(0x50000000 + index * 0x10000, DType.F32, (n, 1))
        up = TensorDesc.from_pointer(0x60000000 + index * 0x100000, DType.BF16, (n, rank))
        out = TensorDesc.from_pointer(0x70000000 + index * 0x1000000, DType.BF16, (tokens, n))
        sequence.linear(f"p{index}", prepared, weight, out, weight_scale=scale, loras=((down, up, 0.5),), rotation_group=256)
    assert [c.name for c in sequence.calls] == [
        "matmul_bf16", "matmul_bf16", "convrot_int8", "matmul_int8", "matmul_bf16", "matmul_int8",
    ]  # fmt: skip
    first_gemm, second_gemm = sequence.calls[3], sequence.calls[5]
    assert first_gemm.arguments.input == second_gemm.arguments.input  # the same quantised activations
    assert first_gemm.arguments.residual == sequence.calls[1].arguments.output  # LoRA update enters as the residual
    assert sequence.calls[4].arguments.input == sequence.calls[0].arguments.output  # the shared compression
    with pytest.raises(TypeError):
        sequence.linear("bad", prepared, weight, out, weight_scale=1.0)
    with pytest.raises(ValueError):
        ops.KernelSequence(ScratchLayout()).linear("other", prepared, weight, out, weight_scale=scale)
