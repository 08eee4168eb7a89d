"""The boundary against the reference itself, where its checkout can be imported (the build container):
every kernel class of this library against the reference class of the same ``name`` (Arguments fields a prefix in
order, Workload fields a superset), and the adapter that lets a reference ``Kernel`` instance launch this library.
Skipped where nano-omni is not importable (the GPU box)."""

import ctypes
import dataclasses
import os
import sys

import pytest

REFERENCE_SRC = os.environ.get("NANO_OMNI_SRC", "/root/reference/src")


@pytest.fixture(scope="module")
def reference_classes():
    if not os.path.isdir(os.path.join(REFERENCE_SRC, "nano_omni")):
        pytest.skip("nano-omni checkout not available")
    sys.path.insert(0, REFERENCE_SRC)
    try:
        from nano_omni import kernels as reference_kernels

        found = reference_kernels.classes()
    except Exception as error:  # an optional dependency of the reference is missing
        pytest.skip(f"nano-omni does not import here: {error}")
    finally:
        sys.path.remove(REFERENCE_SRC)
    return found if isinstance(found, dict) else {cls.name: cls for cls in found}


def test_every_shared_name_agrees_field_for_field(reference_classes):
    from nano_omni_b200 import adapter, kernels

    ours = kernels.classes()
    shared = sorted(set(ours) & set(reference_classes))
    # the attention path of the reference: its dense and sol kernels, the quantisers, pools, router and finalize
    for name in (
        "dense_bf16_attention_d128", "dense_int8_fp8_d128", "dense_nvfp4_attention_d128", "int8_fp8_quantize_qk",
        "int8_fp8_value_scale", "int8_fp8_quantize_value", "nvfp4_prepare", "token_group_mean", "sol_pool", "sol_stats",
        "sol_nvfp4_select", "sol_attention_d128", "sol_int8_fp8_attention_d128", "sol_nvfp4_attention_d128",
        "sol_nvfp4_finalize",
    ):  # fmt: skip
        assert name in shared, f"{name} is missing on one side"
    problems = [p for name in shared for p in adapter.field_differences(ours[name], reference_classes[name])]
    assert not problems, "\n".join(problems)
    # names this library adds (no reference class) must not shadow a reference name by accident
    for name in set(ours) - set(reference_classes):
        assert ours[name].name == name


def test_adapter_routes_a_reference_kernel_to_the_c_abi(reference_classes, monkeypatch):
    """Patch the reference's DenseBf16AttentionKernel, then drive it the way its runtime does: compile() binds the
    symbol, submit() in a prepare pass launches nothing, submit() afterwards calls the C function with the reference
    ABI's values (token count, head offset, four addresses, head counts, stream)."""
    sys.path.insert(0, REFERENCE_SRC)
    try:
        from nano_omni.core.tensor import DType as RefDType, TensorDesc as RefTensorDesc, TensorKind as RefKind
    finally:
        sys.path.remove(REFERENCE_SRC)
    from nano_omni_b200 import _lib, adapter

    calls = []

    def fake_symbol(name):
        def function(*args):
            calls.append((name, [getattr(a, "value", a) for a in args]))
            return 0

        return function

    monkeypatch.setattr(_lib, "symbol", fake_symbol)
    monkeypatch.setattr(_lib, "current_stream", lambda: 0)
    state = {"compiling": "prepare"}
    reference = reference_classes["dense_bf16_attention_d128"]
    saved = reference.compile, reference.submit
    try:
        patched = adapter.install(
            reference_classes=lambda: {"dense_bf16_attention_d128": reference},
            stream=lambda: 0xABC0,
            compiling=lambda: state["compiling"],
        )
        assert list(patched) == ["dense_bf16_attention_d128"]
        T, h, H = 300, 2, 5

        def at(base, heads):
            return RefTensorDesc(RefDType.BF16, (T, heads, 128), RefKind.DEVICE, (base, 0))

        arguments_type = adapter._generic_argument(reference, 0)
        names = [f.name for f in dataclasses.fields(arguments_type)]
        assert names[:5] == ["query", "key", "value", "output", "head_offset"]
        arguments = arguments_type(at(0x1000, h), at(0x2000, h), at(0x3000, h), at(0x4000, H), 2)
        kernel = reference(arguments)
        kernel.compile()
        assert kernel.compiled is not None
        kernel.submit()  # prepare pass
        assert calls == []
        state["compiling"] = None
        kernel.submit()
        assert len(calls) == 1
        name, values = calls[0]
        assert name.startswith("nob200_dense_bf16_attention_d128")
        assert values[:6] == [T, 2, 0x1000, 0x2000, 0x3000, 0x4000]
        assert values[6:8] == [h, H] and values[-1] == 0xABC0
    finally:
        reference.compile, reference.submit = saved
