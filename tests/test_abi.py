"""The shared library loads on a CPU-only host and exports every declared symbol."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "nano_omni_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nob200_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from nano_omni_b200 import _lib, build

    build.build()
    return _lib.library()


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "nob200_dense_bf16_attention_d128" in names
    assert "nob200_last_error" in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_abi_version_and_argument_rejection(lib):
    lib.nob200_abi_version.restype = ctypes.c_int
    assert lib.nob200_abi_version() == 1
    # argument validation happens before any CUDA call, so it can be exercised without a GPU
    fn = lib.nob200_dense_bf16_attention_d128
    fn.restype = ctypes.c_int
    null = ctypes.c_void_p(0)
    code = fn(0, 0, null, null, null, null, 1, 1, null)
    assert code == -1
    lib.nob200_last_error.restype = ctypes.c_char_p
    assert b"positive" in lib.nob200_last_error()
    code = fn(128, 3, ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), 2, 4, null)
    assert code == -1 and b"head_offset" in lib.nob200_last_error()
    fn = lib.nob200_int8_fp8_quantize_qk
    fn.restype = ctypes.c_int
    p = ctypes.c_void_p(16)
    assert fn(64, p, p, p, p, 1, 48, 0, 0, null) == -1
    assert b"tokens_per_block" in lib.nob200_last_error()


def test_kernel_registry_and_contract_round_trip():
    from nano_omni_b200 import kernels
    from nano_omni_b200.kernels.dense_bf16 import DenseBf16AttentionWorkload
    from nano_omni_b200.kernels.dense_int8_fp8 import DenseInt8Fp8AttentionWorkload
    from nano_omni_b200.kernels.dense_nvfp4 import DenseNvfp4Workload
    from nano_omni_b200.kernels.sol import (
        SolAttentionWorkload,
        SolNvfp4SelectWorkload,
        SolPoolWorkload,
        SolStatsWorkload,
    )
    from nano_omni_b200.kernels.quantize import (
        Int8Fp8QkWorkload,
        Int8Fp8ValueWorkload,
        Nvfp4PrepareWorkload,
        TokenGroupMeanWorkload,
    )

    registry = kernels.classes()
    workloads = {
        "dense_bf16_attention_d128": DenseBf16AttentionWorkload(num_tokens=300, heads=2, total_heads=5),
        "dense_int8_fp8_d128": DenseInt8Fp8AttentionWorkload(num_kv_tokens=300, heads=2, num_query_tokens=100),
        "dense_nvfp4_attention_d128": DenseNvfp4Workload(num_query_tokens=300, num_kv_tokens=300, heads=2, total_heads=3),
        "sol_pool": SolPoolWorkload(num_tokens=300, heads=2),
        "sol_int8_fp8_pool": SolPoolWorkload(num_tokens=300, heads=2, block=128),
        "sol_nvfp4_pool": SolPoolWorkload(num_tokens=300, heads=2),
        "sol_stats": SolStatsWorkload(num_blocks=5, heads=2),
        "sol_nvfp4_select": SolNvfp4SelectWorkload(num_tokens=300, heads=2, tau=0.5),
        "sol_attention_d128": SolAttentionWorkload(num_tokens=300, heads=2, total_heads=4, block=128, topk_fraction=0.25),
        "token_group_mean": TokenGroupMeanWorkload(num_tokens=300, columns=256, tokens_per_block=300),
        "int8_fp8_quantize_qk": Int8Fp8QkWorkload(num_tokens=300, heads=2, tokens_per_block=64, center=True),
        "int8_fp8_value_scale": Int8Fp8ValueWorkload(num_tokens=300, heads=2),
        "int8_fp8_quantize_value": Int8Fp8ValueWorkload(num_tokens=300, heads=2),
        "nvfp4_prepare": Nvfp4PrepareWorkload(num_tokens=300, heads=2, center=True, transpose=True),
    }
    for name, workload in workloads.items():
        cls = registry[name]
        # make_workload(make_arguments(w)) == w, the invariant the reference's verifier checks
        assert cls.make_workload(cls.make_arguments(workload)) == workload
        assert cls.symbol in declared_symbols()


def test_validation_errors_follow_the_reference_contract():
    import dataclasses

    from pydantic import ValidationError

    from nano_omni_b200.core import DType, TensorDesc
    from nano_omni_b200.kernels.dense_bf16 import (
        DenseBf16AttentionConfig,
        DenseBf16AttentionKernel,
        DenseBf16AttentionWorkload,
    )

    args = DenseBf16AttentionKernel.make_arguments(DenseBf16AttentionWorkload(num_tokens=64, heads=2, total_heads=4))
    with pytest.raises(AssertionError):
        DenseBf16AttentionKernel(dataclasses.replace(args, head_offset=3))
    with pytest.raises(AssertionError):
        DenseBf16AttentionKernel(dataclasses.replace(args, key=TensorDesc.empty(DType.BF16, (64, 2, 64))))
    with pytest.raises(ValidationError):
        DenseBf16AttentionConfig(tile_query_tokens=48)
    with pytest.raises(ValidationError):
        DenseBf16AttentionWorkload(num_tokens=0, heads=1, total_heads=1)
    kernel = DenseBf16AttentionKernel(args)
    assert kernel.tops(args) == {"BF16BF16F32": 4 * 2 * 64 * 64 * 128}


def test_argument_rejection_of_the_later_entry_points(lib):
    """Size and pointer checks of the sol stages, the block / global-scale variants and norm + RoPE (no GPU needed)."""
    lib.nob200_last_error.restype = ctypes.c_char_p
    null, p = ctypes.c_void_p(0), ctypes.c_void_p(256)

    fn = lib.nob200_sol_int8_fp8_attention_d128
    fn.restype = ctypes.c_int
    assert fn(300, 3, p, p, p, p, p, p, p, p, p, 2, 4, null) == -1 and b"head_offset" in lib.nob200_last_error()
    assert fn(300, 0, p, p, p, p, p, p, p, p, null, 2, 4, null) == -1 and b"NULL" in lib.nob200_last_error()

    # a query tile of the sol exact stages lists at most 4096 key blocks of 64 tokens
    assert fn(4096 * 64 + 1, 0, p, p, p, p, p, p, p, p, p, 2, 4, null) == -1 and b"at most 262144" in lib.nob200_last_error()
    fn = lib.nob200_sol_nvfp4_attention_d128
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 9 + [ctypes.c_int] * 2 + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    assert fn(128, 4096 * 64 + 1, 0, 256, 256, 256, 256, 256, 256, 256, 256, 256, 2, 4, None, 0, None) == -1
    assert b"exceed the 262144" in lib.nob200_last_error()
    assert fn(128, 300, 0, 256, 256, 256, 256, 256, 256, None, 256, 256, 2, 4, None, 0, None) == -1
    assert b"NULL mask" in lib.nob200_last_error()

    fn = lib.nob200_sol_nvfp4_finalize
    fn.restype = ctypes.c_int
    assert fn(300, 0, p, p, p, null, p, p, 2, 4, 64, null) == -1 and b"NULL" in lib.nob200_last_error()
    assert fn(300, 0, p, p, p, p, p, p, 2, 4, 96, null) == -1 and b"block" in lib.nob200_last_error()

    fn = lib.nob200_dense_int8_fp8_d128_blocks
    fn.restype = ctypes.c_int
    assert fn(300, 300, p, p, p, p, p, p, p, 2, 48, 64, null) == -1 and b"query scale block" in lib.nob200_last_error()
    assert fn(300, 300, p, p, p, p, p, p, p, 2, 32, 32, null) == -1 and b"key scale block" in lib.nob200_last_error()

    fn = lib.nob200_dense_nvfp4_attention_d128_global
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 6 + [ctypes.c_float] * 3 + [ctypes.c_void_p] + [ctypes.c_int] * 2 + [
        ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]  # fmt: skip
    assert fn(300, 300, 0, 256, 256, 256, 256, 256, 256, 0.0, 1.0, 1.0, 256, 2, 2, 256, 1 << 30, None) == -1
    assert b"global scales" in lib.nob200_last_error()

    fn = lib.nob200_h3_head_norm_rope
    fn.restype = ctypes.c_int
    assert fn(300, p, p, p, null, p, 2, null) == -1 and b"come together" in lib.nob200_last_error()
    fn = lib.nob200_h3_query_prepare
    fn.restype = ctypes.c_int
    assert fn(0, p, p, null, null, p, p, 2, null) == -1 and b"positive" in lib.nob200_last_error()

    fn = lib.nob200_mma_issue_rate
    fn.restype = ctypes.c_int
    assert fn(7, 1024, 1, p, null) == -1 and b"kind" in lib.nob200_last_error()
    assert fn(0, 1023, 1, p, null) == -1 and b"multiple of 4" in lib.nob200_last_error()
