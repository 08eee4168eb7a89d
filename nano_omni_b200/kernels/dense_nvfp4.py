"""Dense attention on NVFP4 operands, bound to ``nob200_dense_nvfp4_attention_d128``.

Interface of reference ``DenseNvfp4Kernel`` (src/nano_omni/kernels/attention/dense_nvfp4.py:18-52,
562-676): same Arguments fields and order, validation and ``tops``.  The trailing ``workspace``
(no counterpart in the reference) holds the operands expanded to bf16; the op reserves
``workspace_bytes(workload)`` of scratch for it.
"""

from __future__ import annotations

import ctypes
import dataclasses

from pydantic import Field

from nano_omni_b200 import _lib
from nano_omni_b200.core import Arguments, Config, DType, Kernel, MmaType, TensorDesc, Workload


class DenseNvfp4Workload(Workload):
    num_query_tokens: int = Field(gt=0)
    num_kv_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    total_heads: int = Field(gt=0)


class DenseNvfp4Config(Config):
    tile_query_tokens: int = 128
    tile_kv_tokens: int = 128
    threads: int = 384


@dataclasses.dataclass(frozen=True, slots=True)
class DenseNvfp4Arguments(Arguments):
    query: TensorDesc
    key: TensorDesc
    value: TensorDesc
    query_scales: TensorDesc
    key_scales: TensorDesc
    value_scales: TensorDesc
    output: TensorDesc
    num_query_tokens: int
    num_kv_tokens: int
    head_offset: int
    workspace: TensorDesc | None = None
    # global scale of each operand (``nvfp4_prepare`` with ``global_scale`` > 0); 1.0 = the reference's layout
    global_scales: tuple[float, float, float] = (1.0, 1.0, 1.0)

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (
            ("num_query_tokens", self.num_query_tokens),
            ("num_kv_tokens", self.num_kv_tokens),
            ("head_offset", self.head_offset),
        )


def _align(n: int) -> int:
    return (n + 255) // 256 * 256


class DenseNvfp4Kernel(Kernel[DenseNvfp4Arguments, DenseNvfp4Workload, DenseNvfp4Config]):
    name = "dense_nvfp4_attention_d128"
    symbol = "nob200_dense_nvfp4_attention_d128_global"
    reference_rtol = 0.03
    reference_atol = 0.03

    @classmethod
    def workspace_bytes(cls, workload: DenseNvfp4Workload) -> int:
        return _align(workload.num_query_tokens * workload.heads * 256) + 2 * _align(
            workload.num_kv_tokens * workload.heads * 256
        )

    @classmethod
    def make_arguments(cls, workload: DenseNvfp4Workload) -> DenseNvfp4Arguments:
        query_rows = -(-workload.num_query_tokens // 128) * 128
        key_rows = -(-workload.num_kv_tokens // 128) * 128
        return DenseNvfp4Arguments(
            TensorDesc.empty(DType.U8, (workload.heads, query_rows, 64)),
            TensorDesc.empty(DType.U8, (workload.heads, key_rows, 64)),
            TensorDesc.empty(DType.U8, (workload.heads, 128, key_rows // 2)),
            TensorDesc.empty(DType.FP8_UE4M3, (workload.heads, query_rows, 8)),
            TensorDesc.empty(DType.FP8_UE4M3, (workload.heads, key_rows, 8)),
            TensorDesc.empty(DType.FP8_UE4M3, (workload.heads, 128, key_rows // 16)),
            TensorDesc.empty(DType.BF16, (workload.num_query_tokens, workload.total_heads, 128)),
            workload.num_query_tokens,
            workload.num_kv_tokens,
            0,
            TensorDesc.empty(DType.U8, (cls.workspace_bytes(workload),)),
        )

    @classmethod
    def make_config(cls, workload: DenseNvfp4Workload) -> DenseNvfp4Config:
        return DenseNvfp4Config()

    @classmethod
    def make_workload(cls, arguments: DenseNvfp4Arguments) -> DenseNvfp4Workload:
        heads, query_rows, half_dim = arguments.query.shape
        key_heads, key_rows, key_half_dim = arguments.key.shape
        assert arguments.query.dtype == arguments.key.dtype == DType.U8
        assert heads == key_heads and half_dim == key_half_dim == 64
        assert query_rows == -(-arguments.num_query_tokens // 128) * 128
        assert key_rows == -(-arguments.num_kv_tokens // 128) * 128
        assert arguments.value.dtype == DType.U8
        assert arguments.value.shape == (heads, 128, key_rows // 2)
        assert arguments.query_scales.dtype == DType.FP8_UE4M3
        assert arguments.key_scales.dtype == DType.FP8_UE4M3
        assert arguments.value_scales.dtype == DType.FP8_UE4M3
        assert arguments.query_scales.shape == (heads, query_rows, 8)
        assert arguments.key_scales.shape == (heads, key_rows, 8)
        assert arguments.value_scales.shape == (heads, 128, key_rows // 16)
        num_query_tokens, total_heads, dim = arguments.output.shape
        assert arguments.output.dtype == DType.BF16 and dim == 128
        assert num_query_tokens == arguments.num_query_tokens
        assert arguments.num_kv_tokens > 0
        assert arguments.num_kv_tokens == arguments.num_query_tokens, "query slices are not supported on this path"
        assert 0 <= arguments.head_offset <= total_heads - heads
        workload = DenseNvfp4Workload(
            num_query_tokens=num_query_tokens,
            num_kv_tokens=arguments.num_kv_tokens,
            heads=heads,
            total_heads=total_heads,
        )
        assert arguments.workspace is not None, "dense nvfp4 attention needs workspace for the bf16 operands"
        assert arguments.workspace.num_bytes >= cls.workspace_bytes(workload)
        return workload

    @classmethod
    def tops(cls, arguments: DenseNvfp4Arguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        # executed as bf16 MMAs after the exact expansion of the fp4 operands
        return {MmaType.BF16BF16F32: 4 * workload.heads * workload.num_query_tokens * workload.num_kv_tokens * 128}

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.num_query_tokens),
            ctypes.c_int(w.num_kv_tokens),
            ctypes.c_int(a.head_offset),
            _lib.ptr(a.query),
            _lib.ptr(a.key),
            _lib.ptr(a.value),
            _lib.ptr(a.query_scales),
            _lib.ptr(a.key_scales),
            _lib.ptr(a.value_scales),
            ctypes.c_float(a.global_scales[0]),
            ctypes.c_float(a.global_scales[1]),
            ctypes.c_float(a.global_scales[2]),
            _lib.ptr(a.output),
            ctypes.c_int(w.heads),
            ctypes.c_int(w.total_heads),
            _lib.ptr(a.workspace),
            ctypes.c_size_t(a.workspace.num_bytes),
            ctypes.c_void_p(stream),
        )
