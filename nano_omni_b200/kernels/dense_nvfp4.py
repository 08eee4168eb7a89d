"""Dense attention on NVFP4 operands, bound to ``nob200_dense_nvfp4_attention_d128``.

Interface of reference ``DenseNvfp4Kernel`` (src/nano_omni/kernels/attention/dense_nvfp4.py:18-52,
562-676): same Arguments fields and order, the same shapes accepted and rejected, the same ``tops``.  Both
products run as block-scaled fp4 tensor-core MMAs; probabilities are re-quantised to e2m1 with one ue4m3 scale per
16 keys as in the reference kernel (dense_nvfp4.py:255-289).  The trailing ``workspace`` (no counterpart in the
reference) is accepted for callers written against the earlier bf16-expansion path and ignored: the kernel needs
no scratch.
"""

from __future__ import annotations

import ctypes
import dataclasses

from pydantic import Field

from nano_omni_b200 import _lib
from nano_omni_b200.core import Arguments, Config, DType, Kernel, MmaType, TensorDesc, Workload, require_tensor


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


def _padded(tokens: int) -> int:
    """Rows of a packed operand: ``nvfp4_prepare`` pads tokens to whole 128-row scale atoms."""
    return -(-tokens // 128) * 128


class DenseNvfp4Kernel(Kernel[DenseNvfp4Arguments, DenseNvfp4Workload, DenseNvfp4Config]):
    name = "dense_nvfp4_attention_d128"
    symbol = "nob200_dense_nvfp4_attention_d128_global"
    reference_rtol = 0.03
    reference_atol = 0.03

    @classmethod
    def workspace_bytes(cls, workload: DenseNvfp4Workload) -> int:
        return 0

    @classmethod
    def make_arguments(cls, workload: DenseNvfp4Workload) -> DenseNvfp4Arguments:
        heads, rows_q, rows_k = workload.heads, _padded(workload.num_query_tokens), _padded(workload.num_kv_tokens)
        packed = lambda *shape: TensorDesc.empty(DType.U8, shape)  # noqa: E731
        scales = lambda *shape: TensorDesc.empty(DType.FP8_UE4M3, shape)  # noqa: E731
        return DenseNvfp4Arguments(
            query=packed(heads, rows_q, 64),
            key=packed(heads, rows_k, 64),
            value=packed(heads, 128, rows_k // 2),
            query_scales=scales(heads, rows_q, 8),
            key_scales=scales(heads, rows_k, 8),
            value_scales=scales(heads, 128, rows_k // 16),
            output=TensorDesc.empty(DType.BF16, (workload.num_query_tokens, workload.total_heads, 128)),
            num_query_tokens=workload.num_query_tokens,
            num_kv_tokens=workload.num_kv_tokens,
            head_offset=0,
        )

    @classmethod
    def make_config(cls, workload: DenseNvfp4Workload) -> DenseNvfp4Config:
        return DenseNvfp4Config()

    @classmethod
    def make_workload(cls, arguments: DenseNvfp4Arguments) -> DenseNvfp4Workload:
        a = arguments
        assert a.num_query_tokens > 0 and a.num_kv_tokens > 0, "token counts must be positive"
        assert len(a.query.shape) == 3, f"query: expected [heads, rows, 64], got {tuple(a.query.shape)}"
        heads = a.query.shape[0]
        rows_q, rows_k = _padded(a.num_query_tokens), _padded(a.num_kv_tokens)
        # every operand follows from (heads, token counts): Q and K grouped along head_dim, V along tokens
        for what, tensor, dtype, shape in (
            ("query", a.query, DType.U8, (heads, rows_q, 64)),
            ("key", a.key, DType.U8, (heads, rows_k, 64)),
            ("value", a.value, DType.U8, (heads, 128, rows_k // 2)),
            ("query_scales", a.query_scales, DType.FP8_UE4M3, (heads, rows_q, 8)),
            ("key_scales", a.key_scales, DType.FP8_UE4M3, (heads, rows_k, 8)),
            ("value_scales", a.value_scales, DType.FP8_UE4M3, (heads, 128, rows_k // 16)),
        ):
            require_tensor(tensor, dtype, shape, what)
        assert a.output.dtype == DType.BF16 and len(a.output.shape) == 3 and a.output.shape[2] == 128, "output: bf16 [tokens, heads, 128]"
        assert a.output.shape[0] == a.num_query_tokens, "output rows must equal num_query_tokens"
        total_heads = a.output.shape[1]
        assert 0 <= a.head_offset <= total_heads - heads, f"head_offset {a.head_offset} outside [0, {total_heads - heads}]"
        return DenseNvfp4Workload(
            num_query_tokens=a.num_query_tokens, num_kv_tokens=a.num_kv_tokens, heads=heads, total_heads=total_heads
        )

    @classmethod
    def tops(cls, arguments: DenseNvfp4Arguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        return {MmaType.F4F4F32: 4 * workload.heads * workload.num_query_tokens * workload.num_kv_tokens * 128}

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
            ctypes.c_void_p(0),
            ctypes.c_size_t(0),
            ctypes.c_void_p(stream),
        )
