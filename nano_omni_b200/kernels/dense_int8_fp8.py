"""Dense int8-QK / fp8-PV attention, bound to ``nob200_dense_int8_fp8_d128``.

Interface of reference ``DenseInt8Fp8AttentionKernel``
(src/nano_omni/kernels/attention/int8_fp8/dense.py:316-481): same Workload and
Arguments fields, validation and ``tops``.  Query and key/value token counts may
differ (query slices against persistent quantised K/V,
src/nano_omni/ops/minimax_h3/attention_slices.py:60-161).  Trailing fields without a counterpart in the
reference: ``query_block`` / ``key_block``, the tokens per int8 scale (32 / 64 in the reference; 128 for operands
quantised in 128-token blocks), and ``workspace`` with Config ``kv_splits`` (key tiles divided over several CTAs
per 256 query rows and merged by their log-sum-exp: a 4096-token query slice x 56 heads is 896 CTAs, 6.05 waves of
148 SMs).
"""

from __future__ import annotations

import ctypes
import dataclasses
from typing import Literal

from pydantic import Field

from nano_omni_b200 import _lib
from nano_omni_b200.core import Arguments, Config, DType, Kernel, MmaType, TensorDesc, Workload, require_tensor
from nano_omni_b200.kernels.dense_bf16 import splitkv_workspace_bytes


class DenseInt8Fp8AttentionWorkload(Workload):
    num_kv_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    num_query_tokens: int = Field(gt=0)
    query_block: Literal[32, 64, 128] = 32
    key_block: Literal[64, 128] = 64


class DenseInt8Fp8AttentionConfig(Config):
    tile_query_tokens: Literal[64, 128, 256] = 128
    tile_kv_tokens: Literal[64, 128] = 128
    threads: Literal[64, 128, 256, 384] = 384
    # key tiles divided over this many CTAs per (256 query rows, head); > 1 needs `workspace`
    kv_splits: int = Field(default=1, ge=1, le=64)


@dataclasses.dataclass(frozen=True, slots=True)
class DenseInt8Fp8AttentionArguments(Arguments):
    query: TensorDesc
    key: TensorDesc
    value: TensorDesc
    query_scale: TensorDesc
    key_scale: TensorDesc
    value_scale: TensorDesc
    output: TensorDesc
    num_kv_tokens: int
    heads: int
    num_query_tokens: int
    query_block: int = 32
    key_block: int = 64
    workspace: TensorDesc | None = None  # no counterpart in the reference: scratch for kv_splits > 1

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_kv_tokens", self.num_kv_tokens), ("num_query_tokens", self.num_query_tokens))


class DenseInt8Fp8AttentionKernel(
    Kernel[DenseInt8Fp8AttentionArguments, DenseInt8Fp8AttentionWorkload, DenseInt8Fp8AttentionConfig]
):
    name = "dense_int8_fp8_d128"
    symbol = "nob200_dense_int8_fp8_d128_splitkv"

    @classmethod
    def make_arguments(cls, workload: DenseInt8Fp8AttentionWorkload) -> DenseInt8Fp8AttentionArguments:
        qb, kb = workload.query_block, workload.key_block
        query_rows = -(-workload.num_query_tokens // qb) * qb
        key_rows = -(-workload.num_kv_tokens // kb) * kb
        value_columns = -(-workload.num_kv_tokens // 64) * 64
        return DenseInt8Fp8AttentionArguments(
            query=TensorDesc.empty(DType.I8, (workload.heads, query_rows, 128)),
            key=TensorDesc.empty(DType.I8, (workload.heads, key_rows, 128)),
            value=TensorDesc.empty(DType.FP8_E4M3, (workload.heads, 128, value_columns)),
            query_scale=TensorDesc.empty(DType.F32, (workload.heads, query_rows // qb)),
            key_scale=TensorDesc.empty(DType.F32, (workload.heads, key_rows // kb)),
            value_scale=TensorDesc.empty(DType.F32, (workload.heads, 128)),
            output=TensorDesc.empty(DType.BF16, (workload.num_query_tokens, workload.heads * 128)),
            num_kv_tokens=workload.num_kv_tokens,
            heads=workload.heads,
            num_query_tokens=workload.num_query_tokens,
            query_block=qb,
            key_block=kb,
        )

    @classmethod
    def make_config(cls, workload: DenseInt8Fp8AttentionWorkload) -> DenseInt8Fp8AttentionConfig:
        return DenseInt8Fp8AttentionConfig()

    @classmethod
    def make_workload(cls, arguments: DenseInt8Fp8AttentionArguments) -> DenseInt8Fp8AttentionWorkload:
        # Q and K rows are padded to whole scale blocks (one f32 scale per block and head), V is stored transposed
        # with its token axis padded to the 64 tokens one fp8 contraction step covers.
        heads, qb, kb = arguments.heads, arguments.query_block, arguments.key_block
        query_blocks = -(-arguments.num_query_tokens // qb)
        key_blocks = -(-arguments.num_kv_tokens // kb)
        value_columns = -(-arguments.num_kv_tokens // 64) * 64
        expected = {
            "query": (DType.I8, (heads, query_blocks * qb, 128)),
            "key": (DType.I8, (heads, key_blocks * kb, 128)),
            "value": (DType.FP8_E4M3, (heads, 128, value_columns)),
            "query_scale": (DType.F32, (heads, query_blocks)),
            "key_scale": (DType.F32, (heads, key_blocks)),
            "value_scale": (DType.F32, (heads, 128)),
            "output": (DType.BF16, (arguments.num_query_tokens, heads * 128)),
        }
        for what, (dtype, shape) in expected.items():
            require_tensor(getattr(arguments, what), dtype, shape, what)
        return DenseInt8Fp8AttentionWorkload(
            num_kv_tokens=arguments.num_kv_tokens,
            heads=arguments.heads,
            num_query_tokens=arguments.num_query_tokens,
            query_block=qb,
            key_block=kb,
        )

    @classmethod
    def tops(cls, arguments: DenseInt8Fp8AttentionArguments) -> dict[MmaType, int]:
        count = 2 * arguments.heads * arguments.num_query_tokens * arguments.num_kv_tokens * 128
        return {MmaType.I8I8I32: count, MmaType.F8F8F32: count}

    def _launch(self, function, stream: int) -> int:
        a = self.arguments
        splits = self.config.kv_splits
        if splits > 1:
            need = splitkv_workspace_bytes(a.num_query_tokens, a.heads, splits)
            assert a.workspace is not None and a.workspace.num_bytes >= need, "kv_splits > 1 needs workspace"
        return function(
            ctypes.c_int(a.num_kv_tokens),
            ctypes.c_int(a.num_query_tokens),
            _lib.ptr(a.query),
            _lib.ptr(a.key),
            _lib.ptr(a.value),
            _lib.ptr(a.query_scale),
            _lib.ptr(a.key_scale),
            _lib.ptr(a.value_scale),
            _lib.ptr(a.output),
            ctypes.c_int(a.heads),
            ctypes.c_int(a.query_block),
            ctypes.c_int(a.key_block),
            ctypes.c_int(splits),
            _lib.ptr(a.workspace) if splits > 1 else ctypes.c_void_p(0),
            ctypes.c_size_t(a.workspace.num_bytes if splits > 1 else 0),
            ctypes.c_void_p(stream),
        )
