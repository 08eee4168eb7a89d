"""Dense bf16 attention for head slices, bound to ``nob200_dense_bf16_attention_d128``.

Interface of reference ``DenseBf16AttentionKernel``
(src/nano_omni/kernels/attention/dense_bf16.py:13-36, 198-255): same Workload
fields, Arguments fields and order, validation asserts and ``tops`` formula.
The Config keeps the reference's field names so stored configs still validate,
but the sm_100a kernel has one tile shape (two 128-row query tiles x 128 keys,
384 threads) and ignores other choices.
"""

from __future__ import annotations

import ctypes
import dataclasses
from typing import Literal

from pydantic import Field

from nano_omni_b200 import _lib
from nano_omni_b200.core import Arguments, Config, DType, Kernel, MmaType, TensorDesc, Workload, require_tensor


class DenseBf16AttentionWorkload(Workload):
    num_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    total_heads: int = Field(gt=0)


class DenseBf16AttentionConfig(Config):
    tile_query_tokens: Literal[32, 64, 128] = 128
    tile_kv_tokens: Literal[32, 64, 128] = 128
    threads: Literal[64, 128, 256, 384] = 384
    # key tiles divided over this many CTAs per (256 query rows, head); > 1 needs `workspace`
    kv_splits: int = Field(default=1, ge=1, le=64)


def choose_kv_splits(num_tokens: int, heads: int, sm_count: int = 148, num_kv_tokens: int | None = None) -> int:
    """Smallest number of key splits that fills the SMs well.

    One CTA works on 256 query rows of one head; with few heads the last wave of CTAs leaves SMs idle.
    Splitting the keys multiplies the CTAs; each split costs a merge pass and a shorter key loop, so a
    split count is only taken if it raises the fill by more than 5 % per extra split (measured on B200
    at 32768 tokens: 3 heads gain 7 % from 3 splits, 6 heads 5 % from 2, 12 heads lose 1.5 % with 2).
    """
    units = -(-num_tokens // 256) * heads
    key_tiles = -(-(num_tokens if num_kv_tokens is None else num_kv_tokens) // 128)  # query slices: Tq != Tk

    def fill(n: int) -> float:
        return n / (sm_count * -(-n // sm_count))

    best, best_score = 1, fill(units)
    for splits in range(2, 9):
        if key_tiles // splits < 16:
            break
        score = fill(units * splits) - 0.05 * (splits - 1)
        if score > best_score + 1e-9:
            best, best_score = splits, score
    return best


def splitkv_workspace_bytes(num_tokens: int, heads: int, kv_splits: int) -> int:
    if kv_splits <= 1:
        return 0
    share = num_tokens * heads
    return (kv_splits * share * 256 + 255) // 256 * 256 + kv_splits * share * 4


@dataclasses.dataclass(frozen=True, slots=True)
class DenseBf16AttentionArguments(Arguments):
    query: TensorDesc
    key: TensorDesc
    value: TensorDesc
    output: TensorDesc
    head_offset: int
    workspace: TensorDesc | None = None  # no counterpart in the reference: scratch for kv_splits > 1

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.query.shape[0]), ("head_offset", self.head_offset))


class DenseBf16AttentionKernel(
    Kernel[DenseBf16AttentionArguments, DenseBf16AttentionWorkload, DenseBf16AttentionConfig]
):
    name = "dense_bf16_attention_d128"
    symbol = "nob200_dense_bf16_attention_d128"

    @classmethod
    def make_arguments(cls, workload: DenseBf16AttentionWorkload) -> DenseBf16AttentionArguments:
        shape = (workload.num_tokens, workload.heads, 128)
        return DenseBf16AttentionArguments(
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.total_heads, 128)),
            0,
        )

    @classmethod
    def make_config(cls, workload: DenseBf16AttentionWorkload) -> DenseBf16AttentionConfig:
        return DenseBf16AttentionConfig()

    @classmethod
    def make_workload(cls, arguments: DenseBf16AttentionArguments) -> DenseBf16AttentionWorkload:
        # The query fixes tokens and heads of the slice; key and value repeat its layout, the output is the
        # full-width tensor [tokens, total_heads, 128] in which the slice starts at head_offset.
        assert len(arguments.query.shape) == 3 and len(arguments.output.shape) == 3, "attention tensors have rank 3"
        num_tokens, heads, _ = arguments.query.shape
        total_heads = arguments.output.shape[1]
        slice_shape = (num_tokens, heads, 128)
        for what, tensor, shape in (
            ("query", arguments.query, slice_shape),
            ("key", arguments.key, slice_shape),
            ("value", arguments.value, slice_shape),
            ("output", arguments.output, (num_tokens, total_heads, 128)),
        ):
            require_tensor(tensor, DType.BF16, shape, what)
        assert arguments.head_offset >= 0, "head_offset is negative"
        assert arguments.head_offset + heads <= total_heads, "head slice ends past the output's heads"
        return DenseBf16AttentionWorkload(num_tokens=num_tokens, heads=heads, total_heads=total_heads)

    @classmethod
    def tops(cls, arguments: DenseBf16AttentionArguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        return {MmaType.BF16BF16F32: 4 * workload.heads * workload.num_tokens**2 * 128}

    def compile(self) -> None:
        if self.compiled is None:
            self.compiled = (_lib.symbol(type(self).symbol), _lib.symbol(type(self).symbol + "_splitkv"))

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        plain, split = function
        splits = self.config.kv_splits
        if splits > 1:
            need = splitkv_workspace_bytes(w.num_tokens, w.heads, splits)
            assert a.workspace is not None and a.workspace.num_bytes >= need, "kv_splits > 1 needs workspace"
            return split(
                ctypes.c_int(w.num_tokens),
                ctypes.c_int(a.head_offset),
                _lib.ptr(a.query),
                _lib.ptr(a.key),
                _lib.ptr(a.value),
                _lib.ptr(a.output),
                ctypes.c_int(w.heads),
                ctypes.c_int(w.total_heads),
                ctypes.c_int(splits),
                _lib.ptr(a.workspace),
                ctypes.c_size_t(a.workspace.num_bytes),
                ctypes.c_void_p(stream),
            )
        function = plain
        return function(
            ctypes.c_int(w.num_tokens),
            ctypes.c_int(a.head_offset),
            _lib.ptr(a.query),
            _lib.ptr(a.key),
            _lib.ptr(a.value),
            _lib.ptr(a.output),
            ctypes.c_int(w.heads),
            ctypes.c_int(w.total_heads),
            ctypes.c_void_p(stream),
        )
