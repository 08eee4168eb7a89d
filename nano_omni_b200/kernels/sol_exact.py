"""Exact stage and finalize of the quantised sol paths.

Interfaces of the reference classes with the same ``name``:

* ``sol_int8_fp8_attention_d128``  src/nano_omni/kernels/attention/int8_fp8/sol.py:45-165
* ``sol_nvfp4_attention_d128``     src/nano_omni/kernels/attention/sol_nvfp4.py:49-715
* ``sol_nvfp4_finalize``           src/nano_omni/kernels/attention/nvfp4/sol_finalize.py:13-210

The exact stage writes an un-normalised numerator and the online-softmax state (row maximum in raw
q.k units, sum of probabilities); finalize merges the pooled pseudo-keys of the unselected blocks and
normalises.  ``exact`` and ``output`` of finalize may be the same tensor.  Trailing fields without a
counterpart in the reference: ``workspace`` (bf16 expansion of the nvfp4 operands) and ``block``.
"""

from __future__ import annotations

import ctypes
import dataclasses
import math
from typing import Literal

from pydantic import Field

from nano_omni_b200 import _lib
from nano_omni_b200.core import Arguments, Config, DType, Kernel, MmaType, TensorDesc, Workload


def expected_exact_pairs(num_query_tokens: int, num_kv_tokens: int, num_protected_blocks: int, tau: float) -> int:
    """Expected number of (query, key) token pairs that attend exactly under threshold routing.

    Protected key blocks and the three-block band around the diagonal always attend; any other block
    with the Gaussian tail probability of ``tau`` (sol_nvfp4.py:29-46).
    """
    qb_count, kb_count = -(-num_query_tokens // 64), -(-num_kv_tokens // 64)
    tail = 0.5 * math.erfc(tau / math.sqrt(2))
    qlen = [min(64, num_query_tokens - b * 64) for b in range(qb_count)]
    klen = [min(64, num_kv_tokens - b * 64) for b in range(kb_count)]
    total = 0.0
    for qb in range(qb_count):
        always = sum(klen[kb] for kb in range(kb_count) if kb < num_protected_blocks or abs(qb - kb) <= 1)
        total += qlen[qb] * (always + tail * (num_kv_tokens - always))
    return round(total)


# ------------------------------------------------------------------ int8-fp8 exact stage
class SolInt8Fp8AttentionWorkload(Workload):
    num_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    total_heads: int = Field(gt=0)


class SolInt8Fp8AttentionConfig(Config):
    tile_query_tokens: Literal[64, 128] = 128
    tile_kv_tokens: Literal[64, 128] = 128
    threads: Literal[64, 128, 384] = 384


@dataclasses.dataclass(frozen=True, slots=True)
class SolInt8Fp8AttentionArguments(Arguments):
    query: TensorDesc
    key: TensorDesc
    value: TensorDesc
    query_scale: TensorDesc
    key_scale: TensorDesc
    value_scale: TensorDesc
    selected: TensorDesc
    output: TensorDesc
    state: TensorDesc
    num_tokens: int
    head_offset: int
    tau: float
    num_protected_blocks: int

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.num_tokens), ("head_offset", self.head_offset))


class SolInt8Fp8AttentionKernel(
    Kernel[SolInt8Fp8AttentionArguments, SolInt8Fp8AttentionWorkload, SolInt8Fp8AttentionConfig]
):
    name = "sol_int8_fp8_attention_d128"
    symbol = "nob200_sol_int8_fp8_attention_d128"

    @classmethod
    def make_arguments(cls, workload: SolInt8Fp8AttentionWorkload) -> SolInt8Fp8AttentionArguments:
        nb = -(-workload.num_tokens // 64)
        qrows, krows = -(-workload.num_tokens // 32) * 32, nb * 64
        h = workload.heads
        return SolInt8Fp8AttentionArguments(
            TensorDesc.empty(DType.I8, (h, qrows, 128)),
            TensorDesc.empty(DType.I8, (h, krows, 128)),
            TensorDesc.empty(DType.FP8_E4M3, (h, 128, krows)),
            TensorDesc.empty(DType.F32, (h, qrows // 32)),
            TensorDesc.empty(DType.F32, (h, nb)),
            TensorDesc.empty(DType.F32, (h, 128)),
            TensorDesc.empty(DType.U8, (nb, h, nb)),
            TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.total_heads, 128)),
            TensorDesc.empty(DType.F32, (workload.num_tokens, workload.total_heads, 2)),
            workload.num_tokens,
            0,
            1.0,
            0,
        )

    @classmethod
    def make_config(cls, workload: SolInt8Fp8AttentionWorkload) -> SolInt8Fp8AttentionConfig:
        return SolInt8Fp8AttentionConfig()

    @classmethod
    def make_workload(cls, arguments: SolInt8Fp8AttentionArguments) -> SolInt8Fp8AttentionWorkload:
        heads, qrows, dim = arguments.query.shape
        nb = -(-arguments.num_tokens // 64)
        krows = nb * 64
        assert arguments.query.dtype == arguments.key.dtype == DType.I8 and dim == 128
        assert qrows == -(-arguments.num_tokens // 32) * 32
        assert arguments.key.shape == (heads, krows, 128)
        assert arguments.value.dtype == DType.FP8_E4M3 and arguments.value.shape == (heads, 128, krows)
        assert arguments.query_scale.dtype == arguments.key_scale.dtype == arguments.value_scale.dtype == DType.F32
        assert arguments.query_scale.shape == (heads, qrows // 32)
        assert arguments.key_scale.shape == (heads, nb)
        assert arguments.value_scale.shape == (heads, 128)
        assert arguments.selected.dtype == DType.U8 and arguments.selected.shape == (nb, heads, nb)
        assert arguments.output.dtype == DType.BF16 and arguments.state.dtype == DType.F32
        num_tokens, total_heads, out_dim = arguments.output.shape
        assert num_tokens == arguments.num_tokens and out_dim == 128
        assert arguments.state.shape == (num_tokens, total_heads, 2)
        assert 0 <= arguments.head_offset <= total_heads - heads
        assert arguments.tau == 1.0
        assert 0 <= arguments.num_protected_blocks <= nb
        return SolInt8Fp8AttentionWorkload(num_tokens=num_tokens, heads=heads, total_heads=total_heads)

    @classmethod
    def tops(cls, arguments: SolInt8Fp8AttentionArguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        pairs = expected_exact_pairs(workload.num_tokens, workload.num_tokens, arguments.num_protected_blocks, 1.0)
        operations = 2 * workload.heads * 128 * pairs
        return {MmaType.I8I8I32: operations, MmaType.F8F8F32: operations}

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.num_tokens),
            ctypes.c_int(a.head_offset),
            _lib.ptr(a.query),
            _lib.ptr(a.key),
            _lib.ptr(a.value),
            _lib.ptr(a.query_scale),
            _lib.ptr(a.key_scale),
            _lib.ptr(a.value_scale),
            _lib.ptr(a.selected),
            _lib.ptr(a.output),
            _lib.ptr(a.state),
            ctypes.c_int(w.heads),
            ctypes.c_int(w.total_heads),
            ctypes.c_void_p(stream),
        )


# ------------------------------------------------------------------ nvfp4 exact stage
class SolNvfp4Workload(Workload):
    num_query_tokens: int = Field(gt=0)
    num_kv_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    total_heads: int = Field(gt=0)


class SolNvfp4Config(Config):
    tile_query_tokens: int = 128
    tile_kv_tokens: int = 128
    threads: int = 384


@dataclasses.dataclass(frozen=True, slots=True)
class SolNvfp4Arguments(Arguments):
    query: TensorDesc
    key: TensorDesc
    value: TensorDesc
    query_scales: TensorDesc
    key_scales: TensorDesc
    value_scales: TensorDesc
    selected: TensorDesc
    output: TensorDesc
    state: TensorDesc
    num_query_tokens: int
    num_kv_tokens: int
    head_offset: int
    tau: float
    num_protected_blocks: int
    workspace: TensorDesc | None = None

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (
            ("num_query_tokens", self.num_query_tokens),
            ("num_kv_tokens", self.num_kv_tokens),
            ("head_offset", self.head_offset),
        )


def _align(n: int) -> int:
    return (n + 255) // 256 * 256


class SolNvfp4Kernel(Kernel[SolNvfp4Arguments, SolNvfp4Workload, SolNvfp4Config]):
    name = "sol_nvfp4_attention_d128"
    symbol = "nob200_sol_nvfp4_attention_d128"

    @classmethod
    def workspace_bytes(cls, workload: SolNvfp4Workload) -> int:
        return _align(workload.num_query_tokens * workload.heads * 256) + 2 * _align(
            workload.num_kv_tokens * workload.heads * 256
        )

    @classmethod
    def make_arguments(cls, workload: SolNvfp4Workload) -> SolNvfp4Arguments:
        qrows = -(-workload.num_query_tokens // 128) * 128
        krows = -(-workload.num_kv_tokens // 128) * 128
        h = workload.heads
        return SolNvfp4Arguments(
            TensorDesc.empty(DType.U8, (h, qrows, 64)),
            TensorDesc.empty(DType.U8, (h, krows, 64)),
            TensorDesc.empty(DType.U8, (h, 128, krows // 2)),
            TensorDesc.empty(DType.FP8_UE4M3, (h, qrows, 8)),
            TensorDesc.empty(DType.FP8_UE4M3, (h, krows, 8)),
            TensorDesc.empty(DType.FP8_UE4M3, (h, 128, krows // 16)),
            TensorDesc.empty(DType.U8, (-(-workload.num_query_tokens // 64), h, -(-workload.num_kv_tokens // 64))),
            TensorDesc.empty(DType.BF16, (workload.num_query_tokens, workload.total_heads, 128)),
            TensorDesc.empty(DType.F32, (workload.num_query_tokens, workload.total_heads, 2)),
            workload.num_query_tokens,
            workload.num_kv_tokens,
            0,
            1.0,
            1,
            TensorDesc.empty(DType.U8, (cls.workspace_bytes(workload),)),
        )

    @classmethod
    def make_config(cls, workload: SolNvfp4Workload) -> SolNvfp4Config:
        return SolNvfp4Config()

    @classmethod
    def make_workload(cls, arguments: SolNvfp4Arguments) -> SolNvfp4Workload:
        heads, qrows, half_dim = arguments.query.shape
        key_heads, krows, key_half_dim = arguments.key.shape
        assert arguments.query.dtype == arguments.key.dtype == DType.U8
        assert heads == key_heads and half_dim == key_half_dim == 64
        assert qrows == -(-arguments.num_query_tokens // 128) * 128
        assert krows == -(-arguments.num_kv_tokens // 128) * 128
        assert arguments.value.dtype == DType.U8 and arguments.value.shape == (heads, 128, krows // 2)
        assert arguments.query_scales.dtype == DType.FP8_UE4M3
        assert arguments.key_scales.dtype == DType.FP8_UE4M3
        assert arguments.value_scales.dtype == DType.FP8_UE4M3
        assert arguments.query_scales.shape == (heads, qrows, 8)
        assert arguments.key_scales.shape == (heads, krows, 8)
        assert arguments.value_scales.shape == (heads, 128, krows // 16)
        assert arguments.selected.dtype == DType.U8
        assert arguments.selected.shape == (
            -(-arguments.num_query_tokens // 64),
            heads,
            -(-arguments.num_kv_tokens // 64),
        )
        num_query_tokens, total_heads, dim = arguments.output.shape
        assert arguments.output.dtype == DType.BF16 and dim == 128
        assert arguments.state.dtype == DType.F32 and arguments.state.shape == (num_query_tokens, total_heads, 2)
        assert num_query_tokens == arguments.num_query_tokens
        assert arguments.num_kv_tokens > 0
        assert arguments.num_kv_tokens == arguments.num_query_tokens, "query slices are not supported on this path"
        assert 0 <= arguments.head_offset <= total_heads - heads
        assert arguments.tau == 1.0
        assert 1 <= arguments.num_protected_blocks <= -(-arguments.num_kv_tokens // 64)
        workload = SolNvfp4Workload(
            num_query_tokens=num_query_tokens,
            num_kv_tokens=arguments.num_kv_tokens,
            heads=heads,
            total_heads=total_heads,
        )
        assert arguments.workspace is not None, "sol nvfp4 attention needs workspace for the bf16 operands"
        assert arguments.workspace.num_bytes >= cls.workspace_bytes(workload)
        return workload

    @classmethod
    def tops(cls, arguments: SolNvfp4Arguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        pairs = expected_exact_pairs(
            workload.num_query_tokens, workload.num_kv_tokens, arguments.num_protected_blocks, arguments.tau
        )
        # executed as bf16 MMAs after the exact expansion of the fp4 operands
        return {MmaType.BF16BF16F32: 4 * workload.heads * 128 * pairs}

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
            _lib.ptr(a.selected),
            _lib.ptr(a.output),
            _lib.ptr(a.state),
            ctypes.c_int(w.heads),
            ctypes.c_int(w.total_heads),
            _lib.ptr(a.workspace),
            ctypes.c_size_t(a.workspace.num_bytes),
            ctypes.c_void_p(stream),
        )


# ------------------------------------------------------------------ finalize
class SolNvfp4FinalizeWorkload(Workload):
    num_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    total_heads: int = Field(gt=0)
    block: Literal[64, 128] = 64


class SolNvfp4FinalizeConfig(Config):
    threads: Literal[64, 128, 256, 384] = 384


@dataclasses.dataclass(frozen=True, slots=True)
class SolNvfp4FinalizeArguments(Arguments):
    query: TensorDesc
    pooled: TensorDesc
    selected: TensorDesc
    exact: TensorDesc
    state: TensorDesc
    output: TensorDesc
    head_offset: int
    block: int = 64

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.query.shape[0]), ("head_offset", self.head_offset))


class SolNvfp4FinalizeKernel(Kernel[SolNvfp4FinalizeArguments, SolNvfp4FinalizeWorkload, SolNvfp4FinalizeConfig]):
    name = "sol_nvfp4_finalize"
    symbol = "nob200_sol_nvfp4_finalize"

    @classmethod
    def make_arguments(cls, workload: SolNvfp4FinalizeWorkload) -> SolNvfp4FinalizeArguments:
        nb = -(-workload.num_tokens // workload.block)
        wide = (workload.num_tokens, workload.total_heads, 128)
        return SolNvfp4FinalizeArguments(
            TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.heads, 128)),
            TensorDesc.empty(DType.BF16, (3, workload.heads, nb, 128)),
            TensorDesc.empty(DType.U8, (nb, workload.heads, nb)),
            TensorDesc.empty(DType.BF16, wide),
            TensorDesc.empty(DType.F32, (workload.num_tokens, workload.total_heads, 2)),
            TensorDesc.empty(DType.BF16, wide),
            0,
            workload.block,
        )

    @classmethod
    def make_config(cls, workload: SolNvfp4FinalizeWorkload) -> SolNvfp4FinalizeConfig:
        return SolNvfp4FinalizeConfig()

    @classmethod
    def make_workload(cls, arguments: SolNvfp4FinalizeArguments) -> SolNvfp4FinalizeWorkload:
        num_tokens, heads, dim = arguments.query.shape
        nb = -(-num_tokens // arguments.block)
        assert arguments.query.dtype == DType.BF16 and dim == 128
        assert arguments.pooled.dtype == DType.BF16 and arguments.pooled.shape == (3, heads, nb, 128)
        assert arguments.selected.dtype == DType.U8 and arguments.selected.shape == (nb, heads, nb)
        assert arguments.exact.dtype == arguments.output.dtype == DType.BF16
        assert arguments.state.dtype == DType.F32
        assert arguments.exact.shape == arguments.output.shape
        total_heads = arguments.output.shape[1]
        assert arguments.output.shape == (num_tokens, total_heads, 128)
        assert arguments.state.shape == (num_tokens, total_heads, 2)
        assert 0 <= arguments.head_offset <= total_heads - heads
        return SolNvfp4FinalizeWorkload(num_tokens=num_tokens, heads=heads, total_heads=total_heads, block=arguments.block)

    @classmethod
    def tops(cls, arguments: SolNvfp4FinalizeArguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        nb = -(-workload.num_tokens // workload.block)
        return {MmaType.BF16BF16F32: 4 * workload.heads * 128 * workload.num_tokens * nb}

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.num_tokens),
            ctypes.c_int(a.head_offset),
            _lib.ptr(a.query),
            _lib.ptr(a.pooled),
            _lib.ptr(a.selected),
            _lib.ptr(a.exact),
            _lib.ptr(a.state),
            _lib.ptr(a.output),
            ctypes.c_int(w.heads),
            ctypes.c_int(w.total_heads),
            ctypes.c_int(w.block),
            ctypes.c_void_p(stream),
        )
