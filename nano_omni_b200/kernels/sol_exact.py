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
from nano_omni_b200.core import require_tensor, Arguments, Config, DType, Kernel, MmaType, TensorDesc, Workload


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


def _padded(tokens: int) -> int:
    return -(-tokens // 128) * 128


def _blocks64(tokens: int) -> int:
    return -(-tokens // 64)


class SolNvfp4Kernel(Kernel[SolNvfp4Arguments, SolNvfp4Workload, SolNvfp4Config]):
    name = "sol_nvfp4_attention_d128"
    symbol = "nob200_sol_nvfp4_attention_d128"

    @classmethod
    def workspace_bytes(cls, workload: SolNvfp4Workload) -> int:
        return 0  # the fp4 kernel reads the packed operands directly

    @classmethod
    def make_arguments(cls, workload: SolNvfp4Workload) -> SolNvfp4Arguments:
        h, rows_q, rows_k = workload.heads, _padded(workload.num_query_tokens), _padded(workload.num_kv_tokens)
        packed = lambda *shape: TensorDesc.empty(DType.U8, shape)  # noqa: E731
        scales = lambda *shape: TensorDesc.empty(DType.FP8_UE4M3, shape)  # noqa: E731
        return SolNvfp4Arguments(
            query=packed(h, rows_q, 64),
            key=packed(h, rows_k, 64),
            value=packed(h, 128, rows_k // 2),
            query_scales=scales(h, rows_q, 8),
            key_scales=scales(h, rows_k, 8),
            value_scales=scales(h, 128, rows_k // 16),
            selected=packed(_blocks64(workload.num_query_tokens), h, _blocks64(workload.num_kv_tokens)),
            output=TensorDesc.empty(DType.BF16, (workload.num_query_tokens, workload.total_heads, 128)),
            state=TensorDesc.empty(DType.F32, (workload.num_query_tokens, workload.total_heads, 2)),
            num_query_tokens=workload.num_query_tokens,
            num_kv_tokens=workload.num_kv_tokens,
            head_offset=0,
            tau=1.0,
            num_protected_blocks=1,
        )

    @classmethod
    def make_config(cls, workload: SolNvfp4Workload) -> SolNvfp4Config:
        return SolNvfp4Config()

    @classmethod
    def make_workload(cls, arguments: SolNvfp4Arguments) -> SolNvfp4Workload:
        a = arguments
        assert a.num_query_tokens > 0 and a.num_kv_tokens > 0, "token counts must be positive"
        assert len(a.query.shape) == 3, f"query: expected [heads, rows, 64], got {tuple(a.query.shape)}"
        heads = a.query.shape[0]
        rows_q, rows_k = _padded(a.num_query_tokens), _padded(a.num_kv_tokens)
        assert a.output.dtype == DType.BF16 and len(a.output.shape) == 3 and a.output.shape[2] == 128, "output: bf16 [tokens, heads, 128]"
        total_heads = a.output.shape[1]
        for what, tensor, dtype, shape in (
            ("query", a.query, DType.U8, (heads, rows_q, 64)),
            ("key", a.key, DType.U8, (heads, rows_k, 64)),
            ("value", a.value, DType.U8, (heads, 128, rows_k // 2)),
            ("query_scales", a.query_scales, DType.FP8_UE4M3, (heads, rows_q, 8)),
            ("key_scales", a.key_scales, DType.FP8_UE4M3, (heads, rows_k, 8)),
            ("value_scales", a.value_scales, DType.FP8_UE4M3, (heads, 128, rows_k // 16)),
            ("selected", a.selected, DType.U8, (_blocks64(a.num_query_tokens), heads, _blocks64(a.num_kv_tokens))),
            ("output", a.output, DType.BF16, (a.num_query_tokens, total_heads, 128)),
            ("state", a.state, DType.F32, (a.num_query_tokens, total_heads, 2)),
        ):
            require_tensor(tensor, dtype, shape, what)
        assert 0 <= a.head_offset <= total_heads - heads, f"head_offset {a.head_offset} outside [0, {total_heads - heads}]"
        assert a.tau == 1.0, "the routing threshold is fixed at one standard deviation"
        # key block 0 always attends on this path, so at least one block must be protected (sol_nvfp4.py:697)
        assert 1 <= a.num_protected_blocks <= _blocks64(a.num_kv_tokens), "num_protected_blocks outside [1, key blocks]"
        return SolNvfp4Workload(
            num_query_tokens=a.num_query_tokens, num_kv_tokens=a.num_kv_tokens, heads=heads, total_heads=total_heads
        )

    @classmethod
    def tops(cls, arguments: SolNvfp4Arguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        pairs = expected_exact_pairs(
            workload.num_query_tokens, workload.num_kv_tokens, arguments.num_protected_blocks, arguments.tau
        )
        return {MmaType.F4F4F32: 4 * workload.heads * 128 * pairs}

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
            ctypes.c_void_p(0),
            ctypes.c_size_t(0),
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
