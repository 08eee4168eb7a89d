"""Routing kernels of the sol block-sparse attention path.

Interfaces of the reference classes with the same ``name``:

* ``sol_pool``           src/nano_omni/kernels/attention/sol/pool.py:14-114
* ``sol_int8_fp8_pool``  src/nano_omni/kernels/attention/int8_fp8/sol_pool.py:14-119
* ``sol_nvfp4_pool``     src/nano_omni/kernels/attention/nvfp4/sol_pool.py (same arguments)
* ``sol_stats``          src/nano_omni/kernels/attention/sol/stats.py:14-103
* ``sol_nvfp4_select``   src/nano_omni/kernels/attention/nvfp4/sol_select.py:15-201

Trailing, defaulted fields without a counterpart in the reference: ``block`` (64 as in
the reference, or 128, the tile of the sm_100a attention kernels) and, for the selector,
``topk_fraction`` / ``workspace`` (keep the top fraction of key blocks instead of thresholding).
"""

from __future__ import annotations

import ctypes
import dataclasses
import math
from typing import Literal

from pydantic import Field

from nano_omni_b200 import _lib
from nano_omni_b200.core import Arguments, Config, DType, Kernel, MmaType, TensorDesc, Workload


class SolPrepareConfig(Config):
    threads: Literal[64, 128, 256] = 64


class SolPoolWorkload(Workload):
    num_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    block: Literal[64, 128] = 64


@dataclasses.dataclass(frozen=True, slots=True)
class SolPoolArguments(Arguments):
    key: TensorDesc
    value: TensorDesc
    output: TensorDesc
    block: int = 64

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.key.shape[0]),)


@dataclasses.dataclass(frozen=True, slots=True)
class SolCenteredPoolArguments(Arguments):
    key: TensorDesc
    value: TensorDesc
    key_mean: TensorDesc
    output: TensorDesc
    block: int = 64

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.key.shape[0]),)


def _pool_launch(kernel, function, stream: int, key_mean) -> int:
    a, w = kernel.arguments, kernel.workload
    return function(
        ctypes.c_int(w.num_tokens),
        _lib.ptr(a.key),
        _lib.ptr(a.value),
        _lib.ptr(key_mean),
        _lib.ptr(a.output),
        ctypes.c_int(w.heads),
        ctypes.c_int(w.block),
        ctypes.c_void_p(stream),
    )


class SolPoolKernel(Kernel[SolPoolArguments, SolPoolWorkload, SolPrepareConfig]):
    name = "sol_pool"
    symbol = "nob200_sol_pool"
    planes = 2

    @classmethod
    def make_arguments(cls, workload: SolPoolWorkload) -> SolPoolArguments:
        shape = (workload.num_tokens, workload.heads, 128)
        nb = -(-workload.num_tokens // workload.block)
        return SolPoolArguments(
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, (2, workload.heads, nb, 128)),
            workload.block,
        )

    @classmethod
    def make_config(cls, workload: SolPoolWorkload) -> SolPrepareConfig:
        return SolPrepareConfig()

    @classmethod
    def make_workload(cls, arguments: SolPoolArguments) -> SolPoolWorkload:
        assert arguments.key.dtype == arguments.value.dtype == DType.BF16
        assert arguments.key.shape == arguments.value.shape
        num_tokens, heads, dim = arguments.key.shape
        assert dim == 128
        assert arguments.output.dtype == DType.BF16
        assert arguments.output.shape == (2, heads, -(-num_tokens // arguments.block), 128)
        return SolPoolWorkload(num_tokens=num_tokens, heads=heads, block=arguments.block)

    def _launch(self, function, stream: int) -> int:
        return _pool_launch(self, function, stream, None)


class SolInt8Fp8PoolKernel(Kernel[SolCenteredPoolArguments, SolPoolWorkload, SolPrepareConfig]):
    """K centroids, centred K centroids and V sums (three planes)."""

    name = "sol_int8_fp8_pool"
    symbol = "nob200_sol_pool"

    @classmethod
    def make_arguments(cls, workload: SolPoolWorkload) -> SolCenteredPoolArguments:
        shape = (workload.num_tokens, workload.heads, 128)
        nb = -(-workload.num_tokens // workload.block)
        return SolCenteredPoolArguments(
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.F32, (workload.heads, 128)),
            TensorDesc.empty(DType.BF16, (3, workload.heads, nb, 128)),
            workload.block,
        )

    @classmethod
    def make_config(cls, workload: SolPoolWorkload) -> SolPrepareConfig:
        return SolPrepareConfig()

    @classmethod
    def make_workload(cls, arguments: SolCenteredPoolArguments) -> SolPoolWorkload:
        assert arguments.key.dtype == arguments.value.dtype == DType.BF16
        assert arguments.key.shape == arguments.value.shape
        num_tokens, heads, dim = arguments.key.shape
        assert dim == 128
        assert arguments.key_mean.dtype == DType.F32
        assert arguments.key_mean.shape == (heads, 128)
        assert arguments.output.dtype == DType.BF16
        assert arguments.output.shape == (3, heads, -(-num_tokens // arguments.block), 128)
        return SolPoolWorkload(num_tokens=num_tokens, heads=heads, block=arguments.block)

    def _launch(self, function, stream: int) -> int:
        return _pool_launch(self, function, stream, self.arguments.key_mean)


class SolNvfp4PoolKernel(SolInt8Fp8PoolKernel):
    name = "sol_nvfp4_pool"


# ------------------------------------------------------------------ statistics
class SolStatsWorkload(Workload):
    num_blocks: int = Field(gt=0)
    heads: int = Field(gt=0)


@dataclasses.dataclass(frozen=True, slots=True)
class SolStatsArguments(Arguments):
    pooled: TensorDesc
    output: TensorDesc


class SolStatsKernel(Kernel[SolStatsArguments, SolStatsWorkload, SolPrepareConfig]):
    name = "sol_stats"
    symbol = "nob200_sol_stats"

    @classmethod
    def make_arguments(cls, workload: SolStatsWorkload) -> SolStatsArguments:
        return SolStatsArguments(
            TensorDesc.empty(DType.BF16, (2, workload.heads, workload.num_blocks, 128)),
            TensorDesc.empty(DType.F32, (workload.heads, 2, 128)),
        )

    @classmethod
    def make_config(cls, workload: SolStatsWorkload) -> SolPrepareConfig:
        return SolPrepareConfig(threads=128)

    @classmethod
    def make_workload(cls, arguments: SolStatsArguments) -> SolStatsWorkload:
        assert arguments.pooled.dtype == DType.BF16
        assert len(arguments.pooled.shape) == 4 and arguments.pooled.shape[0] in (2, 3)
        _, heads, num_blocks, dim = arguments.pooled.shape
        assert dim == 128
        assert arguments.output.dtype == DType.F32
        assert arguments.output.shape == (heads, 2, 128)
        return SolStatsWorkload(num_blocks=num_blocks, heads=heads)

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            _lib.ptr(a.pooled), _lib.ptr(a.output), ctypes.c_int(w.heads), ctypes.c_int(w.num_blocks), ctypes.c_void_p(stream)
        )


# -------------------------------------------------------------------- selector
class SolNvfp4SelectWorkload(Workload):
    num_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    tau: float = Field(default=1.0, allow_inf_nan=False)
    block: Literal[64, 128] = 64
    topk_fraction: float = Field(default=0.0, ge=0.0, le=1.0)

    @property
    def num_blocks(self) -> int:
        return -(-self.num_tokens // self.block)

    @property
    def topk_blocks(self) -> int:
        return min(self.num_blocks, math.ceil(self.topk_fraction * self.num_blocks)) if self.topk_fraction > 0 else 0


class SolNvfp4SelectConfig(Config):
    threads: Literal[64, 128, 256] = 256


@dataclasses.dataclass(frozen=True, slots=True)
class SolNvfp4SelectArguments(Arguments):
    query: TensorDesc
    pooled_key: TensorDesc
    stats: TensorDesc
    output: TensorDesc
    tau: float
    num_protected_blocks: int
    block: int = 64
    topk_fraction: float = 0.0
    workspace: TensorDesc | None = None

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.query.shape[0]), ("num_protected_blocks", self.num_protected_blocks))


class SolNvfp4SelectKernel(Kernel[SolNvfp4SelectArguments, SolNvfp4SelectWorkload, SolNvfp4SelectConfig]):
    name = "sol_nvfp4_select"
    symbol = "nob200_sol_select"

    @classmethod
    def workspace_bytes(cls, workload: SolNvfp4SelectWorkload) -> int:
        return workload.num_blocks**2 * workload.heads * 4 if workload.topk_fraction > 0 else 0

    @classmethod
    def make_arguments(cls, workload: SolNvfp4SelectWorkload) -> SolNvfp4SelectArguments:
        nb = workload.num_blocks
        scratch = cls.workspace_bytes(workload)
        return SolNvfp4SelectArguments(
            TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.heads, 128)),
            TensorDesc.empty(DType.BF16, (workload.heads, nb, 128)),
            TensorDesc.empty(DType.F32, (workload.heads, 2, 128)),
            TensorDesc.empty(DType.U8, (nb, workload.heads, nb)),
            workload.tau,
            nb,
            workload.block,
            workload.topk_fraction,
            TensorDesc.empty(DType.U8, (scratch,)) if scratch else None,
        )

    @classmethod
    def make_config(cls, workload: SolNvfp4SelectWorkload) -> SolNvfp4SelectConfig:
        return SolNvfp4SelectConfig(threads=256)

    @classmethod
    def make_workload(cls, arguments: SolNvfp4SelectArguments) -> SolNvfp4SelectWorkload:
        num_tokens, heads, dim = arguments.query.shape
        num_blocks = -(-num_tokens // arguments.block)
        assert arguments.query.dtype == DType.BF16 and dim == 128
        assert arguments.pooled_key.dtype == DType.BF16
        assert arguments.pooled_key.shape == (heads, num_blocks, 128)
        assert arguments.stats.dtype == DType.F32
        assert arguments.stats.shape == (heads, 2, 128)
        assert arguments.output.dtype == DType.U8
        assert arguments.output.shape == (num_blocks, heads, num_blocks)
        assert 0 <= arguments.num_protected_blocks <= num_blocks
        workload = SolNvfp4SelectWorkload(
            num_tokens=num_tokens,
            heads=heads,
            tau=arguments.tau,
            block=arguments.block,
            topk_fraction=arguments.topk_fraction,
        )
        need = cls.workspace_bytes(workload)
        if need:
            assert num_blocks <= 2048, "top-k routing supports at most 2048 blocks"
            assert arguments.workspace is not None and arguments.workspace.num_bytes >= need
        return workload

    @classmethod
    def tops(cls, arguments: SolNvfp4SelectArguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        return {MmaType.BF16BF16F32: 2 * workload.heads * 128 * workload.num_tokens * workload.num_blocks}

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.num_tokens),
            ctypes.c_int(a.num_protected_blocks),
            _lib.ptr(a.query),
            _lib.ptr(a.pooled_key),
            _lib.ptr(a.stats),
            _lib.ptr(a.output),
            ctypes.c_int(w.heads),
            ctypes.c_float(w.tau),
            ctypes.c_int(w.block),
            ctypes.c_int(w.topk_blocks),
            _lib.ptr(a.workspace),
            ctypes.c_size_t(a.workspace.num_bytes if a.workspace is not None else 0),
            ctypes.c_void_p(stream),
        )


# ------------------------------------------------------------------- attention
class SolAttentionWorkload(Workload):
    num_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    total_heads: int = Field(gt=0)
    tau: float = Field(default=1.0, allow_inf_nan=False)
    block: Literal[64, 128] = 64
    topk_fraction: float = Field(default=0.0, ge=0.0, le=1.0)

    @property
    def num_blocks(self) -> int:
        return -(-self.num_tokens // self.block)


class SolAttentionConfig(Config):
    blocks_per_group: Literal[16, 32, 64] = 32
    threads: Literal[64, 128, 256, 384] = 384


@dataclasses.dataclass(frozen=True, slots=True)
class SolAttentionArguments(Arguments):
    """Reference fields (sol_attention.py:27-44) followed by the scratch this implementation needs:
    ``mask`` u8 [blocks, heads, blocks] (written by the router, read by the attention kernel) and,
    for top-k routing, ``workspace`` for the scores."""

    query: TensorDesc
    key: TensorDesc
    value: TensorDesc
    pooled: TensorDesc
    stats: TensorDesc
    output: TensorDesc
    tau: float
    head_offset: int
    num_protected_blocks: int
    mask: TensorDesc | None = None
    block: int = 64
    topk_fraction: float = 0.0
    workspace: TensorDesc | None = None

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (
            ("num_tokens", self.query.shape[0]),
            ("head_offset", self.head_offset),
            ("num_protected_blocks", self.num_protected_blocks),
        )


class SolAttentionKernel(Kernel[SolAttentionArguments, SolAttentionWorkload, SolAttentionConfig]):
    """Router + block-sparse attention, two launches on the same stream."""

    name = "sol_attention_d128"
    symbol = "nob200_sol_attention_d128"

    @classmethod
    def workspace_bytes(cls, workload: SolAttentionWorkload) -> int:
        nb = workload.num_blocks
        scores = nb * nb * workload.heads * 4 if workload.topk_fraction > 0 else 0
        return nb * nb * workload.heads + scores

    @classmethod
    def make_arguments(cls, workload: SolAttentionWorkload) -> SolAttentionArguments:
        nb = workload.num_blocks
        shape = (workload.num_tokens, workload.heads, 128)
        return SolAttentionArguments(
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, (2, workload.heads, nb, 128)),
            TensorDesc.empty(DType.F32, (workload.heads, 2, 128)),
            TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.total_heads, 128)),
            workload.tau,
            0,
            0,
            TensorDesc.empty(DType.U8, (nb, workload.heads, nb)),
            workload.block,
            workload.topk_fraction,
            TensorDesc.empty(DType.U8, (nb * nb * workload.heads * 4,)) if workload.topk_fraction > 0 else None,
        )

    @classmethod
    def make_config(cls, workload: SolAttentionWorkload) -> SolAttentionConfig:
        return SolAttentionConfig()

    @classmethod
    def make_workload(cls, arguments: SolAttentionArguments) -> SolAttentionWorkload:
        num_tokens, heads, dim = arguments.query.shape
        assert dim == 128
        assert arguments.query.dtype == arguments.key.dtype == arguments.value.dtype == DType.BF16
        assert arguments.query.shape == arguments.key.shape == arguments.value.shape
        num_blocks = -(-num_tokens // arguments.block)
        assert arguments.pooled.dtype == DType.BF16
        assert arguments.pooled.shape in ((2, heads, num_blocks, 128), (3, heads, num_blocks, 128))
        assert arguments.stats.dtype == DType.F32 and arguments.stats.shape == (heads, 2, 128)
        assert arguments.output.dtype == DType.BF16 and len(arguments.output.shape) == 3
        assert arguments.output.shape[0] == num_tokens and arguments.output.shape[2] == 128
        total_heads = arguments.output.shape[1]
        assert 0 <= arguments.head_offset <= total_heads - heads
        assert 0 <= arguments.num_protected_blocks <= num_blocks
        assert arguments.mask is not None, "sol attention needs the routing mask as op scratch"
        assert arguments.mask.dtype == DType.U8 and arguments.mask.shape == (num_blocks, heads, num_blocks)
        if arguments.topk_fraction > 0:
            assert arguments.workspace is not None
            assert arguments.workspace.num_bytes >= num_blocks * num_blocks * heads * 4
        return SolAttentionWorkload(
            num_tokens=num_tokens,
            heads=heads,
            total_heads=total_heads,
            tau=arguments.tau,
            block=arguments.block,
            topk_fraction=arguments.topk_fraction,
        )

    @classmethod
    def tops(cls, arguments: SolAttentionArguments) -> dict[MmaType, int]:
        """Expected operations of threshold routing (sol_attention.py:281-298)."""
        workload = cls.make_workload(arguments)
        block, tokens = workload.block, workload.num_tokens
        nb = workload.num_blocks
        protected = min(arguments.num_protected_blocks, nb)
        lengths = tuple(min(block, tokens - b * block) for b in range(nb))
        mandatory = tokens * sum(lengths[:protected])
        for qb, qlen in enumerate(lengths):
            for kb in range(max(protected, qb - 1), min(nb, qb + 2)):
                mandatory += qlen * lengths[kb]
        probability = (
            workload.topk_fraction if workload.topk_fraction > 0 else 0.5 * math.erfc(workload.tau / math.sqrt(2))
        )
        exact_pairs = mandatory + probability * (tokens**2 - mandatory)
        return {MmaType.BF16BF16F32: round(4 * workload.heads * 128 * (exact_pairs + tokens * nb))}

    def compile(self) -> None:
        if self.compiled is None:
            self.compiled = (_lib.symbol("nob200_sol_select"), _lib.symbol(type(self).symbol))

    def _launch(self, function, stream: int) -> int:
        select, attend = function
        a, w = self.arguments, self.workload
        topk_blocks = min(w.num_blocks, math.ceil(w.topk_fraction * w.num_blocks)) if w.topk_fraction > 0 else 0
        code = select(
            ctypes.c_int(w.num_tokens),
            ctypes.c_int(a.num_protected_blocks),
            _lib.ptr(a.query),
            _lib.ptr(a.pooled),  # plane 0 = key block means, contiguous [heads, blocks, 128]
            _lib.ptr(a.stats),
            _lib.ptr(a.mask),
            ctypes.c_int(w.heads),
            ctypes.c_float(w.tau),
            ctypes.c_int(w.block),
            ctypes.c_int(topk_blocks),
            _lib.ptr(a.workspace),
            ctypes.c_size_t(a.workspace.num_bytes if a.workspace is not None else 0),
            ctypes.c_void_p(stream),
        )
        if code:
            return code
        return attend(
            ctypes.c_int(w.num_tokens),
            ctypes.c_int(a.head_offset),
            _lib.ptr(a.query),
            _lib.ptr(a.key),
            _lib.ptr(a.value),
            _lib.ptr(a.pooled),
            _lib.ptr(a.mask),
            _lib.ptr(a.output),
            ctypes.c_int(w.heads),
            ctypes.c_int(w.total_heads),
            ctypes.c_int(w.block),
            ctypes.c_int(a.pooled.shape[0]),
            ctypes.c_void_p(stream),
        )
