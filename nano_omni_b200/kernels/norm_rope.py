"""Per-head RMS norm + split-half RoPE, alone and fused into the int8 query quantiser.

Interfaces of the reference classes with the same ``name``:

* ``h3_head_norm_rope``  src/nano_omni/kernels/specialized/h3_head_norm_rope.py:14-162
* ``h3_query_prepare``   src/nano_omni/kernels/specialized/h3_query_prepare.py:16-184
* ``h3_qk_norm_rope``    src/nano_omni/kernels/specialized/h3_qk_norm_rope.py:17-178 (Q and K in place, one launch)

These run immediately before every attention path (ops/minimax_h3/attention.py:51-97).
"""

from __future__ import annotations

import ctypes
import dataclasses
from typing import Literal

from nano_omni_b200 import _lib
from nano_omni_b200.core import Arguments, Config, DType, Kernel, TensorDesc, Workload


def _check_rotation(cosines: TensorDesc | None, sines: TensorDesc | None, tokens: int) -> None:
    assert (cosines is None) == (sines is None)
    if cosines is not None and sines is not None:
        assert cosines.dtype == sines.dtype == DType.F32
        assert cosines.shape == sines.shape == (tokens, 48)


class H3HeadNormRopeWorkload(Workload):
    tokens: int
    heads: int
    use_rope: bool


class H3HeadNormRopeConfig(Config):
    threads: Literal[128, 256] = 256


@dataclasses.dataclass(frozen=True, slots=True)
class H3HeadNormRopeArguments(Arguments):
    input: TensorDesc
    weight: TensorDesc
    cosines: TensorDesc | None
    sines: TensorDesc | None
    output: TensorDesc

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("tokens", self.input.shape[0]),)


class H3HeadNormRopeKernel(Kernel[H3HeadNormRopeArguments, H3HeadNormRopeWorkload, H3HeadNormRopeConfig]):
    name = "h3_head_norm_rope"
    symbol = "nob200_h3_head_norm_rope"

    @classmethod
    def make_arguments(cls, workload: H3HeadNormRopeWorkload) -> H3HeadNormRopeArguments:
        shape = (workload.tokens, workload.heads, 128)
        plane = TensorDesc.empty(DType.F32, (workload.tokens, 48)) if workload.use_rope else None
        return H3HeadNormRopeArguments(
            TensorDesc.empty(DType.BF16, shape), TensorDesc.empty(DType.BF16, (128,)), plane, plane,
            TensorDesc.empty(DType.BF16, shape),
        )  # fmt: skip

    @classmethod
    def make_config(cls, workload: H3HeadNormRopeWorkload) -> H3HeadNormRopeConfig:
        return H3HeadNormRopeConfig()

    @classmethod
    def make_workload(cls, arguments: H3HeadNormRopeArguments) -> H3HeadNormRopeWorkload:
        assert arguments.input.dtype == arguments.output.dtype == DType.BF16
        assert arguments.input.shape == arguments.output.shape
        assert len(arguments.input.shape) == 3 and arguments.input.shape[2] == 128
        assert arguments.weight.dtype == DType.BF16 and arguments.weight.shape == (128,)
        _check_rotation(arguments.cosines, arguments.sines, arguments.input.shape[0])
        return H3HeadNormRopeWorkload(
            tokens=arguments.input.shape[0], heads=arguments.input.shape[1], use_rope=arguments.cosines is not None
        )

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.tokens), _lib.ptr(a.input), _lib.ptr(a.weight), _lib.ptr(a.cosines), _lib.ptr(a.sines),
            _lib.ptr(a.output), ctypes.c_int(w.heads), ctypes.c_void_p(stream),
        )  # fmt: skip


class H3QueryPrepareWorkload(Workload):
    tokens: int
    heads: int
    use_rope: bool


class H3QueryPrepareConfig(Config):
    threads: Literal[128] = 128


@dataclasses.dataclass(frozen=True, slots=True)
class H3QueryPrepareArguments(Arguments):
    source: TensorDesc
    weight: TensorDesc
    cosines: TensorDesc | None
    sines: TensorDesc | None
    quantized: TensorDesc
    scales: TensorDesc

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("tokens", self.source.shape[0]),)


class H3QueryPrepareKernel(Kernel[H3QueryPrepareArguments, H3QueryPrepareWorkload, H3QueryPrepareConfig]):
    name = "h3_query_prepare"
    symbol = "nob200_h3_query_prepare"

    @classmethod
    def make_arguments(cls, workload: H3QueryPrepareWorkload) -> H3QueryPrepareArguments:
        rows = -(-workload.tokens // 32) * 32
        plane = TensorDesc.empty(DType.F32, (workload.tokens, 48)) if workload.use_rope else None
        return H3QueryPrepareArguments(
            TensorDesc.empty(DType.BF16, (workload.tokens, workload.heads * 128)),
            TensorDesc.empty(DType.BF16, (128,)),
            plane,
            plane,
            TensorDesc.empty(DType.I8, (workload.heads, rows, 128)),
            TensorDesc.empty(DType.F32, (workload.heads, rows // 32)),
        )

    @classmethod
    def make_config(cls, workload: H3QueryPrepareWorkload) -> H3QueryPrepareConfig:
        return H3QueryPrepareConfig()

    @classmethod
    def make_workload(cls, arguments: H3QueryPrepareArguments) -> H3QueryPrepareWorkload:
        assert len(arguments.source.shape) == 2
        tokens, columns = arguments.source.shape
        assert not columns % 128
        heads = columns // 128
        assert arguments.source.dtype == arguments.weight.dtype == DType.BF16
        assert arguments.weight.shape == (128,)
        _check_rotation(arguments.cosines, arguments.sines, tokens)
        rows = -(-tokens // 32) * 32
        assert arguments.quantized.dtype == DType.I8 and arguments.quantized.shape == (heads, rows, 128)
        assert arguments.scales.dtype == DType.F32 and arguments.scales.shape == (heads, rows // 32)
        return H3QueryPrepareWorkload(tokens=tokens, heads=heads, use_rope=arguments.cosines is not None)

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.tokens), _lib.ptr(a.source), _lib.ptr(a.weight), _lib.ptr(a.cosines), _lib.ptr(a.sines),
            _lib.ptr(a.quantized), _lib.ptr(a.scales), ctypes.c_int(w.heads), ctypes.c_void_p(stream),
        )  # fmt: skip


@dataclasses.dataclass(frozen=True, slots=True)
class H3QkNormRopeArguments(Arguments):
    query: TensorDesc
    key: TensorDesc
    query_weight: TensorDesc
    key_weight: TensorDesc
    cosines: TensorDesc
    sines: TensorDesc

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("tokens", self.query.shape[0]),)


class H3QkNormRopeKernel(Kernel[H3QkNormRopeArguments, H3HeadNormRopeWorkload, H3HeadNormRopeConfig]):
    name = "h3_qk_norm_rope"
    symbol = "nob200_h3_qk_norm_rope"

    @classmethod
    def make_arguments(cls, workload: H3HeadNormRopeWorkload) -> H3QkNormRopeArguments:
        assert workload.use_rope
        shape = (workload.tokens, workload.heads, 128)
        return H3QkNormRopeArguments(
            TensorDesc.empty(DType.BF16, shape), TensorDesc.empty(DType.BF16, shape),
            TensorDesc.empty(DType.BF16, (128,)), TensorDesc.empty(DType.BF16, (128,)),
            TensorDesc.empty(DType.F32, (workload.tokens, 48)), TensorDesc.empty(DType.F32, (workload.tokens, 48)),
        )  # fmt: skip

    @classmethod
    def make_config(cls, workload: H3HeadNormRopeWorkload) -> H3HeadNormRopeConfig:
        return H3HeadNormRopeConfig()

    @classmethod
    def make_workload(cls, arguments: H3QkNormRopeArguments) -> H3HeadNormRopeWorkload:
        assert arguments.query.dtype == arguments.key.dtype == DType.BF16
        assert arguments.query.shape == arguments.key.shape
        assert len(arguments.query.shape) == 3 and arguments.query.shape[2] == 128
        assert arguments.query_weight.dtype == arguments.key_weight.dtype == DType.BF16
        assert arguments.query_weight.shape == arguments.key_weight.shape == (128,)
        assert arguments.cosines.dtype == arguments.sines.dtype == DType.F32
        assert arguments.cosines.shape == arguments.sines.shape == (arguments.query.shape[0], 48)
        return H3HeadNormRopeWorkload(tokens=arguments.query.shape[0], heads=arguments.query.shape[1], use_rope=True)

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.tokens), _lib.ptr(a.query), _lib.ptr(a.key), _lib.ptr(a.query_weight), _lib.ptr(a.key_weight),
            _lib.ptr(a.cosines), _lib.ptr(a.sines), ctypes.c_int(w.heads), ctypes.c_void_p(stream),
        )  # fmt: skip
