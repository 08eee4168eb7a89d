"""INT8 and BF16 GEMMs with the fused epilogue and the row-wise int8 activation quantisers of the projections.

INT8 GEMM: bound to ``nob200_matmul_int8``.

Interface of reference ``MatmulInt8Kernel`` (src/nano_omni/kernels/matmul/matmul_int8.py:13-240): same Workload
and Arguments fields and order, validation and ``tops``.  The Config keeps the reference's tile fields so stored
configs still validate; the sm_100a kernel has one tile shape (128 x 256 x 128).
"""

from __future__ import annotations

import ctypes
import dataclasses
from typing import Literal

from pydantic import Field

from nano_omni_b200 import _lib
from nano_omni_b200.core import Arguments, Config, DType, Kernel, MmaType, TensorDesc, Workload


class MatmulInt8Workload(Workload):
    num_tokens: int = Field(gt=0)
    n: int = Field(gt=0)
    k: int = Field(gt=0)
    use_bias: bool = False
    use_residual: bool = False
    use_multiply: bool = False
    use_silu: bool = False


class MatmulInt8Config(Config):
    block_m: int = 128
    block_n: int = 256
    block_k: int = 128
    stages: int = 4
    threads: int = 320
    warp_policy: Literal["full_row", "full_col", "square"] = "full_row"
    warp_specialization: bool = True
    swizzle: int = 0


@dataclasses.dataclass(frozen=True, slots=True)
class MatmulInt8Arguments(Arguments):
    input: TensorDesc
    weight: TensorDesc
    bias: TensorDesc | None
    residual: TensorDesc | None
    multiply: TensorDesc | None
    output: TensorDesc
    weight_scale: TensorDesc
    input_scale: TensorDesc
    use_silu: bool

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.input.shape[0]),)


class MatmulInt8Kernel(Kernel[MatmulInt8Arguments, MatmulInt8Workload, MatmulInt8Config]):
    name = "matmul_int8"
    symbol = "nob200_matmul_int8"

    @classmethod
    def make_arguments(cls, workload: MatmulInt8Workload) -> MatmulInt8Arguments:
        wide = (workload.num_tokens, workload.n)
        return MatmulInt8Arguments(
            TensorDesc.empty(DType.I8, (workload.num_tokens, workload.k)),
            TensorDesc.empty(DType.I8, (workload.n, workload.k)),
            TensorDesc.empty(DType.BF16, (workload.n,)) if workload.use_bias else None,
            TensorDesc.empty(DType.BF16, wide) if workload.use_residual else None,
            TensorDesc.empty(DType.BF16, wide) if workload.use_multiply else None,
            TensorDesc.empty(DType.BF16, wide),
            TensorDesc.empty(DType.F32, (workload.n, 1)),
            TensorDesc.empty(DType.F32, (workload.num_tokens,)),
            workload.use_silu,
        )

    @classmethod
    def make_config(cls, workload: MatmulInt8Workload) -> MatmulInt8Config:
        return MatmulInt8Config()

    @classmethod
    def make_workload(cls, arguments: MatmulInt8Arguments) -> MatmulInt8Workload:
        input, weight = arguments.input, arguments.weight
        assert len(input.shape) == len(weight.shape) == 2
        num_tokens, k = input.shape
        n, weight_k = weight.shape
        assert weight_k == k
        assert input.dtype == weight.dtype == DType.I8
        assert arguments.output.dtype == DType.BF16 and arguments.output.shape == (num_tokens, n)
        assert arguments.weight_scale.dtype == DType.F32 and arguments.weight_scale.shape == (n, 1)
        assert arguments.input_scale.dtype == DType.F32 and arguments.input_scale.shape == (num_tokens,)
        if arguments.bias is not None:
            assert arguments.bias.dtype == DType.BF16 and arguments.bias.shape == (n,)
        for operand in (arguments.residual, arguments.multiply):
            if operand is not None:
                assert operand.dtype == DType.BF16 and operand.shape == (num_tokens, n)
        assert k % 16 == 0 and n % 8 == 0, "k must be a multiple of 16 and n of 8"
        return MatmulInt8Workload(
            num_tokens=num_tokens,
            n=n,
            k=k,
            use_bias=arguments.bias is not None,
            use_residual=arguments.residual is not None,
            use_multiply=arguments.multiply is not None,
            use_silu=arguments.use_silu,
        )

    @classmethod
    def tops(cls, arguments: MatmulInt8Arguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        return {MmaType.I8I8I32: 2 * workload.num_tokens * workload.n * workload.k}

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.num_tokens), _lib.ptr(a.input), _lib.ptr(a.weight), _lib.ptr(a.bias), _lib.ptr(a.residual),
            _lib.ptr(a.multiply), _lib.ptr(a.output), _lib.ptr(a.weight_scale), _lib.ptr(a.input_scale),
            ctypes.c_int(w.n), ctypes.c_int(w.k), ctypes.c_int(int(a.use_silu)), ctypes.c_void_p(stream),
        )  # fmt: skip


# ------------------------------------------------------------------ bf16 GEMM (bf16 projections, LoRA products)
class MatmulBf16Workload(Workload):
    num_tokens: int = Field(gt=0)
    n: int = Field(gt=0)
    k: int = Field(gt=0)
    use_bias: bool = False
    use_residual: bool = False
    use_multiply: bool = False
    use_silu: bool = False
    output_scale: float = Field(default=1.0, allow_inf_nan=False)


@dataclasses.dataclass(frozen=True, slots=True)
class MatmulBf16Arguments(Arguments):
    input: TensorDesc
    weight: TensorDesc
    bias: TensorDesc | None
    residual: TensorDesc | None
    multiply: TensorDesc | None
    output: TensorDesc
    output_scale: float | int
    use_silu: bool

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.input.shape[0]),)


class MatmulBf16Kernel(Kernel[MatmulBf16Arguments, MatmulBf16Workload, MatmulInt8Config]):
    """src/nano_omni/kernels/matmul/matmul_bf16.py:15-207: scale, bias, residual, SiLU, multiply in that order."""

    name = "matmul_bf16"
    symbol = "nob200_matmul_bf16"

    @classmethod
    def make_arguments(cls, workload: MatmulBf16Workload) -> MatmulBf16Arguments:
        wide = (workload.num_tokens, workload.n)
        return MatmulBf16Arguments(
            TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.k)),
            TensorDesc.empty(DType.BF16, (workload.n, workload.k)),
            TensorDesc.empty(DType.BF16, (workload.n,)) if workload.use_bias else None,
            TensorDesc.empty(DType.BF16, wide) if workload.use_residual else None,
            TensorDesc.empty(DType.BF16, wide) if workload.use_multiply else None,
            TensorDesc.empty(DType.BF16, wide),
            workload.output_scale,
            workload.use_silu,
        )

    @classmethod
    def make_config(cls, workload: MatmulBf16Workload) -> MatmulInt8Config:
        return MatmulInt8Config(block_k=64)

    @classmethod
    def make_workload(cls, arguments: MatmulBf16Arguments) -> MatmulBf16Workload:
        input, weight = arguments.input, arguments.weight
        assert len(input.shape) == len(weight.shape) == 2
        num_tokens, k = input.shape
        n, weight_k = weight.shape
        assert weight_k == k
        assert input.dtype == weight.dtype == DType.BF16
        assert arguments.output.dtype == DType.BF16 and arguments.output.shape == (num_tokens, n)
        if arguments.bias is not None:
            assert arguments.bias.dtype == DType.BF16 and arguments.bias.shape == (n,)
        for operand in (arguments.residual, arguments.multiply):
            if operand is not None:
                assert operand.dtype == DType.BF16 and operand.shape == (num_tokens, n)
        assert k % 8 == 0 and n % 8 == 0, "k and n must be multiples of 8"
        return MatmulBf16Workload(
            num_tokens=num_tokens,
            n=n,
            k=k,
            use_bias=arguments.bias is not None,
            use_residual=arguments.residual is not None,
            use_multiply=arguments.multiply is not None,
            use_silu=arguments.use_silu,
            output_scale=float(arguments.output_scale),
        )

    @classmethod
    def tops(cls, arguments: MatmulBf16Arguments) -> dict[MmaType, int]:
        workload = cls.make_workload(arguments)
        return {MmaType.BF16BF16F32: 2 * workload.num_tokens * workload.n * workload.k}

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.num_tokens), _lib.ptr(a.input), _lib.ptr(a.weight), _lib.ptr(a.bias), _lib.ptr(a.residual),
            _lib.ptr(a.multiply), _lib.ptr(a.output), ctypes.c_float(w.output_scale), ctypes.c_int(w.n),
            ctypes.c_int(w.k), ctypes.c_int(int(a.use_silu)), ctypes.c_void_p(stream),
        )  # fmt: skip


# ------------------------------------------------------------------ row-wise int8 activations
class Int8RowwiseWorkload(Workload):
    num_tokens: int = Field(gt=0)
    columns: int = Field(gt=0)


class ConvRotInt8Workload(Workload):
    num_tokens: int = Field(gt=0)
    columns: int = Field(gt=0)
    group: int = 256


class RowwiseConfig(Config):
    threads: Literal[128, 256, 512] = 128


@dataclasses.dataclass(frozen=True, slots=True)
class Int8RowwiseArguments(Arguments):
    input: TensorDesc
    output: TensorDesc
    scales: TensorDesc

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.input.shape[0]),)


@dataclasses.dataclass(frozen=True, slots=True)
class ConvRotInt8Arguments(Arguments):
    input: TensorDesc
    output: TensorDesc
    scales: TensorDesc
    group: int = 256

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.input.shape[0]),)


def _check_rowwise(arguments) -> tuple[int, int]:
    assert len(arguments.input.shape) == 2
    num_tokens, columns = arguments.input.shape
    assert arguments.input.dtype == DType.BF16
    assert arguments.output.dtype == DType.I8 and arguments.output.shape == (num_tokens, columns)
    assert arguments.scales.dtype == DType.F32 and arguments.scales.shape == (num_tokens,)
    assert columns % 8 == 0, "columns must be a multiple of 8"
    return num_tokens, columns


def _launch_rowwise(kernel, function, group: int, stream: int) -> int:
    a, w = kernel.arguments, kernel.workload
    return function(
        ctypes.c_int(w.num_tokens), _lib.ptr(a.input), _lib.ptr(a.output), _lib.ptr(a.scales), ctypes.c_int(w.columns),
        ctypes.c_int(group), ctypes.c_void_p(stream),
    )  # fmt: skip


class Int8RowwiseKernel(Kernel[Int8RowwiseArguments, Int8RowwiseWorkload, RowwiseConfig]):
    """src/nano_omni/kernels/quantization/int8_rowwise.py:18-116."""

    name = "int8_rowwise"
    symbol = "nob200_int8_rowwise"

    @classmethod
    def make_arguments(cls, workload: Int8RowwiseWorkload) -> Int8RowwiseArguments:
        shape = (workload.num_tokens, workload.columns)
        return Int8RowwiseArguments(
            TensorDesc.empty(DType.BF16, shape), TensorDesc.empty(DType.I8, shape),
            TensorDesc.empty(DType.F32, (workload.num_tokens,)),
        )  # fmt: skip

    @classmethod
    def make_config(cls, workload: Int8RowwiseWorkload) -> RowwiseConfig:
        return RowwiseConfig()

    @classmethod
    def make_workload(cls, arguments: Int8RowwiseArguments) -> Int8RowwiseWorkload:
        num_tokens, columns = _check_rowwise(arguments)
        return Int8RowwiseWorkload(num_tokens=num_tokens, columns=columns)

    def _launch(self, function, stream: int) -> int:
        return _launch_rowwise(self, function, 0, stream)


class ConvRotInt8Kernel(Kernel[ConvRotInt8Arguments, ConvRotInt8Workload, RowwiseConfig]):
    """src/nano_omni/kernels/quantization/convrot_int8.py:22-161; groups of 256 columns only."""

    name = "convrot_int8"
    symbol = "nob200_int8_rowwise"

    @classmethod
    def make_arguments(cls, workload: ConvRotInt8Workload) -> ConvRotInt8Arguments:
        shape = (workload.num_tokens, workload.columns)
        return ConvRotInt8Arguments(
            TensorDesc.empty(DType.BF16, shape), TensorDesc.empty(DType.I8, shape),
            TensorDesc.empty(DType.F32, (workload.num_tokens,)), workload.group,
        )  # fmt: skip

    @classmethod
    def make_config(cls, workload: ConvRotInt8Workload) -> RowwiseConfig:
        return RowwiseConfig()

    @classmethod
    def make_workload(cls, arguments: ConvRotInt8Arguments) -> ConvRotInt8Workload:
        num_tokens, columns = _check_rowwise(arguments)
        group = arguments.group
        assert group >= 4 and not group & (group - 1) and not (group.bit_length() - 1) % 2 and not columns % group, (
            "ConvRot requires a power-of-four group dividing columns"
        )
        assert group == 256, "this implementation rotates groups of 256 columns"
        return ConvRotInt8Workload(num_tokens=num_tokens, columns=columns, group=group)

    def _launch(self, function, stream: int) -> int:
        return _launch_rowwise(self, function, self.workload.group, stream)
