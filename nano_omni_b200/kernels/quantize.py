"""Quantiser and statistics kernels of the int8-fp8 and nvfp4 attention paths.

Each class keeps the interface of the reference class with the same ``name``:

* ``token_group_mean``        src/nano_omni/kernels/normalization/token_group_mean.py:13-189
* ``int8_fp8_quantize_qk``    src/nano_omni/kernels/attention/int8_fp8/quantize_qk.py:71-201
* ``int8_fp8_value_scale``    src/nano_omni/kernels/attention/int8_fp8/value_scale.py:58-123
* ``int8_fp8_quantize_value`` src/nano_omni/kernels/attention/int8_fp8/quantize_value.py:68-152
* ``nvfp4_prepare``           src/nano_omni/kernels/attention/nvfp4_prepare.py:11-168

Additions that have no counterpart in the reference are trailing, defaulted
fields: ``hadamard`` (rotate each head's 128 channels by a normalised
Walsh-Hadamard transform before quantising), ``global_scale`` (per-tensor NVFP4
scale) and ``workspace`` (caller-reserved scratch for the column mean).
"""

from __future__ import annotations

import ctypes
import dataclasses
from typing import Literal

from pydantic import Field

from nano_omni_b200 import _lib
from nano_omni_b200.core import Arguments, Config, DType, Kernel, TensorDesc, Workload

_c_int = ctypes.c_int


class Int8Fp8ThreadConfig(Config):
    threads: Literal[64, 128, 256] = 128


# ------------------------------------------------------------ token_group_mean
class TokenGroupMeanWorkload(Workload):
    num_tokens: int = Field(gt=0)
    columns: int = Field(gt=0)
    tokens_per_block: int = Field(gt=0)
    include_padding: bool = False


class TokenGroupMeanConfig(Config):
    tile_columns: int = Field(gt=0)
    threads: int = Field(gt=0)


@dataclasses.dataclass(frozen=True, slots=True)
class TokenGroupMeanArguments(Arguments):
    input: TensorDesc
    output: TensorDesc
    tokens_per_block: int
    include_padding: bool
    workspace: TensorDesc | None = None

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.input.shape[0]), ("tokens_per_block", self.tokens_per_block))


class TokenGroupMeanKernel(Kernel[TokenGroupMeanArguments, TokenGroupMeanWorkload, TokenGroupMeanConfig]):
    name = "token_group_mean"
    symbol = "nob200_token_group_mean"

    @classmethod
    def workspace_bytes(cls, workload: TokenGroupMeanWorkload) -> int:
        chunks = -(-workload.tokens_per_block // 128)
        if chunks <= 1:
            return 0
        groups = -(-workload.num_tokens // workload.tokens_per_block)
        return groups * chunks * workload.columns * 4

    @classmethod
    def make_arguments(cls, workload: TokenGroupMeanWorkload) -> TokenGroupMeanArguments:
        num_blocks = -(-workload.num_tokens // workload.tokens_per_block)
        scratch = cls.workspace_bytes(workload)
        return TokenGroupMeanArguments(
            input=TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.columns)),
            output=TensorDesc.empty(DType.F32, (num_blocks, workload.columns)),
            tokens_per_block=workload.tokens_per_block,
            include_padding=workload.include_padding,
            workspace=TensorDesc.empty(DType.U8, (scratch,)) if scratch else None,
        )

    @classmethod
    def make_workload(cls, arguments: TokenGroupMeanArguments) -> TokenGroupMeanWorkload:
        assert len(arguments.input.shape) == 2
        num_tokens, columns = arguments.input.shape
        assert arguments.tokens_per_block > 0
        num_blocks = -(-num_tokens // arguments.tokens_per_block)
        assert arguments.input.dtype == DType.BF16
        assert arguments.output.dtype == DType.F32
        assert arguments.output.shape == (num_blocks, columns)
        workload = TokenGroupMeanWorkload(
            num_tokens=num_tokens,
            columns=columns,
            tokens_per_block=arguments.tokens_per_block,
            include_padding=arguments.include_padding,
        )
        need = cls.workspace_bytes(workload)
        if need:
            assert arguments.workspace is not None, "token_group_mean needs a workspace for groups over 128 tokens"
            assert arguments.workspace.num_bytes >= need
        return workload

    @classmethod
    def make_config(cls, workload: TokenGroupMeanWorkload) -> TokenGroupMeanConfig:
        return TokenGroupMeanConfig(threads=128, tile_columns=512)

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            _c_int(w.num_tokens),
            _lib.ptr(a.input),
            _lib.ptr(a.output),
            _c_int(w.columns),
            _c_int(w.tokens_per_block),
            _c_int(int(w.include_padding)),
            _lib.ptr(a.workspace),
            ctypes.c_size_t(a.workspace.num_bytes if a.workspace is not None else 0),
            ctypes.c_void_p(stream),
        )


# -------------------------------------------------------- int8_fp8_quantize_qk
class Int8Fp8QkWorkload(Workload):
    num_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    tokens_per_block: int = Field(default=32, gt=0)
    center: bool = False
    hadamard: bool = False

    @property
    def num_padded_tokens(self) -> int:
        return -(-self.num_tokens // self.tokens_per_block) * self.tokens_per_block

    @property
    def packed_bytes(self) -> int:
        return self.heads * self.num_padded_tokens * 128

    @property
    def storage_bytes(self) -> int:
        return self.packed_bytes + self.heads * (self.num_padded_tokens // self.tokens_per_block) * 4


@dataclasses.dataclass(frozen=True, slots=True)
class Int8Fp8QuantizeQKArguments(Arguments):
    source: TensorDesc
    statistics: TensorDesc
    quantized: TensorDesc
    scales: TensorDesc
    heads: int
    tokens_per_block: int = 32
    center: bool = False
    hadamard: bool = False

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.source.shape[0]),)


class Int8Fp8QuantizeQKKernel(Kernel[Int8Fp8QuantizeQKArguments, Int8Fp8QkWorkload, Int8Fp8ThreadConfig]):
    name = "int8_fp8_quantize_qk"
    symbol = "nob200_int8_fp8_quantize_qk"

    @classmethod
    def make_arguments(cls, workload: Int8Fp8QkWorkload) -> Int8Fp8QuantizeQKArguments:
        return Int8Fp8QuantizeQKArguments(
            source=TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.heads * 128)),
            statistics=TensorDesc.empty(DType.F32, (1, workload.heads * 128)),
            quantized=TensorDesc.empty(DType.I8, (workload.heads, workload.num_padded_tokens, 128)),
            scales=TensorDesc.empty(
                DType.F32, (workload.heads, workload.num_padded_tokens // workload.tokens_per_block)
            ),
            heads=workload.heads,
            tokens_per_block=workload.tokens_per_block,
            center=workload.center,
            hadamard=workload.hadamard,
        )

    @classmethod
    def make_config(cls, workload: Int8Fp8QkWorkload) -> Int8Fp8ThreadConfig:
        return Int8Fp8ThreadConfig(threads=128 if workload.tokens_per_block == 32 else 256)

    @classmethod
    def make_workload(cls, arguments: Int8Fp8QuantizeQKArguments) -> Int8Fp8QkWorkload:
        assert len(arguments.source.shape) == 2
        num_tokens, columns = arguments.source.shape
        assert columns == arguments.heads * 128
        assert arguments.tokens_per_block in (32, 64, 128)
        assert arguments.source.dtype == DType.BF16
        assert arguments.statistics.dtype == DType.F32
        assert arguments.statistics.shape == (1, columns)
        padded = -(-num_tokens // arguments.tokens_per_block) * arguments.tokens_per_block
        assert arguments.quantized.dtype == DType.I8
        assert arguments.quantized.shape == (arguments.heads, padded, 128)
        assert arguments.scales.dtype == DType.F32
        assert arguments.scales.shape == (arguments.heads, padded // arguments.tokens_per_block)
        return Int8Fp8QkWorkload(
            num_tokens=num_tokens,
            heads=arguments.heads,
            tokens_per_block=arguments.tokens_per_block,
            center=arguments.center,
            hadamard=arguments.hadamard,
        )

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            _c_int(w.num_tokens),
            _lib.ptr(a.source),
            _lib.ptr(a.statistics),
            _lib.ptr(a.quantized),
            _lib.ptr(a.scales),
            _c_int(w.heads),
            _c_int(w.tokens_per_block),
            _c_int(int(w.center)),
            _c_int(int(w.hadamard)),
            ctypes.c_void_p(stream),
        )


# ------------------------------------------------ int8_fp8_value_scale / value
class Int8Fp8ValueWorkload(Workload):
    num_tokens: int = Field(gt=0)
    heads: int = Field(gt=0)


@dataclasses.dataclass(frozen=True, slots=True)
class Int8Fp8ValueScaleArguments(Arguments):
    source: TensorDesc
    output: TensorDesc
    heads: int

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.source.shape[0]),)


class Int8Fp8ValueScaleKernel(Kernel[Int8Fp8ValueScaleArguments, Int8Fp8ValueWorkload, Int8Fp8ThreadConfig]):
    name = "int8_fp8_value_scale"
    symbol = "nob200_int8_fp8_value_scale"

    @classmethod
    def make_arguments(cls, workload: Int8Fp8ValueWorkload) -> Int8Fp8ValueScaleArguments:
        return Int8Fp8ValueScaleArguments(
            source=TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.heads * 128)),
            output=TensorDesc.empty(DType.F32, (workload.heads, 128)),
            heads=workload.heads,
        )

    @classmethod
    def make_config(cls, workload: Int8Fp8ValueWorkload) -> Int8Fp8ThreadConfig:
        return Int8Fp8ThreadConfig(threads=256)

    @classmethod
    def make_workload(cls, arguments: Int8Fp8ValueScaleArguments) -> Int8Fp8ValueWorkload:
        assert len(arguments.source.shape) == 2
        num_tokens, columns = arguments.source.shape
        assert columns == arguments.heads * 128
        assert arguments.source.dtype == DType.BF16
        assert arguments.output.dtype == DType.F32
        assert arguments.output.shape == (arguments.heads, 128)
        return Int8Fp8ValueWorkload(num_tokens=num_tokens, heads=arguments.heads)

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            _c_int(w.num_tokens), _lib.ptr(a.source), _lib.ptr(a.output), _c_int(w.heads), ctypes.c_void_p(stream)
        )


@dataclasses.dataclass(frozen=True, slots=True)
class Int8Fp8QuantizeValueArguments(Arguments):
    source: TensorDesc
    scale: TensorDesc
    output: TensorDesc
    heads: int

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.source.shape[0]),)


class Int8Fp8QuantizeValueKernel(Kernel[Int8Fp8QuantizeValueArguments, Int8Fp8ValueWorkload, Int8Fp8ThreadConfig]):
    name = "int8_fp8_quantize_value"
    symbol = "nob200_int8_fp8_quantize_value"

    @classmethod
    def make_arguments(cls, workload: Int8Fp8ValueWorkload) -> Int8Fp8QuantizeValueArguments:
        padded = -(-workload.num_tokens // 64) * 64
        return Int8Fp8QuantizeValueArguments(
            source=TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.heads * 128)),
            scale=TensorDesc.empty(DType.F32, (workload.heads, 128)),
            output=TensorDesc.empty(DType.FP8_E4M3, (workload.heads, 128, padded)),
            heads=workload.heads,
        )

    @classmethod
    def make_config(cls, workload: Int8Fp8ValueWorkload) -> Int8Fp8ThreadConfig:
        return Int8Fp8ThreadConfig(threads=256)

    @classmethod
    def make_workload(cls, arguments: Int8Fp8QuantizeValueArguments) -> Int8Fp8ValueWorkload:
        assert len(arguments.source.shape) == 2
        num_tokens, columns = arguments.source.shape
        assert columns == arguments.heads * 128
        assert arguments.source.dtype == DType.BF16
        assert arguments.scale.dtype == DType.F32
        assert arguments.scale.shape == (arguments.heads, 128)
        assert arguments.output.dtype == DType.FP8_E4M3
        assert arguments.output.shape == (arguments.heads, 128, -(-num_tokens // 64) * 64)
        return Int8Fp8ValueWorkload(num_tokens=num_tokens, heads=arguments.heads)

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            _c_int(w.num_tokens),
            _lib.ptr(a.source),
            _lib.ptr(a.scale),
            _lib.ptr(a.output),
            _c_int(w.heads),
            ctypes.c_void_p(stream),
        )


# --------------------------------------------------------------- nvfp4_prepare
class Nvfp4PrepareWorkload(Workload):
    num_tokens: int
    heads: int
    center: bool = False
    transpose: bool = False
    hadamard: bool = False
    global_scale: float = 0.0


class Nvfp4PrepareConfig(Config):
    tile_tokens: int = 16
    threads: int = 256


@dataclasses.dataclass(frozen=True, slots=True)
class Nvfp4PrepareArguments(Arguments):
    source: TensorDesc
    mean: TensorDesc | None
    quantized: TensorDesc
    scales: TensorDesc
    heads: int
    transpose: bool = False
    hadamard: bool = False
    global_scale: float = 0.0

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("num_tokens", self.source.shape[0]),)


class Nvfp4PrepareKernel(Kernel[Nvfp4PrepareArguments, Nvfp4PrepareWorkload, Nvfp4PrepareConfig]):
    name = "nvfp4_prepare"
    symbol = "nob200_nvfp4_prepare"

    @classmethod
    def make_arguments(cls, workload: Nvfp4PrepareWorkload) -> Nvfp4PrepareArguments:
        padded = -(-workload.num_tokens // 128) * 128
        num_rows = 128 if workload.transpose else padded
        columns = padded if workload.transpose else 128
        return Nvfp4PrepareArguments(
            TensorDesc.empty(DType.BF16, (workload.num_tokens, workload.heads * 128)),
            TensorDesc.empty(DType.F32, (workload.heads, 128)) if workload.center else None,
            TensorDesc.empty(DType.U8, (workload.heads, num_rows, columns // 2)),
            TensorDesc.empty(DType.FP8_UE4M3, (workload.heads, num_rows, columns // 16)),
            workload.heads,
            workload.transpose,
            workload.hadamard,
            workload.global_scale,
        )

    @classmethod
    def make_workload(cls, arguments: Nvfp4PrepareArguments) -> Nvfp4PrepareWorkload:
        assert arguments.source.dtype == DType.BF16
        num_tokens, width = arguments.source.shape
        assert width == arguments.heads * 128
        padded = -(-num_tokens // 128) * 128
        num_rows = 128 if arguments.transpose else padded
        columns = padded if arguments.transpose else 128
        assert arguments.quantized.dtype == DType.U8
        assert arguments.quantized.shape == (arguments.heads, num_rows, columns // 2)
        assert arguments.scales.dtype == DType.FP8_UE4M3
        assert arguments.scales.shape == (arguments.heads, num_rows, columns // 16)
        if arguments.mean is not None:
            assert arguments.mean.dtype == DType.F32
            assert arguments.mean.shape == (arguments.heads, 128)
        assert arguments.global_scale >= 0
        return Nvfp4PrepareWorkload(
            num_tokens=num_tokens,
            heads=arguments.heads,
            center=arguments.mean is not None,
            transpose=arguments.transpose,
            hadamard=arguments.hadamard,
            global_scale=arguments.global_scale,
        )

    @classmethod
    def make_config(cls, workload: Nvfp4PrepareWorkload) -> Nvfp4PrepareConfig:
        return Nvfp4PrepareConfig()

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            _c_int(w.num_tokens),
            _lib.ptr(a.source),
            _lib.ptr(a.mean),
            _lib.ptr(a.quantized),
            _lib.ptr(a.scales),
            _c_int(w.heads),
            _c_int(int(w.transpose)),
            _c_int(int(w.hadamard)),
            ctypes.c_float(w.global_scale),
            ctypes.c_void_p(stream),
        )


class Hadamard128Workload(Workload):
    tokens: int = Field(gt=0)
    heads: int = Field(gt=0)
    total_heads: int = Field(gt=0)


@dataclasses.dataclass(frozen=True, slots=True)
class Hadamard128Arguments(Arguments):
    input: TensorDesc
    output: TensorDesc
    heads: int
    head_offset: int = 0

    def dynamic_parameters(self) -> tuple[tuple[str, int], ...]:
        return (("tokens", self.input.shape[0]), ("head_offset", self.head_offset))


class Hadamard128Kernel(Kernel[Hadamard128Arguments, Hadamard128Workload, Int8Fp8ThreadConfig]):
    """The normalised 128-point Walsh-Hadamard transform of the quantisers on heads [head_offset, head_offset + heads)
    of a bf16 tensor [tokens, total_heads, 128]; its own inverse, in place allowed.  It brings an attention output
    computed on rotated V back to the original channels.  No counterpart in the reference."""

    name = "hadamard128_heads"
    symbol = "nob200_hadamard128_heads"

    @classmethod
    def make_arguments(cls, workload: Hadamard128Workload) -> Hadamard128Arguments:
        shape = (workload.tokens, workload.total_heads, 128)
        return Hadamard128Arguments(TensorDesc.empty(DType.BF16, shape), TensorDesc.empty(DType.BF16, shape), workload.heads)

    @classmethod
    def make_config(cls, workload: Hadamard128Workload) -> Int8Fp8ThreadConfig:
        return Int8Fp8ThreadConfig()

    @classmethod
    def make_workload(cls, arguments: Hadamard128Arguments) -> Hadamard128Workload:
        assert arguments.input.dtype == arguments.output.dtype == DType.BF16
        assert arguments.input.shape == arguments.output.shape and len(arguments.input.shape) == 3
        tokens, total_heads, dim = arguments.input.shape
        assert dim == 128 and 0 <= arguments.head_offset <= total_heads - arguments.heads
        return Hadamard128Workload(tokens=tokens, heads=arguments.heads, total_heads=total_heads)

    def _launch(self, function, stream: int) -> int:
        a, w = self.arguments, self.workload
        return function(
            ctypes.c_int(w.tokens), ctypes.c_int(a.head_offset), _lib.ptr(a.input), _lib.ptr(a.output),
            ctypes.c_int(w.heads), ctypes.c_int(w.total_heads), ctypes.c_void_p(stream),
        )  # fmt: skip


def hadamard128_rows(tensor, output=None, stream: int | None = None):
    """Transform of bf16 rows ``[..., 128]`` (see ``Hadamard128Kernel``); ``output`` defaults to in place."""
    import torch

    assert tensor.is_cuda and tensor.is_contiguous() and tensor.dtype == torch.bfloat16 and tensor.shape[-1] == 128
    output = tensor if output is None else output
    assert output.shape == tensor.shape and output.dtype == tensor.dtype and output.is_contiguous()
    code = _lib.symbol("nob200_hadamard128_rows")(
        ctypes.c_longlong(tensor.numel() // 128), _lib.ptr(tensor), _lib.ptr(output),
        ctypes.c_void_p(_lib.current_stream() if stream is None else stream),
    )  # fmt: skip
    if code != 0:
        raise RuntimeError(f"nob200_hadamard128_rows: {_lib.last_error()} (status {code})")
    return output
