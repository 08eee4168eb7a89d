"""Attention operators: the kernel order, scratch tensors and argument wiring of one head slice.

These follow the attention part of the reference operators

* ``DenseBf16Attention``      src/nano_omni/ops/minimax_h3/dense_bf16_attention.py:24-98
* ``project_attention``       src/nano_omni/ops/minimax_h3/attention.py:73-139 (dense int8-fp8)
* ``PrepareKeyValue`` / ``QuerySlice``  src/nano_omni/ops/minimax_h3/attention_slices.py:60-161
* ``DenseNvfp4Attention``     src/nano_omni/ops/minimax_h3/dense_nvfp4_attention.py:33-151
* ``SolAttention``            src/nano_omni/ops/minimax_h3/sol_attention.py:62-160
* ``SolInt8Fp8Attention``     src/nano_omni/ops/minimax_h3/sol_int8_fp8_attention.py:57-230
* ``SolNvfp4Attention``       src/nano_omni/ops/minimax_h3/sol_nvfp4_attention.py:50-228
* ``KernelSequence.linear`` / ``PreparedInput``  src/nano_omni/ops/matmul/sequence.py:29-235 (bf16 and int8 weights)

from the point where the projected, normalised and rotated Q, K, V of a head slice exist as bf16
``[tokens, heads * 128]``.  The projections, norm-RoPE and the output projection around them are the
reference's own kernels and stay where they are; an operator here takes ``query, key, value`` as inputs
and produces ``attended`` ``[tokens, total_heads, 128]`` at ``head_offset``.

``Op`` keeps the reference's planning interface (core/op.py:14-82): inputs at construction, outputs bound
once with ``to()``, ``prepare()`` returning the ordered kernel calls and the scratch bytes, every temporary
reserved by name in a ``ScratchLayout`` at 256-byte alignment.  ``bind`` resolves the scratch offsets
against a base address, which is what the reference planner does for its arena.
"""

from __future__ import annotations

import abc
import dataclasses
from collections.abc import Iterable

from nano_omni_b200.core import DType, Kernel, ScratchLayout, TensorDesc, TensorKind
from nano_omni_b200.kernels.dense_bf16 import (
    DenseBf16AttentionArguments,
    DenseBf16AttentionConfig,
    DenseBf16AttentionKernel,
    choose_kv_splits,
    splitkv_workspace_bytes,
)
from nano_omni_b200.kernels.dense_int8_fp8 import (
    DenseInt8Fp8AttentionArguments,
    DenseInt8Fp8AttentionConfig,
    DenseInt8Fp8AttentionKernel,
)
from nano_omni_b200.kernels.dense_nvfp4 import DenseNvfp4Arguments, DenseNvfp4Kernel, DenseNvfp4Workload
from nano_omni_b200.kernels.matmul import (
    ConvRotInt8Arguments,
    ConvRotInt8Kernel,
    Int8RowwiseArguments,
    Int8RowwiseKernel,
    MatmulBf16Arguments,
    MatmulBf16Kernel,
    MatmulInt8Arguments,
    MatmulInt8Kernel,
)
from nano_omni_b200.kernels.norm_rope import (
    H3HeadNormRopeArguments,
    H3HeadNormRopeKernel,
    H3QueryPrepareArguments,
    H3QueryPrepareKernel,
)
from nano_omni_b200.kernels.quantize import (
    Hadamard128Arguments,
    Hadamard128Kernel,
    Int8Fp8QuantizeQKArguments,
    Int8Fp8QuantizeQKKernel,
    Int8Fp8QuantizeValueArguments,
    Int8Fp8QuantizeValueKernel,
    Int8Fp8ValueScaleArguments,
    Int8Fp8ValueScaleKernel,
    Nvfp4PrepareArguments,
    Nvfp4PrepareKernel,
    TokenGroupMeanArguments,
    TokenGroupMeanKernel,
    TokenGroupMeanWorkload,
)
from nano_omni_b200.kernels.sol import (
    SolAttentionArguments,
    SolAttentionKernel,
    SolCenteredPoolArguments,
    SolInt8Fp8PoolKernel,
    SolNvfp4PoolKernel,
    SolNvfp4SelectArguments,
    SolNvfp4SelectKernel,
    SolPoolArguments,
    SolPoolKernel,
    SolStatsArguments,
    SolStatsKernel,
)
from nano_omni_b200.kernels.sol_exact import (
    SolInt8Fp8AttentionArguments,
    SolInt8Fp8AttentionKernel,
    SolNvfp4Arguments,
    SolNvfp4FinalizeArguments,
    SolNvfp4FinalizeKernel,
    SolNvfp4Kernel,
    SolNvfp4Workload,
)


@dataclasses.dataclass(frozen=True, slots=True)
class PreparedInput:
    """One unchanged projection input whose quantised form and LoRA compressions are shared by sibling projections
    (ops/matmul/sequence.py:29-122).  INT8 only: the fp8 branch of the reference is not built."""

    sequence: "KernelSequence"
    input: TensorDesc
    _quantized: dict = dataclasses.field(default_factory=dict, init=False, repr=False)
    _compressed: dict = dataclasses.field(default_factory=dict, init=False, repr=False)

    def compress(self, name: str, weight: TensorDesc) -> TensorDesc:
        if weight not in self._compressed:
            output = self.sequence.temporary(f"{name}.down", DType.BF16, (self.input.shape[0], weight.shape[0]))
            self.sequence.emit(MatmulBf16Kernel, MatmulBf16Arguments(self.input, weight, None, None, None, output, 1.0, False))
            self._compressed[weight] = output
        return self._compressed[weight]

    def quantize(self, name: str, dtype: DType, input_scale: TensorDesc | None, rotation_group: int):
        if dtype != DType.I8:
            raise ValueError(f"unsupported quantized input dtype: {dtype}")
        key = (dtype, None, rotation_group)
        if key not in self._quantized:
            sequence, input = self.sequence, self.input
            quantized = sequence.temporary(f"{name}.quantized", dtype, input.shape)
            scales = sequence.temporary(f"{name}.scales", DType.F32, (input.shape[0],))
            if rotation_group:
                # The reference sends rows wider than 16384 columns through a separate rotation kernel (bf16 out) and
                # then int8_rowwise; the fused kernel here rounds the rotated row to bf16 as well and stages up to
                # 65536 columns in shared memory, so it serves both branches with the same bytes.
                sequence.emit(ConvRotInt8Kernel, ConvRotInt8Arguments(input, quantized, scales, rotation_group))
            else:
                sequence.emit(Int8RowwiseKernel, Int8RowwiseArguments(input, quantized, scales))
            self._quantized[key] = quantized, scales
        return self._quantized[key]


class KernelSequence:
    """Named temporaries and ordered kernel calls of one operator (ops/matmul/sequence.py:125-235)."""

    def __init__(self, scratch: ScratchLayout) -> None:
        self.scratch = scratch
        self.calls: list[Kernel] = []

    def temporary(self, name: str, dtype: DType, shape: tuple[int, ...]) -> TensorDesc:
        return self.scratch.reserve(name, dtype, shape)

    def emit(self, kernel: type[Kernel], arguments, config=None) -> None:
        self.calls.append(kernel(arguments, config))

    def prepare(self, input: TensorDesc) -> PreparedInput:
        return PreparedInput(self, input)

    def linear(self, name: str, input: TensorDesc | PreparedInput, weight: TensorDesc, output: TensorDesc, *,
               weight_scale: float | TensorDesc = 1.0, input_scale: TensorDesc | None = None,
               bias: TensorDesc | None = None, residual: TensorDesc | None = None, multiply: TensorDesc | None = None,
               use_silu: bool = False, loras: tuple[tuple[TensorDesc, TensorDesc, float], ...] = (),
               rotation_group: int = 0) -> None:  # fmt: skip
        """Emit a projection (ops/matmul/sequence.py:141-235): every LoRA pair adds
        ``strength * (input x down^T) x up^T`` through the residual chain, in order, before the main GEMM;
        bf16 and int8 weights (int8 needs a weight-scale tensor; the activations are quantised once per input)."""
        prepared = input if isinstance(input, PreparedInput) else self.prepare(input)
        if prepared.sequence is not self:
            raise ValueError("prepared input belongs to a different kernel sequence")
        source = prepared.input
        if source.dtype != DType.BF16 or source.shape[1] != weight.shape[1]:
            raise ValueError("linear expects BF16 input with matching inner dimension")
        if output.shape != (source.shape[0], weight.shape[0]) or output.dtype != DType.BF16:
            raise ValueError("linear output shape or dtype mismatch")
        if weight.dtype == DType.I8 and not isinstance(weight_scale, TensorDesc):
            raise TypeError("INT8 linear requires a weight_scale buffer")
        for index, (down, up, strength) in enumerate(loras):
            compressed = prepared.compress(f"{name}.lora{index}", down)
            update = self.temporary(f"{name}.lora{index}.up", DType.BF16, output.shape)
            self.emit(MatmulBf16Kernel, MatmulBf16Arguments(compressed, up, None, residual, None, update, strength, False))
            residual = update
        if weight.dtype == DType.BF16:
            self.emit(MatmulBf16Kernel, MatmulBf16Arguments(source, weight, bias, residual, multiply, output, 1.0, use_silu))
        elif weight.dtype == DType.I8:
            quantized, scales = prepared.quantize(name, DType.I8, None, rotation_group)
            self.emit(
                MatmulInt8Kernel,
                MatmulInt8Arguments(quantized, weight, bias, residual, multiply, output, weight_scale, scales, use_silu),
            )
        else:
            raise ValueError(f"unsupported linear weight dtype: {weight.dtype}")


class Op(abc.ABC):
    def __init__(self, *inputs: TensorDesc, outputs: tuple[tuple[DType, tuple[int, ...]], ...]) -> None:
        self.inputs = inputs
        self.output_specs = outputs
        self.outputs: tuple[TensorDesc, ...] | None = None

    def to(self, *outputs: TensorDesc):
        """Bind the outputs once; returns this operator."""
        assert self.outputs is None, "operator already finalized"
        assert len(outputs) == len(self.output_specs), "operator output count mismatch"
        for tensor, (dtype, shape) in zip(outputs, self.output_specs, strict=True):
            assert tensor.dtype == dtype, "operator output dtype mismatch"
            assert tensor.shape == shape, "operator output shape mismatch"
        self.outputs = tuple(outputs)
        return self

    @property
    def bound_outputs(self) -> tuple[TensorDesc, ...]:
        assert self.outputs is not None, "operator output bindings are required"
        return self.outputs

    def prepare(self) -> tuple[tuple[Kernel, ...], int]:
        """Kernel calls in execution order (scratch still as offsets) and the scratch bytes they need."""
        assert self.outputs is not None, "operator output bindings are required"
        scratch = ScratchLayout()
        calls = tuple(self.kernels(scratch))
        return calls, scratch.num_bytes

    def bind(self, scratch_base: int) -> tuple[Kernel, ...]:
        """``prepare()`` with every scratch descriptor resolved to ``scratch_base + offset``."""
        calls, _ = self.prepare()

        def resolve(tensor: TensorDesc) -> TensorDesc:
            if tensor.kind != TensorKind.SCRATCH:
                return tensor
            return TensorDesc(tensor.dtype, tensor.shape, TensorKind.DEVICE, (scratch_base, tensor.info[1]))

        return tuple(call.map_arguments(resolve) for call in calls)

    def run(self, scratch, stream: int | None = None) -> None:
        """Submit every call on ``stream``; ``scratch`` is a CUDA uint8 tensor of at least ``prepare()[1]`` bytes."""
        _, need = self.prepare()
        assert scratch.numel() * scratch.element_size() >= need, f"operator needs {need} B of scratch"
        assert scratch.data_ptr() % 256 == 0, "scratch must be 256-byte aligned"
        for call in self.bind(scratch.data_ptr()):
            call.submit(stream)

    @abc.abstractmethod
    def kernels(self, scratch: ScratchLayout) -> Iterable[Kernel]:
        raise NotImplementedError


class Linear(Op):
    """One projection as an operator: ``KernelSequence.linear`` with its temporaries in the operator's scratch.
    ``loras`` are (down [rank, k], up [n, rank], strength) triples."""

    def __init__(self, input: TensorDesc, weight: TensorDesc, **options) -> None:
        super().__init__(input, weight, outputs=((DType.BF16, (input.shape[0], weight.shape[0])),))
        self.options = options

    def kernels(self, scratch: ScratchLayout) -> list[Kernel]:
        sequence = KernelSequence(scratch)
        sequence.linear("linear", self.inputs[0], self.inputs[1], self.bound_outputs[0], **self.options)
        return sequence.calls


@dataclasses.dataclass(frozen=True, slots=True)
class Rotation:
    """Per-head RMS-norm weights of Q and K (bf16 [128]) and the rotary planes (f32 [tokens, 48], or both None).

    An operator given a ``Rotation`` takes Q and K as they leave the projections and applies the norm and the
    split-half RoPE itself (``h3_head_norm_rope``, or ``h3_query_prepare`` where the query goes straight to int8),
    as the reference operators do before attention (ops/minimax_h3/attention.py:51-97, sol_attention.py:105-131).
    """

    query_norm: TensorDesc
    key_norm: TensorDesc
    cosines: TensorDesc | None = None
    sines: TensorDesc | None = None


def _rotated(sequence: KernelSequence, name: str, tensor: TensorDesc, norm: TensorDesc, rotation: Rotation) -> TensorDesc:
    """Norm + RoPE of a projected ``[tokens, heads * 128]`` tensor into a temporary of the same shape."""
    rows, width = tensor.shape
    head_shape = (rows, width // 128, 128)
    out = sequence.temporary(f"{name}.rotated", DType.BF16, (rows, width))
    sequence.emit(
        H3HeadNormRopeKernel,
        H3HeadNormRopeArguments(tensor.view(head_shape), norm, rotation.cosines, rotation.sines, out.view(head_shape)),
    )
    return out


def _slice_shape(query: TensorDesc, key: TensorDesc, value: TensorDesc) -> tuple[int, int]:
    rows, width = query.shape
    assert query.dtype == key.dtype == value.dtype == DType.BF16
    assert key.shape == value.shape == (rows, width) and width % 128 == 0
    return rows, width // 128


def _key_mean(sequence: KernelSequence, key: TensorDesc, rows: int, width: int) -> TensorDesc:
    """Per-channel mean of K over all tokens (ops/minimax_h3/attention.py:98-101)."""
    mean = sequence.temporary("key.mean", DType.F32, (1, width))
    need = TokenGroupMeanKernel.workspace_bytes(
        TokenGroupMeanWorkload(num_tokens=rows, columns=width, tokens_per_block=rows, include_padding=False)
    )
    partial = sequence.temporary("key.mean.partial", DType.U8, (need,)) if need else None
    sequence.emit(TokenGroupMeanKernel, TokenGroupMeanArguments(key, mean, rows, False, partial))
    return mean


class _SliceAttention(Op):
    """Common construction: Q, K, V of one head slice in, ``[tokens, total_heads, 128]`` out at ``head_offset``."""

    def __init__(self, query: TensorDesc, key: TensorDesc, value: TensorDesc, *, total_heads: int, head_offset: int = 0,
                 rotation: Rotation | None = None):  # fmt: skip
        self.rows, self.heads = _slice_shape(query, key, value)
        assert 0 <= head_offset <= total_heads - self.heads
        self.total_heads, self.head_offset = total_heads, head_offset
        self.rotation = rotation
        super().__init__(query, key, value, outputs=((DType.BF16, (self.rows, total_heads, 128)),))

    def prepared_inputs(self, sequence: KernelSequence) -> tuple[TensorDesc, TensorDesc, TensorDesc]:
        """Q, K, V as attention consumes them: Q and K normalised and rotated when the operator was given a Rotation."""
        query, key, value = self.inputs
        if self.rotation is not None:
            query = _rotated(sequence, "query", query, self.rotation.query_norm, self.rotation)
            key = _rotated(sequence, "key", key, self.rotation.key_norm, self.rotation)
        return query, key, value

    @property
    def head_shape(self) -> tuple[int, int, int]:
        return (self.rows, self.heads, 128)


class DenseBf16Attention(_SliceAttention):
    """One launch; key splits (and their workspace) chosen for the slice when it leaves SMs idle."""

    def __init__(self, query, key, value, *, total_heads: int, head_offset: int = 0, kv_splits: int | None = None,
                 rotation: Rotation | None = None):  # fmt: skip
        super().__init__(query, key, value, total_heads=total_heads, head_offset=head_offset, rotation=rotation)
        self.kv_splits = kv_splits if kv_splits is not None else choose_kv_splits(self.rows, self.heads)

    def kernels(self, scratch: ScratchLayout) -> list[Kernel]:
        sequence = KernelSequence(scratch)
        query, key, value = (t.view(self.head_shape) for t in self.prepared_inputs(sequence))
        need = splitkv_workspace_bytes(self.rows, self.heads, self.kv_splits)
        workspace = sequence.temporary("splitkv", DType.U8, (need,)) if need else None
        sequence.emit(
            DenseBf16AttentionKernel,
            DenseBf16AttentionArguments(query, key, value, self.bound_outputs[0], self.head_offset, workspace),
            DenseBf16AttentionConfig(kv_splits=self.kv_splits),
        )
        return sequence.calls


def _quantise_key_value_int8(sequence: KernelSequence, key, value, rows: int, heads: int, outputs=None, rotated=False):
    """K mean, centred int8 K with 64-token scales, V scale, permuted channel-major e4m3 V
    (ops/minimax_h3/attention.py:98-124).  ``outputs`` places the four results in given tensors.
    ``rotated``: the benchmark's variant instead - K through the Walsh-Hadamard rotation, not centred, one scale
    per 128 tokens."""
    width = heads * 128
    block = 128 if rotated else 64
    krows = -(-rows // block) * block
    if rotated:
        mean = sequence.temporary("key.statistics", DType.F32, (1, width))  # slot of the ABI; not read
    else:
        mean = _key_mean(sequence, key, rows, width)
    if outputs is None:
        key_i8 = sequence.temporary("key.values", DType.I8, (heads, krows, 128))
        key_scale = sequence.temporary("key.scales", DType.F32, (heads, krows // block))
        value_fp8 = sequence.temporary("value.packed", DType.FP8_E4M3, (heads, 128, -(-rows // 64) * 64))
        value_scale = sequence.temporary("value.fp8_scales", DType.F32, (heads, 128))
    else:
        key_i8, key_scale, value_fp8, value_scale = outputs
    sequence.emit(
        Int8Fp8QuantizeQKKernel,
        Int8Fp8QuantizeQKArguments(key, mean, key_i8, key_scale, heads, block, not rotated, rotated),
    )
    sequence.emit(Int8Fp8ValueScaleKernel, Int8Fp8ValueScaleArguments(value, value_scale, heads))
    sequence.emit(Int8Fp8QuantizeValueKernel, Int8Fp8QuantizeValueArguments(value, value_scale, value_fp8, heads))
    return mean, key_i8, key_scale, value_fp8, value_scale


def _quantise_query_int8(
    sequence: KernelSequence, query, mean, rows: int, heads: int, rotation: Rotation | None = None, rotated=False
):
    """int8 Q with 32-token scales; with a Rotation the norm, RoPE and quantiser run as one kernel
    (ops/minimax_h3/attention.py:51-70).  ``rotated``: Walsh-Hadamard rotation and one scale per 128 tokens."""
    block = 128 if rotated else 32
    qrows = -(-rows // block) * block
    query_i8 = sequence.temporary("query.values", DType.I8, (heads, qrows, 128))
    query_scale = sequence.temporary("query.qk_scales", DType.F32, (heads, qrows // block))
    if rotated:
        sequence.emit(
            Int8Fp8QuantizeQKKernel, Int8Fp8QuantizeQKArguments(query, mean, query_i8, query_scale, heads, 128, False, True)
        )
    elif rotation is not None:
        sequence.emit(
            H3QueryPrepareKernel,
            H3QueryPrepareArguments(query, rotation.query_norm, rotation.cosines, rotation.sines, query_i8, query_scale),
        )
    else:
        sequence.emit(
            Int8Fp8QuantizeQKKernel, Int8Fp8QuantizeQKArguments(query, mean, query_i8, query_scale, heads, 32, False)
        )
    return query_i8, query_scale


class DenseInt8Fp8Attention(Op):
    """Quantise Q, K, V and attend; output ``[tokens, heads * 128]`` (this path has no head offset,
    int8_fp8/dense.py:21-60)."""

    def __init__(self, query: TensorDesc, key: TensorDesc, value: TensorDesc, *, rotation: Rotation | None = None,
                 hadamard: bool = False) -> None:  # fmt: skip
        self.rows, self.heads = _slice_shape(query, key, value)
        self.rotation = rotation
        # the benchmark's int8-fp8 configuration: Q and K through the Walsh-Hadamard rotation, scales per 128 tokens
        self.hadamard = hadamard
        super().__init__(query, key, value, outputs=((DType.BF16, (self.rows, self.heads * 128)),))

    def kernels(self, scratch: ScratchLayout) -> list[Kernel]:
        query, key, value = self.inputs
        sequence = KernelSequence(scratch)
        if self.rotation is not None:
            key = _rotated(sequence, "key", key, self.rotation.key_norm, self.rotation)
            if self.hadamard:  # the fused query kernel has no Hadamard stage
                query = _rotated(sequence, "query", query, self.rotation.query_norm, self.rotation)
        mean, key_i8, key_scale, value_fp8, value_scale = _quantise_key_value_int8(
            sequence, key, value, self.rows, self.heads, rotated=self.hadamard
        )
        query_i8, query_scale = _quantise_query_int8(
            sequence, query, mean, self.rows, self.heads, self.rotation, rotated=self.hadamard
        )
        blocks = (128, 128) if self.hadamard else (32, 64)
        sequence.emit(
            DenseInt8Fp8AttentionKernel,
            DenseInt8Fp8AttentionArguments(
                query_i8, key_i8, value_fp8, query_scale, key_scale, value_scale, self.bound_outputs[0],
                self.rows, self.heads, self.rows, *blocks,
            ),
        )
        return sequence.calls


class PrepareKeyValue(Op):
    """Quantised K and V that persist across query slices (attention_slices.py:60-110): outputs
    int8 K ``[heads, rows64, 128]``, its scales, e4m3 V ``[heads, 128, rows64]``, its scales."""

    def __init__(self, key: TensorDesc, value: TensorDesc, *, rotation: Rotation | None = None) -> None:
        self.rows, self.heads = _slice_shape(key, key, value)
        self.rotation = rotation
        krows = -(-self.rows // 64) * 64
        super().__init__(
            key,
            value,
            outputs=(
                (DType.I8, (self.heads, krows, 128)),
                (DType.F32, (self.heads, krows // 64)),
                (DType.FP8_E4M3, (self.heads, 128, krows)),
                (DType.F32, (self.heads, 128)),
            ),
        )

    def kernels(self, scratch: ScratchLayout) -> list[Kernel]:
        key, value = self.inputs
        sequence = KernelSequence(scratch)
        if self.rotation is not None:
            key = _rotated(sequence, "key", key, self.rotation.key_norm, self.rotation)
        _quantise_key_value_int8(sequence, key, value, self.rows, self.heads, self.bound_outputs)
        return sequence.calls


class QuerySlice(Op):
    """A chunk of queries against the persistent quantised K/V (attention_slices.py:113-161)."""

    def __init__(self, query, key_i8, key_scale, value_fp8, value_scale, *, total_tokens: int,
                 rotation: Rotation | None = None) -> None:  # fmt: skip
        rows, width = query.shape
        assert query.dtype == DType.BF16 and width % 128 == 0
        self.rows, self.heads, self.total_tokens = rows, width // 128, total_tokens
        self.rotation = rotation  # its rotary planes cover the rows of this slice
        assert key_i8.shape == (self.heads, -(-total_tokens // 64) * 64, 128)
        super().__init__(query, key_i8, key_scale, value_fp8, value_scale, outputs=((DType.BF16, (rows, width)),))

    def kernels(self, scratch: ScratchLayout) -> list[Kernel]:
        query, key_i8, key_scale, value_fp8, value_scale = self.inputs
        sequence = KernelSequence(scratch)
        # queries are not centred, so the statistics slot only needs a valid [1, width] tensor
        unused = sequence.temporary("query.statistics", DType.F32, (1, self.heads * 128))
        query_i8, query_scale = _quantise_query_int8(sequence, query, unused, self.rows, self.heads, self.rotation)
        # a slice of queries is few CTAs: divide the keys when that fills the last wave of SMs better
        splits = choose_kv_splits(self.rows, self.heads, num_kv_tokens=self.total_tokens)
        need = splitkv_workspace_bytes(self.rows, self.heads, splits)
        workspace = sequence.temporary("splitkv", DType.U8, (need,)) if need else None
        sequence.emit(
            DenseInt8Fp8AttentionKernel,
            DenseInt8Fp8AttentionArguments(
                query_i8, key_i8, value_fp8, query_scale, key_scale, value_scale, self.bound_outputs[0],
                self.total_tokens, self.heads, self.rows, workspace=workspace,
            ),
            DenseInt8Fp8AttentionConfig(kv_splits=splits),
        )
        return sequence.calls


def _prepare_nvfp4(sequence: KernelSequence, query, key, value, rows: int, heads: int, global_scales=None):
    """K mean, then e2m1 + ue4m3 operands: Q plain, K centred, V transposed (dense_nvfp4_attention.py:107-133).
    ``global_scales`` (q, k, v): the benchmark's variant instead - all three through the Walsh-Hadamard rotation, K not
    centred, block scales divided by the tensor's global scale."""
    padded = -(-rows // 128) * 128
    mean = None if global_scales else _key_mean(sequence, key, rows, heads * 128)
    query_fp4 = sequence.temporary("query.fp4", DType.U8, (heads, padded, 64))
    key_fp4 = sequence.temporary("key.fp4", DType.U8, (heads, padded, 64))
    value_fp4 = sequence.temporary("value.fp4", DType.U8, (heads, 128, padded // 2))
    query_scale = sequence.temporary("query.scale", DType.FP8_UE4M3, (heads, padded, 8))
    key_scale = sequence.temporary("key.scale", DType.FP8_UE4M3, (heads, padded, 8))
    value_scale = sequence.temporary("value.scale", DType.FP8_UE4M3, (heads, 128, padded // 16))
    if global_scales:
        gq, gk, gv = global_scales
        sequence.emit(Nvfp4PrepareKernel, Nvfp4PrepareArguments(query, None, query_fp4, query_scale, heads, False, True, gq))
        sequence.emit(Nvfp4PrepareKernel, Nvfp4PrepareArguments(key, None, key_fp4, key_scale, heads, False, True, gk))
        sequence.emit(Nvfp4PrepareKernel, Nvfp4PrepareArguments(value, None, value_fp4, value_scale, heads, True, True, gv))
    else:
        sequence.emit(Nvfp4PrepareKernel, Nvfp4PrepareArguments(query, None, query_fp4, query_scale, heads, False))
        sequence.emit(
            Nvfp4PrepareKernel, Nvfp4PrepareArguments(key, mean.view((heads, 128)), key_fp4, key_scale, heads, False)
        )
        sequence.emit(Nvfp4PrepareKernel, Nvfp4PrepareArguments(value, None, value_fp4, value_scale, heads, True))
    return mean, (query_fp4, key_fp4, value_fp4, query_scale, key_scale, value_scale)


class DenseNvfp4Attention(_SliceAttention):
    """``global_scales`` (q, k, v) selects the benchmark's NVFP4 configuration: operands through the Walsh-Hadamard
    rotation with one global scale per tensor; the output, computed on rotated V, is rotated back in place."""

    def __init__(self, query, key, value, *, total_heads: int, head_offset: int = 0, rotation: Rotation | None = None,
                 global_scales: tuple[float, float, float] | None = None):  # fmt: skip
        super().__init__(query, key, value, total_heads=total_heads, head_offset=head_offset, rotation=rotation)
        self.global_scales = global_scales

    def kernels(self, scratch: ScratchLayout) -> list[Kernel]:
        sequence = KernelSequence(scratch)
        query, key, value = self.prepared_inputs(sequence)
        _, operands = _prepare_nvfp4(sequence, query, key, value, self.rows, self.heads, self.global_scales)
        sequence.emit(
            DenseNvfp4Kernel,
            DenseNvfp4Arguments(
                *operands, self.bound_outputs[0], self.rows, self.rows, self.head_offset, None,
                self.global_scales or (1.0, 1.0, 1.0),
            ),
        )
        if self.global_scales:
            attended = self.bound_outputs[0]
            sequence.emit(Hadamard128Kernel, Hadamard128Arguments(attended, attended, self.heads, self.head_offset))
        return sequence.calls


class _SolSliceAttention(_SliceAttention):
    def __init__(self, query, key, value, *, total_heads: int, head_offset: int = 0, protected_tokens: int, tau: float = 1.0,
                 rotation: Rotation | None = None):  # fmt: skip
        super().__init__(query, key, value, total_heads=total_heads, head_offset=head_offset, rotation=rotation)
        assert 0 <= protected_tokens <= self.rows
        self.tau = tau
        self.protected_tokens = protected_tokens

    def blocks(self, block: int) -> int:
        return -(-self.rows // block)

    def protected_blocks(self, block: int) -> int:
        return -(-self.protected_tokens // block)


class SolAttention(_SolSliceAttention):
    """bf16 sol: pool, statistics, then router + block-sparse attention (sol_attention.py:62-160).
    ``block`` 128 and ``topk_fraction`` select the top-k routing over 128-token blocks."""

    def __init__(self, query, key, value, *, total_heads: int, head_offset: int = 0, protected_tokens: int,
                 tau: float = 1.0, block: int = 64, topk_fraction: float = 0.0, rotation: Rotation | None = None):  # fmt: skip
        super().__init__(query, key, value, total_heads=total_heads, head_offset=head_offset,
                         protected_tokens=protected_tokens, tau=tau, rotation=rotation)  # fmt: skip
        self.block, self.topk_fraction = block, topk_fraction

    def kernels(self, scratch: ScratchLayout) -> list[Kernel]:
        nb = self.blocks(self.block)
        sequence = KernelSequence(scratch)
        query, key, value = (t.view(self.head_shape) for t in self.prepared_inputs(sequence))
        pooled = sequence.temporary("pooled", DType.BF16, (2, self.heads, nb, 128))
        stats = sequence.temporary("stats", DType.F32, (self.heads, 2, 128))
        mask = sequence.temporary("selected", DType.U8, (nb, self.heads, nb))
        scores = (
            sequence.temporary("scores", DType.U8, (nb * nb * self.heads * 4,)) if self.topk_fraction > 0 else None
        )
        sequence.emit(SolPoolKernel, SolPoolArguments(key, value, pooled, self.block))
        sequence.emit(SolStatsKernel, SolStatsArguments(pooled, stats))
        sequence.emit(
            SolAttentionKernel,
            SolAttentionArguments(
                query, key, value, pooled, stats, self.bound_outputs[0], self.tau, self.head_offset,
                self.protected_blocks(self.block), mask, self.block, self.topk_fraction, scores,
            ),
        )
        return sequence.calls


def _route(
    sequence: KernelSequence, op: _SolSliceAttention, pool_kernel: type[Kernel], query, key, value, mean
) -> tuple[TensorDesc, TensorDesc]:
    """Three pooled planes, statistics of the plain block means, threshold mask
    (sol_int8_fp8_attention.py:161-190): returns (pooled, selected)."""
    nb = op.blocks(64)
    pooled = sequence.temporary("pooled", DType.BF16, (3, op.heads, nb, 128))
    stats = sequence.temporary("stats", DType.F32, (op.heads, 2, 128))
    selected = sequence.temporary("selected", DType.U8, (nb, op.heads, nb))
    sequence.emit(pool_kernel, SolCenteredPoolArguments(key, value, mean.view((op.heads, 128)), pooled, 64))
    sequence.emit(SolStatsKernel, SolStatsArguments(pooled, stats))
    sequence.emit(
        SolNvfp4SelectKernel,
        SolNvfp4SelectArguments(query, pooled.plane(0), stats, selected, op.tau, op.protected_blocks(64)),
    )
    return pooled, selected


class SolInt8Fp8Attention(_SolSliceAttention):
    """int8-fp8 sol: quantise, route, exact stage with state, finalize in place
    (sol_int8_fp8_attention.py:57-230: ``exact`` is the output tensor itself)."""

    def kernels(self, scratch: ScratchLayout) -> list[Kernel]:
        attended = self.bound_outputs[0]
        sequence = KernelSequence(scratch)
        # the router and finalize read the rotated bf16 query, so it is materialised even on the int8 path
        query, key, value = self.prepared_inputs(sequence)
        mean, key_i8, key_scale, value_fp8, value_scale = _quantise_key_value_int8(sequence, key, value, self.rows, self.heads)
        query_i8, query_scale = _quantise_query_int8(sequence, query, mean, self.rows, self.heads)
        q3, k3, v3 = (t.view(self.head_shape) for t in (query, key, value))
        pooled, selected = _route(sequence, self, SolInt8Fp8PoolKernel, q3, k3, v3, mean)
        state = sequence.temporary("state", DType.F32, (self.rows, self.total_heads, 2))
        sequence.emit(
            SolInt8Fp8AttentionKernel,
            SolInt8Fp8AttentionArguments(
                query_i8, key_i8, value_fp8, query_scale, key_scale, value_scale, selected, attended, state,
                self.rows, self.head_offset, self.tau, self.protected_blocks(64),
            ),
        )
        sequence.emit(
            SolNvfp4FinalizeKernel,
            SolNvfp4FinalizeArguments(q3, pooled, selected, attended, state, attended, self.head_offset),
        )
        return sequence.calls


class SolNvfp4Attention(_SolSliceAttention):
    """nvfp4 sol: prepare, route, exact stage with state, finalize in place (sol_nvfp4_attention.py:50-228)."""

    def kernels(self, scratch: ScratchLayout) -> list[Kernel]:
        attended = self.bound_outputs[0]
        sequence = KernelSequence(scratch)
        query, key, value = self.prepared_inputs(sequence)
        mean, operands = _prepare_nvfp4(sequence, query, key, value, self.rows, self.heads)
        q3, k3, v3 = (t.view(self.head_shape) for t in (query, key, value))
        pooled, selected = _route(sequence, self, SolNvfp4PoolKernel, q3, k3, v3, mean)
        state = sequence.temporary("state", DType.F32, (self.rows, self.total_heads, 2))
        sequence.emit(
            SolNvfp4Kernel,
            SolNvfp4Arguments(
                *operands, selected, attended, state, self.rows, self.rows, self.head_offset, self.tau,
                max(1, self.protected_blocks(64)),
            ),
        )
        sequence.emit(
            SolNvfp4FinalizeKernel,
            SolNvfp4FinalizeArguments(q3, pooled, selected, attended, state, attended, self.head_offset),
        )
        return sequence.calls


ATTENTION_OPS = {
    ("dense", "bf16"): DenseBf16Attention,
    ("dense", "int8_fp8"): DenseInt8Fp8Attention,
    ("dense", "nvfp4"): DenseNvfp4Attention,
    ("sol", "bf16"): SolAttention,
    ("sol", "int8_fp8"): SolInt8Fp8Attention,
    ("sol", "nvfp4"): SolNvfp4Attention,
}
"""The reference's dispatch strings: attention ``dense|sol`` x precision ``bf16|int8_fp8|nvfp4``
(src/nano_omni/models/h3/blocks.py:213-239)."""
