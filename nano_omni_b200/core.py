"""Kernel plug-in contract: tensor descriptors, argument records and the Kernel base.

The value types here restate the interface that nano-omni kernels are written
against (reference: src/nano_omni/core/tensor.py:17-147 for DType/TensorDesc,
src/nano_omni/core/kernel.py:56-228 for Workload/Config/Arguments/Kernel), so a
kernel class from this package can stand where the reference class of the same
``name`` stands: same constructor, same ``make_arguments / make_workload /
make_config / tops`` classmethods, same argument order at launch (dynamic
scalars first, then every tensor leaf in dataclass field order).

What differs: ``compile()`` binds a symbol of the prebuilt C-ABI shared library
instead of JIT-compiling a TileLang program, and ``submit()`` enqueues that
symbol on a CUDA stream.  There is no CPU path; a missing library is an error.
"""

from __future__ import annotations

import abc
import dataclasses
import math
from enum import StrEnum
from typing import Any, Callable, ClassVar, Generic, TypeVar

from pydantic import BaseModel, ConfigDict


class DType(StrEnum):
    """Element types carried by tensor descriptors (tensor.py:17-40)."""

    F32 = "F32"
    F16 = "F16"
    I32 = "I32"
    U32 = "U32"
    I8 = "I8"
    BF16 = "BF16"
    FP8_E4M3 = "FP8_E4M3"
    FP8_UE4M3 = "FP8_UE4M3"
    U8 = "U8"
    FP4 = "U8"  # two e2m1 codes per byte travel as U8

    @property
    def itemsize(self) -> int:
        if self in (DType.F32, DType.I32, DType.U32):
            return 4
        return 2 if self in (DType.F16, DType.BF16) else 1


class TensorKind(StrEnum):
    EMPTY = "empty"
    FILE = "file"
    INPUT = "input"
    OUTPUT = "output"
    ACTIVATION = "activation"
    SCRATCH = "scratch"
    SCALAR = "scalar"
    WEIGHT = "weight"
    WORKSPACE = "workspace"
    PINNED = "pinned"
    DEVICE = "device"
    HOST = "host"


class MmaType(StrEnum):
    """Operand/accumulator signature used by ``Kernel.tops`` (kernel.py:20-29)."""

    F4F4F32 = "F4F4F32"
    F8F8F16 = "F8F8F16"
    F8F8F32 = "F8F8F32"
    F16F16F32 = "F16F16F32"
    BF16BF16F32 = "BF16BF16F32"
    TF32TF32F32 = "TF32TF32F32"
    I8I8I32 = "I8I8I32"


def _torch_dtype(dtype: DType):
    import torch

    return {
        DType.F32: torch.float32,
        DType.F16: torch.float16,
        DType.I32: torch.int32,
        DType.U32: torch.uint32,
        DType.I8: torch.int8,
        DType.BF16: torch.bfloat16,
        DType.FP8_E4M3: torch.float8_e4m3fn,
        # positive e4m3 bytes are the carrier of ue4m3 scale factors
        DType.FP8_UE4M3: torch.float8_e4m3fn,
        DType.U8: torch.uint8,
    }[dtype]


@dataclasses.dataclass(frozen=True, slots=True, eq=False)
class TensorDesc:
    """Shape and dtype paired with an address (tensor.py:66-160).

    ``info`` is ``(base, byte_offset)`` once addressed.  ``tensor`` optionally
    keeps the torch tensor the descriptor was made from alive; it takes no part
    in equality or hashing.
    """

    dtype: DType
    shape: tuple[int, ...]
    kind: TensorKind
    info: tuple[int, ...]
    tensor: Any = None

    def __eq__(self, other: object) -> bool:
        if not isinstance(other, TensorDesc):
            return NotImplemented
        return (self.dtype, self.shape, self.kind, self.info) == (
            other.dtype,
            other.shape,
            other.kind,
            other.info,
        )

    def __hash__(self) -> int:
        return hash((self.dtype, self.shape, self.kind, self.info))

    @classmethod
    def empty(cls, dtype: DType, shape: tuple[int, ...]) -> "TensorDesc":
        return cls(dtype, tuple(shape), TensorKind.EMPTY, ())

    @classmethod
    def scratch(cls, offset: int, dtype: DType, shape: tuple[int, ...]) -> "TensorDesc":
        return cls(dtype, tuple(shape), TensorKind.SCRATCH, (0, offset))

    @classmethod
    def from_pointer(cls, pointer: int, dtype: DType, shape: tuple[int, ...]) -> "TensorDesc":
        return cls(dtype, tuple(shape), TensorKind.DEVICE, (pointer, 0))

    @classmethod
    def from_torch(cls, tensor, dtype: DType | None = None) -> "TensorDesc":
        """Describe a contiguous torch tensor (CUDA for launches, CPU for checks)."""
        import torch

        assert tensor.is_contiguous(), "kernel tensors are contiguous row-major"
        if dtype is None:
            dtype = {
                torch.float32: DType.F32,
                torch.float16: DType.F16,
                torch.int32: DType.I32,
                torch.int8: DType.I8,
                torch.bfloat16: DType.BF16,
                torch.float8_e4m3fn: DType.FP8_E4M3,
                torch.uint8: DType.U8,
            }[tensor.dtype]
        assert tensor.element_size() == dtype.itemsize
        kind = TensorKind.DEVICE if tensor.is_cuda else TensorKind.HOST
        return cls(dtype, tuple(tensor.shape), kind, (tensor.data_ptr(), 0), tensor)

    @property
    def num_bytes(self) -> int:
        return math.prod(self.shape) * self.dtype.itemsize

    def view(self, shape: tuple[int, ...], dtype: DType | None = None) -> "TensorDesc":
        """Same bytes under another shape (tensor.py view semantics: contiguous reinterpretation)."""
        dtype = dtype or self.dtype
        assert math.prod(shape) * dtype.itemsize == self.num_bytes, "view must cover the same bytes"
        return TensorDesc(dtype, tuple(shape), self.kind, self.info, self.tensor)

    def plane(self, index: int) -> "TensorDesc":
        """Sub-tensor ``self[index]`` of an addressed or scratch tensor (contiguous leading slice)."""
        assert self.kind in (TensorKind.DEVICE, TensorKind.HOST, TensorKind.SCRATCH) and 0 <= index < self.shape[0]
        step = self.num_bytes // self.shape[0]
        base, byte_offset = self.info
        return TensorDesc(self.dtype, self.shape[1:], self.kind, (base, byte_offset + index * step), None)

    def data_ptr(self) -> int:
        assert self.kind in (TensorKind.DEVICE, TensorKind.HOST), "tensor has not been addressed"
        base, byte_offset = self.info
        return base + byte_offset

    def as_torch(self):
        """Return the torch tensor behind this descriptor, typed as ``dtype``."""
        assert self.tensor is not None, "descriptor was not made from a torch tensor"
        wanted = _torch_dtype(self.dtype)
        tensor = self.tensor
        return tensor if tensor.dtype == wanted else tensor.view(wanted)


class Workload(BaseModel):
    """Logical dimensions that select a kernel specialisation (kernel.py:56-59)."""

    model_config = ConfigDict(frozen=True, extra="forbid")


class Config(BaseModel):
    """Launch-shape choices for a workload (kernel.py:62-65)."""

    model_config = ConfigDict(frozen=True, extra="forbid")


class Arguments:
    """Dataclass of tensor descriptors and scalars shared by planning and launch."""

    def dynamic_parameters(self) -> tuple[tuple[str, int | float], ...]:
        return ()

    def _leaves(self) -> list[tuple[tuple, TensorDesc | None]]:
        """(path, leaf) of every tensor slot in declaration order, depth first.  A path is the chain of field names
        and tuple positions from this object to the slot; optional slots that are empty appear with leaf None."""
        out: list[tuple[tuple, TensorDesc | None]] = []
        stack: list[tuple[tuple, object]] = [((), self)]
        while stack:
            path, node = stack.pop()
            if node is None or isinstance(node, TensorDesc):
                out.append((path, node))
                continue
            if isinstance(node, tuple):
                children = list(enumerate(node))
            elif dataclasses.is_dataclass(node) and not isinstance(node, type):
                children = [(f.name, getattr(node, f.name)) for f in dataclasses.fields(node)]
            else:
                continue  # a scalar field
            stack.extend((path + (key,), child) for key, child in reversed(children))
        return out

    def values(self, *, include_absent: bool = False) -> tuple[TensorDesc | None, ...]:
        """Tensor descriptors in the order the launch ABI passes them (the reference walks its Arguments the same
        way, kernel.py:101-120); empty optional slots are returned as None only on request.  A None that is not a
        tensor slot (a scalar default) cannot be told apart from an empty one, as in the reference."""
        return tuple(leaf for _, leaf in self._leaves() if leaf is not None or include_absent)

    def map(self, function: Callable[[TensorDesc], TensorDesc]):
        """A copy with ``function`` applied to every tensor descriptor (kernel.py:73-99)."""

        def rebuild(node, path: tuple):
            if isinstance(node, TensorDesc):
                return function(node)
            if isinstance(node, tuple):
                return tuple(rebuild(child, path + (i,)) for i, child in enumerate(node))
            if dataclasses.is_dataclass(node) and not isinstance(node, type):
                fields = {f.name: rebuild(getattr(node, f.name), path + (f.name,)) for f in dataclasses.fields(node)}
                return dataclasses.replace(node, **fields)
            return node

        return rebuild(self, ())


def require_tensor(tensor: TensorDesc, dtype: DType, shape: tuple[int, ...], what: str) -> None:
    """Shape and element type of one argument, as an AssertionError naming the argument (the error type callers
    of the reference's ``make_workload`` expect)."""
    assert tensor.dtype == dtype, f"{what}: expected {dtype.name}, got {tensor.dtype.name}"
    assert tuple(tensor.shape) == tuple(shape), f"{what}: expected shape {tuple(shape)}, got {tuple(tensor.shape)}"


ArgumentsT = TypeVar("ArgumentsT", bound=Arguments)
WorkloadT = TypeVar("WorkloadT", bound=Workload)
ConfigT = TypeVar("ConfigT", bound=Config)


class Kernel(abc.ABC, Generic[ArgumentsT, WorkloadT, ConfigT]):
    """One kernel invocation bound to a C-ABI entry point (kernel.py:123-228).

    ``name`` equals the reference kernel's registry name; ``symbol`` is the
    exported function of the shared library that implements it.
    """

    name: ClassVar[str] = ""
    symbol: ClassVar[str] = ""
    reference_rtol: ClassVar[float] = 0.02
    reference_atol: ClassVar[float] = 0.01

    def __init__(self, arguments: ArgumentsT, config: ConfigT | None = None, compiled: Any | None = None) -> None:
        self.arguments = arguments
        self.workload = self.make_workload(arguments)
        self.config = config if config is not None else type(self).make_config(self.workload)
        self.compiled = compiled

    @classmethod
    @abc.abstractmethod
    def make_arguments(cls, workload: WorkloadT) -> ArgumentsT: ...

    @classmethod
    @abc.abstractmethod
    def make_workload(cls, arguments: ArgumentsT) -> WorkloadT: ...

    @classmethod
    @abc.abstractmethod
    def make_config(cls, workload: WorkloadT) -> ConfigT: ...

    @classmethod
    def tops(cls, arguments: ArgumentsT) -> dict[MmaType, int]:
        return {}

    @classmethod
    def workspace_bytes(cls, workload: WorkloadT) -> int:
        """Scratch bytes the caller must reserve and pass as ``workspace``."""
        return 0

    @classmethod
    def _type_argument(cls, index: int):
        for klass in cls.__mro__:
            for base in getattr(klass, "__orig_bases__", ()):
                arguments = getattr(base, "__args__", ())
                if len(arguments) == 3:
                    return arguments[index]
        raise TypeError(f"{cls.__name__} does not name its Arguments / Workload / Config types")

    @classmethod
    def arguments_type(cls):
        return cls._type_argument(0)

    @classmethod
    def workload_type(cls):
        return cls._type_argument(1)

    @classmethod
    def bound_symbol(cls):
        """The C-ABI function this class launches; raises if the library was not built."""
        from nano_omni_b200 import _lib

        return _lib.symbol(cls.symbol)

    def compile(self) -> None:
        """Bind the shared-library symbol; raises if the library was not built."""
        if self.compiled is None:
            self.compiled = type(self).bound_symbol()

    @abc.abstractmethod
    def _launch(self, function: Any, stream: int) -> int:
        """Call the bound symbol with this invocation's scalars and pointers."""

    def submit(self, stream: int | None = None) -> None:
        """Enqueue on ``stream`` (default: torch's current stream); never syncs."""
        from nano_omni_b200 import _lib

        if self.compiled is None:
            self.compile()
        if stream is None:
            stream = _lib.current_stream()
        code = self._launch(self.compiled, stream)
        if code != 0:
            raise RuntimeError(f"{type(self).symbol}: {_lib.last_error()} (status {code})")

    def __call__(self, stream: int | None = None) -> None:
        self.submit(stream)

    def map_arguments(self, function: Callable[[TensorDesc], TensorDesc]):
        import copy

        result = copy.copy(self)
        result.arguments = self.arguments.map(function)
        return result


def aligned(size: int, alignment: int) -> int:
    assert size >= 0 and alignment > 0 and not alignment & (alignment - 1)
    return (size + alignment - 1) // alignment * alignment


class ScratchLayout:
    """Named 256-byte-aligned scratch regions of one operator (layout.py:86-106)."""

    def __init__(self) -> None:
        self.regions: set[str] = set()
        self.num_bytes = 0

    def reserve(self, name: str, dtype: DType, shape: tuple[int, ...], alignment: int = 256) -> TensorDesc:
        assert name not in self.regions, f"scratch region already declared: {name}"
        offset = aligned(self.num_bytes, alignment)
        tensor = TensorDesc.scratch(offset, dtype, shape)
        self.regions.add(name)
        self.num_bytes = offset + tensor.num_bytes
        return tensor
