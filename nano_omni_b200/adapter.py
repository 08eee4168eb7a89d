"""Reference-side binding: let nano-omni's own ``Kernel`` classes launch this library.

nano-omni compiles a TileLang program in ``Kernel.compile()`` and launches it in ``Kernel.submit()``
(src/nano_omni/core/kernel.py:192-222).  ``install()`` walks the reference's kernel registry
(src/nano_omni/kernels/__init__.py:11-29) and, for every class whose ``name`` this library implements, replaces
those two methods: ``compile`` binds the C-ABI symbol instead of compiling, ``submit`` translates the reference
``Arguments`` (same field names, same order; this library's extra trailing fields take their defaults) into this
library's class of the same ``name`` and enqueues its launch on the reference runtime's compute stream.  Nothing
above the ``Kernel`` layer changes.

    import nano_omni_b200.adapter as adapter
    adapter.install()            # once, after `import nano_omni`

The prepare / bind passes of the reference runtime (``execution._compiling`` set, launches stubbed and pointers
null: src/nano_omni/core/runtime/execution.py:212-216,246-287) launch nothing here either.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable

from nano_omni_b200 import kernels
from nano_omni_b200.core import DType, Kernel, TensorDesc, TensorKind


def translate_tensor(tensor: Any) -> TensorDesc | None:
    """A reference ``TensorDesc`` (dtype, shape, kind, info) as this library's; addressed tensors keep their address."""
    if tensor is None:
        return None
    dtype = DType(str(tensor.dtype.value)) if hasattr(tensor.dtype, "value") else DType(str(tensor.dtype))
    info = tuple(tensor.info)
    if str(getattr(tensor.kind, "value", tensor.kind)) == "device":
        return TensorDesc(dtype, tuple(tensor.shape), TensorKind.DEVICE, info)
    return TensorDesc(dtype, tuple(tensor.shape), TensorKind(str(getattr(tensor.kind, "value", tensor.kind))), info)


def translate_arguments(ours: type[Kernel], reference_arguments: Any):
    """Build ``ours``' Arguments from the reference's: fields are matched by name, in the reference's order."""
    target = ours.arguments_type()
    wanted = {f.name for f in dataclasses.fields(target)}
    values = {}
    for field in dataclasses.fields(reference_arguments):
        assert field.name in wanted, f"{ours.name}: reference field {field.name!r} has no counterpart"
        value = getattr(reference_arguments, field.name)
        if isinstance(value, tuple) and value and hasattr(value[0], "info"):
            value = tuple(translate_tensor(item) for item in value)
        elif hasattr(value, "info") and hasattr(value, "shape"):
            value = translate_tensor(value)
        values[field.name] = value
    return target(**values)


def field_differences(ours: type[Kernel], reference: type) -> list[str]:
    """Where the two classes of one ``name`` disagree: Arguments fields (the reference's must be a prefix of ours,
    in order) and Workload fields (ours a superset).  Empty when they agree."""
    problems: list[str] = []
    ref_args = [f.name for f in dataclasses.fields(_generic_argument(reference, 0))]
    our_args = [f.name for f in dataclasses.fields(ours.arguments_type())]
    if our_args[: len(ref_args)] != ref_args:
        problems.append(f"{ours.name}: Arguments {our_args} do not start with the reference's {ref_args}")
    ref_workload = set(_generic_argument(reference, 1).model_fields)
    our_workload = set(ours.workload_type().model_fields)
    if not ref_workload <= our_workload:
        problems.append(f"{ours.name}: Workload lacks {sorted(ref_workload - our_workload)}")
    return problems


def _generic_argument(cls: type, index: int):
    """Type argument ``index`` of the ``Kernel[...]`` base a reference class was declared with."""
    for base in getattr(cls, "__orig_bases__", ()):
        arguments = getattr(base, "__args__", ())
        if len(arguments) == 3:
            return arguments[index]
    raise TypeError(f"{cls.__name__} does not name its Arguments / Workload / Config types")


def install(
    reference_classes: Callable[[], dict[str, type]] | None = None,
    stream: Callable[[], int] | None = None,
    compiling: Callable[[], Any] | None = None,
) -> dict[str, type]:
    """Patch every reference kernel class this library implements; returns {name: patched reference class}.

    The three hooks default to the reference's own modules (``nano_omni.kernels.classes``,
    ``execution.stream()``, ``execution._compiling``); tests pass stand-ins.
    """
    if reference_classes is None:
        from nano_omni import kernels as reference_kernels

        reference_classes = reference_kernels.classes
    if stream is None or compiling is None:
        from nano_omni.core.runtime import execution

        stream = stream or (lambda: int(execution.stream()))
        compiling = compiling or (lambda: execution._compiling)
    ours_by_name = kernels.classes()
    found = reference_classes()
    if not isinstance(found, dict):
        found = {cls.name: cls for cls in found}
    patched: dict[str, type] = {}
    for name, reference in found.items():
        ours = ours_by_name.get(name)
        if ours is None:
            continue
        problems = field_differences(ours, reference)
        assert not problems, "; ".join(problems)
        _patch(reference, ours, stream, compiling)
        patched[name] = reference
    return patched


def _patch(reference: type, ours: type[Kernel], stream: Callable[[], int], compiling: Callable[[], Any]) -> None:
    def compile(self) -> None:  # noqa: A001 - the reference's method name
        if self.compiled is None:
            self.compiled = ours.bound_symbol()

    def submit(self) -> None:
        assert self.compiled is not None, "kernel must be compiled before submission"
        if compiling() is not None:
            return  # prepare / bind pass: nothing is launched and pointers are placeholders
        ours(translate_arguments(ours, self.arguments)).submit(stream())

    reference.compile = compile
    reference.submit = submit
    reference.b200_implementation = ours
