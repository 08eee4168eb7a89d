"""Registry of kernel classes by reference ``name`` (src/nano_omni/kernels/__init__.py:11-29)."""

from __future__ import annotations

from functools import cache

from nano_omni_b200.core import Kernel


@cache
def classes() -> dict[str, type[Kernel]]:
    from nano_omni_b200.kernels import dense_bf16, dense_int8_fp8, dense_nvfp4, matmul, norm_rope, quantize, sol, sol_exact

    found: dict[str, type[Kernel]] = {}
    for module in (dense_bf16, dense_int8_fp8, dense_nvfp4, matmul, norm_rope, quantize, sol, sol_exact):
        for value in vars(module).values():
            if isinstance(value, type) and issubclass(value, Kernel) and value is not Kernel and value.name:
                assert value.name not in found or found[value.name] is value, f"duplicate kernel {value.name}"
                found[value.name] = value
    return found
