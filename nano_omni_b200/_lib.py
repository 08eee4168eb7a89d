"""ctypes loader for the C-ABI shared library (built by ``nano_omni_b200.build``).

There is no fallback: if ``libnano_omni_b200.so`` is missing every launch raises.
"""

from __future__ import annotations

import ctypes
import os
from functools import cache

LIB_NAME = "libnano_omni_b200.so"
# NOB200_LIBRARY names another build of the same library (the checked build of ``nano_omni_b200.build --checked``)
LIB_PATH = os.environ.get("NOB200_LIBRARY") or os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)


class LibraryMissing(RuntimeError):
    pass


@cache
def library() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            f"{LIB_PATH} is not built; run `python -m nano_omni_b200.build` "
            "(needs nvcc with sm_100a support). There is no CPU or eager fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.nob200_last_error.restype = ctypes.c_char_p
    lib.nob200_last_error.argtypes = []
    return lib


def symbol(name: str):
    function = getattr(library(), name)
    function.restype = ctypes.c_int
    return function


def last_error() -> str:
    text = library().nob200_last_error()
    return text.decode() if text else ""


def current_stream() -> int:
    import torch

    return int(torch.cuda.current_stream().cuda_stream)


def ptr(value) -> ctypes.c_void_p:
    """Device pointer of a TensorDesc / torch tensor / int, or NULL for None."""
    if value is None:
        return ctypes.c_void_p(0)
    if isinstance(value, int):
        return ctypes.c_void_p(value)
    return ctypes.c_void_p(value.data_ptr())


def read_status(stream: int | None = None) -> int:
    """Synchronise ``stream`` and return-and-clear the device status word.

    Non-zero means a bounded device-side wait gave up (the kernel returned
    early and its outputs are not valid).
    """
    out = ctypes.c_uint32(0)
    code = symbol("nob200_read_status")(
        ctypes.byref(out), ctypes.c_void_p(current_stream() if stream is None else stream)
    )
    if code != 0:
        raise RuntimeError(f"nob200_read_status: {last_error()}")
    return int(out.value)
