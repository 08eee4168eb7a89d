"""The attention parity tests once more against the checked build of the library (``nano_omni_b200.build --checked``):
every store index the kernels compute by hand is tested against its tensor's extent there, and a failed test sets a
status bit that the parity tests' ``read_status() == 0`` assertions would see.  Stands in for a memory checker."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED = os.path.join(ROOT, "nano_omni_b200", "libnano_omni_b200_checked.so")
FILES = [
    "tests/test_gpu_attention_bf16.py",
    "tests/test_gpu_attention_int8.py",
    "tests/test_gpu_attention_nvfp4.py",
    "tests/test_gpu_sol_attention.py",
    "tests/test_gpu_sol_exact.py",
]


def test_attention_parity_with_index_checks():
    if not os.path.exists(CHECKED):
        pytest.skip("checked library not built (python -m nano_omni_b200.build --checked)")
    if os.environ.get("NOB200_LIBRARY"):
        pytest.skip("already running against another build of the library")
    env = dict(os.environ, NOB200_LIBRARY=CHECKED)
    run = subprocess.run(
        [sys.executable, "-m", "pytest", *FILES, "-x", "-q", "-m", "gpu", "-k", "not full_size", "-p", "no:cacheprovider"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=1500,
    )
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-2000:]


def test_out_of_range_heads_never_reach_the_checks():
    """The index checks guard arithmetic inside the kernels; arguments that would put a store outside its tensor (here a
    head slice [1, 3) of a tensor with 2 heads) are refused on the host before anything is launched."""
    import ctypes

    import torch

    lib = ctypes.CDLL(CHECKED if os.path.exists(CHECKED) else os.path.join(ROOT, "nano_omni_b200", "libnano_omni_b200.so"))
    q = torch.zeros(256, 2, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(256, 2, 128, dtype=torch.bfloat16, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    code = lib.nob200_dense_bf16_attention_d128(
        ctypes.c_int(256), ctypes.c_int(1), p(q), p(q), p(q), p(out), ctypes.c_int(2), ctypes.c_int(2), ctypes.c_void_p(0)
    )
    assert code != 0
    torch.cuda.synchronize()
    assert (out == 0).all()
