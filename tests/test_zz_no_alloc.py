"""The allocation-free column mean must agree with the workspace-taking entry point.

``nob200_token_group_mean_static`` exists for callers that cannot hand the kernel a
scratch buffer because their device memory was laid out before execution began (or
whose hot path must not call cudaMalloc, which stalls all streams of the device).  It
keeps its partial sums in an array built into the library.  Both entry points run the
same kernels in the same summation order, so their outputs must be bit-identical, also
when the built-in array still holds the sums of an earlier, differently shaped call.

This file is named to be collected last, so a run that stops at the first failure has
already covered every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

LIMIT = 4 << 20


def _call_static(src, out, tpb, pad):
    from nano_omni_b200 import _lib

    fn = _lib.symbol("nob200_token_group_mean_static")
    T, C = src.shape
    return fn(
        ctypes.c_int(T),
        ctypes.c_void_p(src.data_ptr()),
        ctypes.c_void_p(out.data_ptr()),
        ctypes.c_int(C),
        ctypes.c_int(tpb),
        ctypes.c_int(int(pad)),
        ctypes.c_void_p(_lib.current_stream()),
    )


def _call_workspace(src, out, tpb, pad):
    from nano_omni_b200 import _lib

    T, C = src.shape
    size = _lib.library().nob200_token_group_mean_workspace_bytes
    size.restype = ctypes.c_size_t
    need = size(ctypes.c_int(T), ctypes.c_int(C), ctypes.c_int(tpb))
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    rc = _lib.symbol("nob200_token_group_mean")(
        ctypes.c_int(T),
        ctypes.c_void_p(src.data_ptr()),
        ctypes.c_void_p(out.data_ptr()),
        ctypes.c_int(C),
        ctypes.c_int(tpb),
        ctypes.c_int(int(pad)),
        ctypes.c_void_p(ws.data_ptr()),
        ctypes.c_size_t(need),
        ctypes.c_void_p(_lib.current_stream()),
    )
    torch.cuda.synchronize()
    return rc


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    from nano_omni_b200 import _lib

    g = torch.Generator().manual_seed(11)
    # two calls in a row with different shapes: the second finds the first call's sums in the array
    cases = [(5000, 512, 5000, False), (3001, 256, 1000, True)]
    for T, C, tpb, pad in cases:
        src = (torch.randn(T, C, generator=g) * 3).bfloat16().cuda()
        groups = -(-T // tpb)
        want = torch.full((groups, C), float("nan"), device="cuda")
        got = torch.full((groups, C), float("nan"), device="cuda")
        assert _call_workspace(src, want, tpb, pad) == 0, _lib.last_error()
        assert _call_static(src, got, tpb, pad) == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want)  # same kernels, same order of additions: tolerance zero
        assert torch.isfinite(got).all()


def test_static_scratch_rejects_shapes_beyond_its_limit():
    from nano_omni_b200 import _lib

    T, C = 65536, 4096  # 512 chunks x 4096 columns x 4 B = 8 MiB > 4 MiB
    src = torch.zeros(8, C, dtype=torch.bfloat16, device="cuda")  # never read: the call is refused first
    out = torch.zeros(1, C, device="cuda")
    fn = _lib.symbol("nob200_token_group_mean_static")
    rc = fn(
        ctypes.c_int(T),
        ctypes.c_void_p(src.data_ptr()),
        ctypes.c_void_p(out.data_ptr()),
        ctypes.c_int(C),
        ctypes.c_int(T),
        ctypes.c_int(0),
        ctypes.c_void_p(_lib.current_stream()),
    )
    assert rc == -1
    message = _lib.last_error()
    assert str(8 << 20) in message and str(LIMIT) in message


def test_static_scratch_direct_path_exact_limit_and_oracle():
    """Three more corners: groups of up to 128 tokens (no scratch touched at all), a shape that needs exactly the
    whole built-in array (the accepting side of the limit), and the CPU oracle's column mean."""
    from nano_omni_b200 import _lib
    from oracle import reference_math as rm

    g = torch.Generator().manual_seed(12)
    # (tokens, columns, tokens per group, count padding): 256 chunks x 1024 columns x 4 B = 4 MiB exactly
    for T, C, tpb, pad in [(300, 256, 64, False), (32768, 1024, 32768, False)]:
        src = torch.randn(T, C, generator=g).bfloat16().cuda()
        groups = -(-T // tpb)
        want = torch.full((groups, C), float("nan"), device="cuda")
        got = torch.full((groups, C), float("nan"), device="cuda")
        assert _call_workspace(src, want, tpb, pad) == 0, _lib.last_error()
        assert _call_static(src, got, tpb, pad) == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert torch.equal(got.cpu(), rm.token_group_mean(src.cpu(), tpb, pad))


def test_static_entry_point_leaves_device_memory_alone():
    """Backs the statement that the call allocates nothing: free device memory is the same before and after a call
    (the first call of the process, which looks up the array's address, has happened in the tests above or here)."""
    from nano_omni_b200 import _lib

    src = torch.ones(4096, 512, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(1, 512, device="cuda")
    assert _call_static(src, out, 4096, False) == 0, _lib.last_error()
    torch.cuda.synchronize()
    before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        assert _call_static(src, out, 4096, False) == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == before
    assert torch.equal(out, torch.ones_like(out))
