"""Pack/unpack kernels of the sequence<->head reshard against torch permutes (bit-exact copies)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,heads,world", [(1, 2, 2), (130, 24, 8), (4096, 56, 4), (777, 6, 1)])
def test_pack_and_unpack_round_trip(tokens, heads, world):
    from nano_omni_b200 import _lib
    from nano_omni_b200.ulysses import _cuda_pack, _cuda_unpack

    g = torch.Generator().manual_seed(tokens)
    src = torch.randn(tokens, heads, 128, generator=g).bfloat16().cuda()
    packed = torch.zeros(world, tokens, heads // world, 128, dtype=torch.bfloat16, device="cuda")
    _cuda_pack(src, packed, world)
    want = src.view(tokens, world, heads // world, 128).permute(1, 0, 2, 3).contiguous()
    assert torch.equal(packed, want)
    back = torch.zeros_like(src)
    _cuda_unpack(packed, back, world)
    assert torch.equal(back, src)
    assert _lib.read_status() == 0


def test_single_rank_plan_matches_plain_kernel():
    """world=1 degenerates to pack -> attention -> unpack and must equal the direct launch."""
    import os

    import torch.distributed as dist

    from nano_omni_b200.ulysses import UlyssesAttention, _cuda_dense_bf16

    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29617")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        T, H = 512, 4
        g = torch.Generator().manual_seed(9)
        q, k, v = (torch.randn(T, H, 128, generator=g).bfloat16().cuda() for _ in range(3))
        direct = torch.empty_like(q)
        _cuda_dense_bf16(q, k, v, direct)
        plan = UlyssesAttention(T, H, 1, 0)
        out = torch.empty_like(q)
        plan.dense_bf16(q, k, v, out)
        torch.cuda.synchronize()
        assert torch.equal(out, direct)
    finally:
        dist.destroy_process_group()


def test_barrier_wait_runs_out_and_reports():
    """A cross-rank barrier whose peer never signals returns after its wait budget with status bit 16 set,
    leaves the GPU usable, and closes the scatter epilogue: attention launched afterwards stores nothing into the
    (here emulated) peers' tensors until the status word is read and cleared.  One GPU plays rank 0 of a world of 2;
    both flag arrays live on it and nothing ever writes rank 1's slot."""
    import ctypes
    import time

    from nano_omni_b200 import _lib

    kWaitTimeoutPeer = 16
    assert _lib.read_status() == 0
    flags = torch.zeros(2, 8, dtype=torch.int32, device="cuda")  # [rank][slot]
    table = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    stream = ctypes.c_void_p(_lib.current_stream())
    set_budget = _lib.symbol("nob200_set_wait_budget_ns")
    set_budget.argtypes = [ctypes.c_ulonglong]
    assert set_budget(0) != 0 and "outside" in _lib.last_error()
    assert set_budget(20_000_000) == 0  # 20 ms
    try:
        start = time.perf_counter()
        rc = _lib.symbol("nob200_ulysses_barrier")(table, ctypes.c_int(2), ctypes.c_int(0), ctypes.c_uint(1), stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        waited = time.perf_counter() - start
        assert 0.015 <= waited < 1.0, waited  # the budget, not the 2 s default and not forever
        # rank 0 signalled both ranks' arrays; its own array never saw rank 1
        assert flags.cpu().tolist()[0][:2] == [1, 0] and flags.cpu().tolist()[1][0] == 1

        # with the bit standing, the scatter epilogue must not touch the owners' tensors
        T, H = 256, 2
        g = torch.Generator().manual_seed(3)
        q, k, v = (torch.randn(T, H, 128, generator=g).bfloat16().cuda() for _ in range(3))
        halves = [torch.full((T // 2, H, 128), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        outs = (ctypes.c_void_p * 2)(halves[0].data_ptr(), halves[1].data_ptr())
        scatter = _lib.symbol("nob200_dense_bf16_attention_d128_scatter")
        args = (ctypes.c_int(T), ctypes.c_int(0), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), outs, ctypes.c_int(2), ctypes.c_int(H),
                ctypes.c_int(H), ctypes.c_int(1), ctypes.c_void_p(0), ctypes.c_size_t(0), stream)
        assert scatter(*args) == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert all(bool((h == 7.0).all()) for h in halves)
        assert _lib.read_status() == kWaitTimeoutPeer  # reported once, then cleared
        assert _lib.read_status() == 0

        # the context is intact: the same launch now writes the rows, equal to the plain kernel's
        assert scatter(*args) == 0, _lib.last_error()
        plain = torch.empty(T, H, 128, dtype=torch.bfloat16, device="cuda")
        rc = _lib.symbol("nob200_dense_bf16_attention_d128")(
            ctypes.c_int(T), ctypes.c_int(0), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(plain), ctypes.c_int(H), ctypes.c_int(H), stream
        )
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert torch.equal(torch.cat(halves), plain)
        assert _lib.read_status() == 0
    finally:
        assert set_budget(2_000_000_000) == 0
