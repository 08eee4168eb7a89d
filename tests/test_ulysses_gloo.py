"""Exchange plan of the Ulysses reshard on CPU: world_size 2 over gloo.

The CUDA pack/unpack/attention kernels are replaced by torch equivalents here, so what is
tested is the host logic: which slab goes to which rank, and that sharded attention equals
single-process attention bit for bit.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torch_pack(src, dst, world):
    tokens, heads, _ = src.shape
    dst.copy_(src.view(tokens, world, heads // world, 128).permute(1, 0, 2, 3))


def _torch_unpack(src, dst, world):
    tokens, heads, _ = dst.shape
    dst.copy_(src.permute(1, 0, 2, 3).reshape(tokens, heads, 128))


def _oracle_attend(q, k, v, out):
    from oracle import reference_math as rm

    out.copy_(rm.dense_attention_fp32(q, k, v).to(torch.bfloat16))


def _worker(rank, world, port, tokens, heads, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nano_omni_b200.ulysses import UlyssesAttention

        g = torch.Generator().manual_seed(3)
        q, k, v = (torch.randn(tokens, heads, 128, generator=g).bfloat16() for _ in range(3))
        lt = tokens // world
        plan = UlyssesAttention(
            tokens, heads, world, rank, device="cpu", pack=_torch_pack, unpack=_torch_unpack, attend=_oracle_attend
        )
        out = torch.empty(lt, heads, 128, dtype=torch.bfloat16)
        sl = slice(rank * lt, (rank + 1) * lt)
        plan.dense_bf16(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), out)
        full = torch.empty(tokens, heads, 128, dtype=torch.bfloat16)
        _oracle_attend(q, k, v, full)
        result[rank] = bool(torch.equal(out, full[sl]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_sharded_attention_equals_single_process(world):
    tokens, heads = 64, 4
    manager = mp.get_context("spawn").Manager()
    result = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), tokens, heads, result), nprocs=world, join=True)
    assert dict(result) == {r: True for r in range(world)}


def test_geometry_is_validated():
    from nano_omni_b200.ulysses import UlyssesAttention

    with pytest.raises(ValueError):
        UlyssesAttention(64, 3, 2, 0, device="cpu")
    with pytest.raises(ValueError):
        UlyssesAttention(65, 4, 2, 0, device="cpu")


def _transport_worker(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nano_omni_b200.ulysses import make_plan

        def p2p():
            if rank == 1:
                raise RuntimeError("symmetric allocation failed on this rank")
            return "peer-memory plan"

        plan, transport = make_plan(64, 4, world, rank, device="cpu", p2p_factory=p2p, nccl_factory=lambda: "collective plan")
        result[rank] = (plan, transport)
    finally:
        dist.destroy_process_group()


def test_ranks_agree_on_the_transport_when_one_cannot_map_peer_memory():
    """One rank fails to build the peer-memory plan: every rank must fall back to the collective transport, not
    only that one (mixed transports would leave the others waiting at the flag barrier)."""
    world = 2
    manager = mp.get_context("spawn").Manager()
    result = manager.dict()
    mp.spawn(_transport_worker, args=(world, _free_port(), result), nprocs=world, join=True)
    assert dict(result) == {0: ("collective plan", "nccl"), 1: ("collective plan", "nccl")}
