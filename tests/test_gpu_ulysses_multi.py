"""Two-GPU check of the sequence<->head reshard (skipped on a single-GPU box): both transports must
reproduce the single-GPU attention of the full problem on every rank's rows."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, transport, result, groups=0):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nano_omni_b200 import _lib
        from nano_omni_b200.ulysses import _cuda_dense_bf16, make_plan

        T, H = 2048, 4
        g = torch.Generator().manual_seed(17)
        q, k, v = (torch.randn(T, H, 128, generator=g).bfloat16().cuda() for _ in range(3))
        full = torch.empty_like(q)
        _cuda_dense_bf16(q, k, v, full)
        lt = T // world
        sl = slice(rank * lt, (rank + 1) * lt)
        plan, used = make_plan(T, H, world, rank, transport=transport)
        assert used == transport
        out = torch.empty(lt, H, 128, dtype=torch.bfloat16, device="cuda")
        ok = True
        for _ in range(3):  # repeated steps exercise buffer reuse and the epoch barriers
            out.fill_(float("nan"))
            if groups:
                plan.dense_bf16_pipelined(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), out, groups)
            else:
                plan.dense_bf16(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), out)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(out, full[sl]))
        ok = ok and _lib.read_status() == 0
        result[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("transport", ["nccl", "p2p"])
def test_two_gpu_reshard_equals_single_gpu(transport):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    manager = mp.get_context("spawn").Manager()
    result = manager.dict()
    mp.spawn(_worker, args=(2, _free_port(), transport, result), nprocs=2, join=True)
    assert dict(result) == {0: True, 1: True}


@pytest.mark.parametrize("groups", [1, 2])
def test_two_gpu_pipelined_reshard_equals_single_gpu(groups):
    """Head groups pushed on a second stream while the previous group is attended: same rows as one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    manager = mp.get_context("spawn").Manager()
    result = manager.dict()
    mp.spawn(_worker, args=(2, _free_port(), "p2p", result, groups), nprocs=2, join=True)
    assert dict(result) == {0: True, 1: True}


def _int8_worker(rank, world, port, result):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nano_omni_b200 import _lib, ops
        from nano_omni_b200.core import TensorDesc
        from nano_omni_b200.ulysses import make_plan

        T, H = 2048, 4
        g = torch.Generator().manual_seed(29)
        q, k, v = (torch.randn(T, H, 128, generator=g).bfloat16().cuda() for _ in range(3))
        k = k + 0.5  # a non-zero column mean, so that the centring matters
        desc = TensorDesc.from_torch
        # single GPU: the operator on the whole problem
        whole = torch.empty(T, H * 128, dtype=torch.bfloat16, device="cuda")
        op = ops.DenseInt8Fp8Attention(*(desc(t.view(T, H * 128)) for t in (q, k, v)))
        op.to(desc(whole))
        scratch = torch.empty(op.prepare()[1] + 256, dtype=torch.uint8, device="cuda")
        op.run(scratch[(-scratch.data_ptr()) % 256 :])
        lt = T // world
        sl = slice(rank * lt, (rank + 1) * lt)
        plan, used = make_plan(T, H, world, rank, transport="p2p")
        out = torch.empty(lt, H, 128, dtype=torch.bfloat16, device="cuda")
        ok = True
        for _ in range(2):
            out.fill_(float("nan"))
            plan.dense_int8_fp8(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), out)
            torch.cuda.synchronize()
            got, want = out.float(), whole.view(T, H, 128)[sl].float()
            # the K mean is summed shard by shard: K bytes may differ by one step on rounding boundaries
            ok = ok and bool(torch.isfinite(got).all()) and float((got - want).abs().max()) <= 0.02
            ok = ok and float(torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)) >= 0.9999
        # what crossed NVLink are the quantisers' own bytes: Q and V bit for bit
        I = plan._int8
        mine = slice(rank * plan.local_heads, (rank + 1) * plan.local_heads)
        q8 = torch.empty(H, T, 128, dtype=torch.int8, device="cuda")
        qs = torch.empty(H, T // 32, device="cuda")
        from nano_omni_b200.kernels import quantize as qz

        qz.Int8Fp8QuantizeQKKernel(
            qz.Int8Fp8QuantizeQKArguments(desc(q.view(T, H * 128)), desc(I["mean"]), desc(q8), desc(qs), H, 32, False)
        ).submit()
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(I["recv"]["q8"], q8[mine])) and bool(torch.equal(I["recv"]["qs"], qs[mine]))
        ok = ok and _lib.read_status() == 0
        result[rank] = ok
    finally:
        dist.destroy_process_group()


def test_two_gpu_int8_quantised_before_the_exchange():
    """Dense int8-fp8 attention whose quantisers run on the token shards: bytes and scales cross NVLink."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    manager = mp.get_context("spawn").Manager()
    result = manager.dict()
    mp.spawn(_int8_worker, args=(2, _free_port(), result), nprocs=2, join=True)
    assert dict(result) == {0: True, 1: True}


def _sol_worker(rank, world, port, result):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nano_omni_b200 import _lib
        from nano_omni_b200.ulysses import make_plan
        from tests.test_gpu_sol_attention import sol_attend
        from tests.test_gpu_sol_route import gpu_pool, gpu_stats, structured_keys

        T, H, block, protected = 2048, 4, 128, 1
        g = torch.Generator().manual_seed(23)
        q = torch.randn(T, H, 128, generator=g).bfloat16().cuda()
        k = structured_keys(24, T, H, block)
        v = torch.randn(T, H, 128, generator=g).bfloat16().cuda()
        pooled = gpu_pool(k, v, None, block)
        stats = gpu_stats(pooled)
        full, full_mask = sol_attend(q, k, v, pooled, stats, 1.0, protected, block, topk=0.25)
        lt, lh = T // world, H // world
        sl = slice(rank * lt, (rank + 1) * lt)
        plan, used = make_plan(T, H, world, rank, transport="p2p")
        out = torch.empty(lt, H, 128, dtype=torch.bfloat16, device="cuda")
        ok = True
        for _ in range(2):
            out.fill_(float("nan"))
            mask = plan.sol_bf16(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), out, protected,
                                 block=block, topk_fraction=0.25)
            torch.cuda.synchronize()
            # masks of this rank's heads equal the single-GPU masks bit for bit; so do the output rows
            ok = ok and bool(torch.equal(mask, full_mask[:, rank * lh : (rank + 1) * lh]))
            ok = ok and bool(torch.equal(out, full[sl]))
        ok = ok and _lib.read_status() == 0
        result[rank] = ok
    finally:
        dist.destroy_process_group()


def test_two_gpu_sol_attention_equals_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    manager = mp.get_context("spawn").Manager()
    result = manager.dict()
    mp.spawn(_sol_worker, args=(2, _free_port(), result), nprocs=2, join=True)
    assert dict(result) == {0: True, 1: True}


def _sol_quantised_worker(rank, world, port, precision, result):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nano_omni_b200 import _lib, ops
        from nano_omni_b200.core import TensorDesc
        from nano_omni_b200.ulysses import make_plan
        from tests.test_gpu_sol_route import structured_keys

        T, H, protected_tokens = 2048, 4, 100
        g = torch.Generator().manual_seed(29)
        q = torch.randn(T, H, 128, generator=g).bfloat16().cuda()
        k = structured_keys(30, T, H, 64)
        v = torch.randn(T, H, 128, generator=g).bfloat16().cuda()
        lt, lh = T // world, H // world
        # single-GPU result, head group by head group (statistics and routing are per head)
        full = torch.empty(T, H, 128, dtype=torch.bfloat16, device="cuda")
        for group in range(world):
            heads = slice(group * lh, (group + 1) * lh)
            flat = lambda t: TensorDesc.from_torch(t[:, heads].contiguous().view(T, lh * 128))  # noqa: E731
            op = ops.ATTENTION_OPS[("sol", precision)](
                flat(q), flat(k), flat(v), total_heads=H, head_offset=group * lh, protected_tokens=protected_tokens
            ).to(TensorDesc.from_torch(full))
            scratch = torch.empty(op.prepare()[1] + 256, dtype=torch.uint8, device="cuda")
            op.run(scratch[(-scratch.data_ptr()) % 256 :])
        torch.cuda.synchronize()
        sl = slice(rank * lt, (rank + 1) * lt)
        plan, used = make_plan(T, H, world, rank, transport="p2p")
        out = torch.empty(lt, H, 128, dtype=torch.bfloat16, device="cuda")
        ok = True
        for _ in range(2):
            out.fill_(float("nan"))
            plan.sol_quantised(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), out, precision, protected_tokens)
            torch.cuda.synchronize()
            ok = ok and bool(torch.isfinite(out.float()).all()) and bool(torch.equal(out, full[sl]))
        ok = ok and _lib.read_status() == 0
        result[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("precision", ["int8_fp8", "nvfp4"])
def test_two_gpu_quantised_sol_equals_single_gpu(precision):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    manager = mp.get_context("spawn").Manager()
    result = manager.dict()
    mp.spawn(_sol_quantised_worker, args=(2, _free_port(), precision, result), nprocs=2, join=True)
    assert dict(result) == {0: True, 1: True}
