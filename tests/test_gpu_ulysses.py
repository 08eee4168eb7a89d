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
