"""Pinned-host front end: results of pipelined calls equal the direct device launch."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pipelined_calls_match_direct_launch():
    from nano_omni_b200.host_pipeline import HostAttentionPipeline
    from nano_omni_b200.ulysses import _cuda_dense_bf16

    T, h = 1024, 2
    g = torch.Generator().manual_seed(21)
    hosts = [[torch.randn(T, h, 128, generator=g).bfloat16().pin_memory() for _ in range(3)] for _ in range(5)]
    outs = [torch.empty(T, h, 128, dtype=torch.bfloat16).pin_memory() for _ in range(5)]
    pipe = HostAttentionPipeline((T, h, 128), _cuda_dense_bf16)
    for (q, k, v), o in zip(hosts, outs):
        pipe.submit(q, k, v, o)
    pipe.finish()
    for (q, k, v), o in zip(hosts, outs):
        direct = torch.empty(T, h, 128, dtype=torch.bfloat16, device="cuda")
        _cuda_dense_bf16(q.cuda(), k.cuda(), v.cuda(), direct)
        torch.cuda.synchronize()
        assert torch.equal(o, direct.cpu())
