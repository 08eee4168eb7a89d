"""Sequence<->head reshard around attention for 2-8 GPUs (Ulysses style).

The reference runs on one GPU only (device ordinal 0 is hard-wired,
src/nano_omni/core/runtime/execution.py:68,86); its attention ops already compute
arbitrary head subsets into a shared output through ``heads/total_heads/head_offset``
(src/nano_omni/ops/minimax_h3/dense_bf16_attention.py:60-91).  This module uses that
seam across GPUs: every rank holds ``tokens/world`` tokens of all heads; one
all-to-all gives it all tokens of ``heads/world`` heads, attention runs locally,
and a second all-to-all returns the output rows to their owners.

Per step and rank: one pack kernel per tensor (Q, K, V), one grouped exchange of all
three (NCCL point-to-point operations batched into a single group), one attention launch
(with the keys split over several CTAs when ``heads / world`` alone would leave SMs idle),
one exchange out, one unpack kernel.  Requirements: ``heads % world == 0`` and equal token
counts per rank.

``pack`` / ``unpack`` / ``attend`` are injectable so that the exchange plan can be
exercised with gloo on CPU tensors in tests; the defaults are the CUDA kernels of
this library and raise when it is missing.
"""

from __future__ import annotations

import ctypes
from typing import Callable

import torch
import torch.distributed as dist


def _cuda_pack(src: torch.Tensor, dst: torch.Tensor, world: int) -> None:
    from nano_omni_b200 import _lib

    tokens, heads, _ = src.shape
    code = _lib.symbol("nob200_ulysses_pack_heads")(
        _lib.ptr(src), _lib.ptr(dst), ctypes.c_int(tokens), ctypes.c_int(heads), ctypes.c_int(world),
        ctypes.c_void_p(_lib.current_stream()),
    )
    if code:
        raise RuntimeError(_lib.last_error())


def _cuda_unpack(src: torch.Tensor, dst: torch.Tensor, world: int) -> None:
    from nano_omni_b200 import _lib

    tokens, heads, _ = dst.shape
    code = _lib.symbol("nob200_ulysses_unpack_heads")(
        _lib.ptr(src), _lib.ptr(dst), ctypes.c_int(tokens), ctypes.c_int(heads), ctypes.c_int(world),
        ctypes.c_void_p(_lib.current_stream()),
    )
    if code:
        raise RuntimeError(_lib.last_error())


def _cuda_dense_bf16(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, kv_splits: int = 1, workspace: torch.Tensor | None = None
) -> None:
    from nano_omni_b200.core import DType, TensorDesc
    from nano_omni_b200.kernels.dense_bf16 import (
        DenseBf16AttentionArguments,
        DenseBf16AttentionConfig,
        DenseBf16AttentionKernel,
    )

    desc = TensorDesc.from_torch
    ws = desc(workspace, DType.U8) if workspace is not None and kv_splits > 1 else None
    DenseBf16AttentionKernel(
        DenseBf16AttentionArguments(desc(q), desc(k), desc(v), desc(out), 0, ws),
        DenseBf16AttentionConfig(kv_splits=kv_splits),
    ).submit()


def exchange(recv: list[torch.Tensor], send: list[torch.Tensor], rank: int, world: int, group=None) -> None:
    """All-to-all of several tensors at once: chunk p of every ``send`` tensor goes to rank p.

    All point-to-point operations are issued as one batch, which NCCL runs as a single group.
    """
    if world == 1:
        for r, s in zip(recv, send):
            r.copy_(s)
        return
    ops = []
    for r, s in zip(recv, send):
        r[rank].copy_(s[rank])
        for peer in range(world):
            if peer != rank:
                ops.append(dist.P2POp(dist.isend, s[peer], peer, group))
                ops.append(dist.P2POp(dist.irecv, r[peer], peer, group))
    for work in dist.batch_isend_irecv(ops):
        work.wait()


class UlyssesAttention:
    """Buffers and exchange plan for one (sequence length, heads, world) geometry."""

    launches_per_step = 5  # 3 pack + attention + unpack (+ 1 merge when keys are split); exchanges are NCCL's

    def __init__(
        self,
        num_tokens: int,
        heads: int,
        world: int,
        rank: int,
        device: torch.device | str = "cuda",
        group=None,
        pack: Callable = _cuda_pack,
        unpack: Callable = _cuda_unpack,
        attend: Callable | None = None,
    ) -> None:
        if heads % world:
            raise ValueError(f"heads ({heads}) must be divisible by the world size ({world})")
        if num_tokens % world:
            raise ValueError(f"tokens ({num_tokens}) must be divisible by the world size ({world})")
        self.num_tokens, self.heads, self.world, self.rank = num_tokens, heads, world, rank
        self.local_tokens = num_tokens // world
        self.local_heads = heads // world
        self.group = group
        self.pack, self.unpack = pack, unpack
        if attend is None:
            from nano_omni_b200.kernels.dense_bf16 import choose_kv_splits, splitkv_workspace_bytes

            self.kv_splits = choose_kv_splits(num_tokens, self.local_heads)
            need = splitkv_workspace_bytes(num_tokens, self.local_heads, self.kv_splits)
            self.workspace = torch.empty(need, dtype=torch.uint8, device=device) if need else None
            if self.kv_splits > 1:
                self.launches_per_step = 6
            attend = lambda q, k, v, o: _cuda_dense_bf16(q, k, v, o, self.kv_splits, self.workspace)  # noqa: E731
        self.attend = attend
        shape = (world, self.local_tokens, self.local_heads, 128)
        make = lambda: torch.empty(shape, dtype=torch.bfloat16, device=device)  # noqa: E731
        self.send = [make() for _ in range(3)]
        self.recv = [make() for _ in range(3)]
        self.out_heads = make()  # [tokens, local_heads, 128] seen as [world, local_tokens, ...]
        self.out_recv = make()

    def seq_to_head(self, local: torch.Tensor, slot: int) -> torch.Tensor:
        """[local_tokens, heads, 128] on every rank -> [tokens, local_heads, 128] on this rank."""
        assert local.shape == (self.local_tokens, self.heads, 128)
        self.pack(local, self.send[slot], self.world)
        dist.all_to_all_single(self.recv[slot], self.send[slot], group=self.group)
        return self.recv[slot].view(self.num_tokens, self.local_heads, 128)

    def head_to_seq(self, full: torch.Tensor, out_local: torch.Tensor) -> None:
        """[tokens, local_heads, 128] on every rank -> [local_tokens, heads, 128] on this rank."""
        assert out_local.shape == (self.local_tokens, self.heads, 128)
        dist.all_to_all_single(self.out_recv, full.view(self.out_recv.shape), group=self.group)
        self.unpack(self.out_recv, out_local, self.world)

    def dense_bf16(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor) -> None:
        for slot, local in enumerate((q, k, v)):
            assert local.shape == (self.local_tokens, self.heads, 128)
            self.pack(local, self.send[slot], self.world)
        exchange(self.recv, self.send, self.rank, self.world, self.group)
        qf, kf, vf = (r.view(self.num_tokens, self.local_heads, 128) for r in self.recv)
        of = self.out_heads.view(self.num_tokens, self.local_heads, 128)
        self.attend(qf, kf, vf, of)
        exchange([self.out_recv], [self.out_heads], self.rank, self.world, self.group)
        self.unpack(self.out_recv, out, self.world)
