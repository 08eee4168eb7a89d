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


class UlyssesAttentionP2P:
    """The same reshard without a collective library: peers' memory is written directly.

    All ranks allocate one symmetric buffer (``torch.distributed._symmetric_memory``: device memory
    that every rank maps into its address space over NVLink).  Per step:

    1. ``push``: this rank's Q/K/V rows are stored straight into every peer's receive area
       (``nob200_ulysses_push_heads``: the pack and the all-to-all are one kernel);
    2. cross-rank barrier (``nob200_ulysses_barrier``, bounded wait);
    3. attention on the local ``heads / world`` heads, whose epilogue stores every output row straight
       into its owner's output area (``nob200_dense_bf16_attention_d128_scatter``: the attention and
       the reverse all-to-all are one kernel);
    4. cross-rank barrier, then the output area is copied into the caller's tensor.

    Only plain loads/stores to peer memory are used (no multicast, no TMA on peer memory).
    """

    def __init__(self, num_tokens: int, heads: int, world: int, rank: int, device: torch.device | str = "cuda", group=None) -> None:
        import os

        # plain peer mappings only: this path never uses NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        from nano_omni_b200 import _lib
        from nano_omni_b200.kernels.dense_bf16 import choose_kv_splits, splitkv_workspace_bytes

        if heads % world or num_tokens % world or world > 8:
            raise ValueError(f"tokens ({num_tokens}) and heads ({heads}) must be divisible by the world size ({world} <= 8)")
        self.num_tokens, self.heads, self.world, self.rank = num_tokens, heads, world, rank
        self.group = group
        self.local_tokens, self.local_heads = num_tokens // world, heads // world
        slab = num_tokens * self.local_heads * 256  # one tensor, all sources: [world, local_tokens, local_heads, 128] bf16
        self.recv_bytes = 3 * slab
        self.out_bytes = self.local_tokens * heads * 256
        self.flag_offset = self.recv_bytes + self.out_bytes
        total = self.flag_offset + 256
        self.buffer = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buffer[self.flag_offset :].zero_()
        torch.cuda.synchronize()
        self.handle = symm_mem.rendezvous(self.buffer, group if group is not None else dist.group.WORLD)
        bases = [int(p) for p in self.handle.buffer_ptrs]
        assert bases[rank] == self.buffer.data_ptr()
        table = ctypes.c_void_p * world
        self.peer_recv = table(*bases)
        self.peer_out = table(*[b + self.recv_bytes for b in bases])
        self.peer_flags = table(*[b + self.flag_offset for b in bases])
        recv = self.buffer[: self.recv_bytes].view(torch.bfloat16).view(3, num_tokens, self.local_heads, 128)
        self.q, self.k, self.v = recv[0], recv[1], recv[2]
        self.out_local = self.buffer[self.recv_bytes : self.flag_offset].view(torch.bfloat16).view(self.local_tokens, heads, 128)
        self.kv_splits = choose_kv_splits(num_tokens, self.local_heads)
        need = splitkv_workspace_bytes(num_tokens, self.local_heads, self.kv_splits)
        self.workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
        self.workspace_bytes = need
        self.epoch = 0
        self.launches_per_step = 4 + (1 if self.kv_splits > 1 else 0)  # push, 2 barriers, attention (+ merge)
        self._lib = _lib
        self._push = _lib.symbol("nob200_ulysses_push_heads")
        self._barrier = _lib.symbol("nob200_ulysses_barrier")
        self._attend = _lib.symbol("nob200_dense_bf16_attention_d128_scatter")
        dist.barrier(group)  # every rank has zeroed its flags before anyone signals

    def _check(self, code: int) -> None:
        if code:
            raise RuntimeError(self._lib.last_error())

    def check_status(self) -> None:
        """Synchronise and raise if a bounded device-side wait gave up during the steps since the last call.

        A cross-rank barrier that ran out (a peer more than the wait budget late: ``nob200_set_wait_budget_ns``,
        2 s by default) sets bit 16 of the device status word; the scatter epilogues then store nothing into the
        peers' tensors, so the step's output is incomplete on every rank.  Callers that cannot rule such a skew
        out call this after a step (it costs a stream synchronisation), or construct the plan with
        ``verify=True`` to have every step checked.
        """
        status = self._lib.read_status()
        if status:
            raise RuntimeError(f"Ulysses step invalid: device status {status:#x} (16 = a rank missed the barrier)")

    def barrier(self) -> None:
        self.epoch += 1
        self._check(
            self._barrier(self.peer_flags, ctypes.c_int(self.world), ctypes.c_int(self.rank), ctypes.c_uint(self.epoch),
                          ctypes.c_void_p(self._lib.current_stream()))
        )

    def dense_bf16(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor) -> None:
        lib = self._lib
        for t in (q, k, v, out):
            assert t.shape == (self.local_tokens, self.heads, 128) and t.is_contiguous()
        stream = ctypes.c_void_p(lib.current_stream())
        self._check(
            self._push(lib.ptr(q), lib.ptr(k), lib.ptr(v), self.peer_recv, ctypes.c_int(self.local_tokens),
                       ctypes.c_int(self.heads), ctypes.c_int(self.world), ctypes.c_int(self.rank), stream)
        )
        self.barrier()  # every rank's rows have landed here
        self._check(
            self._attend(
                ctypes.c_int(self.num_tokens), ctypes.c_int(self.rank * self.local_heads), lib.ptr(self.q), lib.ptr(self.k),
                lib.ptr(self.v), self.peer_out, ctypes.c_int(self.world), ctypes.c_int(self.local_heads),
                ctypes.c_int(self.heads), ctypes.c_int(self.kv_splits), lib.ptr(self.workspace),
                ctypes.c_size_t(self.workspace_bytes), stream,
            )
        )
        self.barrier()  # every rank's output rows have landed here; peers are done reading our pushes
        out.copy_(self.out_local)

    def _prepare_groups(self, groups: int) -> None:
        """Streams, events, receive areas and split-KV scratch of the pipelined dense path with ``groups`` head groups."""
        from nano_omni_b200.kernels.dense_bf16 import choose_kv_splits, splitkv_workspace_bytes

        if self.local_heads % groups:
            raise ValueError(f"{self.local_heads} heads per rank do not divide into {groups} groups")
        hg = self.local_heads // groups
        dev = self.buffer.device
        region = 3 * self.num_tokens * hg * 256  # one group's receive area: [3, world, local_tokens, hg, 128] bf16
        table = ctypes.c_void_p * self.world
        bases = [int(p) for p in self.handle.buffer_ptrs]
        splits = choose_kv_splits(self.num_tokens, hg)
        need = splitkv_workspace_bytes(self.num_tokens, hg, splits)
        self._groups = {
            "count": groups,
            "heads": hg,
            "splits": splits,
            "peer_recv": [table(*[b + g * region for b in bases]) for g in range(groups)],
            "recv": [
                self.buffer[g * region : (g + 1) * region].view(torch.bfloat16).view(3, self.num_tokens, hg, 128)
                for g in range(groups)
            ],
            "workspace": [torch.empty(max(need, 1), dtype=torch.uint8, device=dev) for _ in range(groups)],
            "workspace_bytes": need,
            "push_stream": torch.cuda.Stream(device=dev),
            "attend_stream": torch.cuda.Stream(device=dev),
            "landed": [torch.cuda.Event() for _ in range(groups)],
            "start": torch.cuda.Event(),
            "side_done": torch.cuda.Event(),
        }
        self.launches_per_step = 2 * groups + 1 + groups * (2 if splits > 1 else 1)  # pushes, barriers, attention (+ merge)

    def dense_bf16_pipelined(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, groups: int) -> None:
        """``dense_bf16`` with the reshard hidden behind the attention: the local heads are divided into ``groups``
        groups; group g + 1 is pushed and its arrival awaited on a second stream while group g is attended, and
        consecutive groups' attention kernels run on two streams so that one fills the SMs the other's last wave
        leaves idle.  The receive area holds the groups one after the other, each as tight [3, tokens, heads, 128]
        tensors.  Results equal ``dense_bf16``'s (same kernels per head)."""
        lib = self._lib
        for t in (q, k, v, out):
            assert t.shape == (self.local_tokens, self.heads, 128) and t.is_contiguous()
        if getattr(self, "_groups", None) is None or self._groups["count"] != groups:
            self._prepare_groups(groups)
        G = self._groups
        ci = ctypes.c_int
        main = torch.cuda.current_stream()
        push_stream, side = G["push_stream"], G["attend_stream"]
        push = lib.symbol("nob200_ulysses_push_head_group")
        G["start"].record(main)  # q, k, v are ready; the previous step's final barrier has been enqueued
        push_stream.wait_event(G["start"])
        with torch.cuda.stream(push_stream):
            for g in range(groups):
                self._check(
                    push(lib.ptr(q), lib.ptr(k), lib.ptr(v), G["peer_recv"][g], ci(self.local_tokens), ci(self.heads),
                         ci(self.world), ci(self.rank), ci(g * G["heads"]), ci(G["heads"]),
                         ctypes.c_void_p(push_stream.cuda_stream))
                )
                self.barrier()  # group g of every rank has landed here
                G["landed"][g].record(push_stream)
        side.wait_event(G["start"])
        for g in range(groups):
            stream = main if g % 2 == 0 else side
            stream.wait_event(G["landed"][g])
            recv = G["recv"][g]
            with torch.cuda.stream(stream):
                self._check(
                    self._attend(
                        ci(self.num_tokens), ci(self.rank * self.local_heads + g * G["heads"]), lib.ptr(recv[0]),
                        lib.ptr(recv[1]), lib.ptr(recv[2]), self.peer_out, ci(self.world), ci(G["heads"]), ci(self.heads),
                        ci(G["splits"]), lib.ptr(G["workspace"][g]), ctypes.c_size_t(G["workspace_bytes"]),
                        ctypes.c_void_p(stream.cuda_stream),
                    )
                )
        G["side_done"].record(side)
        main.wait_event(G["side_done"])
        self.barrier()  # every rank's output rows have landed here; peers are done reading our pushes
        out.copy_(self.out_local)


    def _prepare_int8(self) -> None:
        """Buffers and kernel calls of ``dense_int8_fp8``: quantisers on the local token shard (all heads), the layout
        of the quantised operands inside the receive area (all tokens, this rank's heads), the local attention."""
        from nano_omni_b200.core import TensorDesc
        from nano_omni_b200.kernels import quantize as qz
        from nano_omni_b200.kernels.dense_int8_fp8 import DenseInt8Fp8AttentionArguments, DenseInt8Fp8AttentionKernel

        T, Tl, H, lh = self.num_tokens, self.local_tokens, self.heads, self.local_heads
        if Tl % 256:
            raise ValueError(f"{Tl} tokens per rank: the quantised reshard needs a multiple of 256 (whole scale blocks, 16-byte rows)")
        dev = self.buffer.device
        desc = TensorDesc.from_torch
        new = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=dev)  # noqa: E731
        # quantised shard, head-major as the quantisers write it
        I = {
            "mean_local": new((1, H * 128), torch.float32),
            "means": new((self.world, H * 128), torch.float32),
            "mean": new((1, H * 128), torch.float32),
            "q8": new((H, Tl, 128), torch.int8),
            "qs": new((H, Tl // 32), torch.float32),
            "k8": new((H, Tl, 128), torch.int8),
            "ks": new((H, Tl // 64), torch.float32),
            "v8": new((H, 128, Tl), torch.float8_e4m3fn),
            "vs": new((H, 128), torch.float32),
            "attended": new((T, lh * 128), torch.bfloat16),
        }
        need = qz.TokenGroupMeanKernel.workspace_bytes(
            qz.TokenGroupMeanWorkload(num_tokens=Tl, columns=H * 128, tokens_per_block=Tl, include_padding=False)
        )
        I["partial"] = new((max(need, 1),), torch.uint8)
        # receive area: Q8 [lh, T, 128] | K8 [lh, T, 128] | V8 [lh, 128, T] | Q scales [lh, T / 32] | K scales [lh, T / 64]
        n8 = lh * T * 128
        offsets = {"q8": 0, "k8": n8, "v8": 2 * n8, "qs": 3 * n8, "ks": 3 * n8 + lh * (T // 32) * 4}
        assert offsets["ks"] + lh * (T // 64) * 4 <= self.recv_bytes
        bases = [int(p) for p in self.handle.buffer_ptrs]
        table = ctypes.c_void_p * self.world
        I["peer"] = {name: table(*[b + off for b in bases]) for name, off in offsets.items()}
        area = self.buffer
        view = lambda name, nbytes, dtype, shape: area[offsets[name] : offsets[name] + nbytes].view(dtype).view(shape)  # noqa: E731
        R = {
            "q8": view("q8", n8, torch.int8, (lh, T, 128)),
            "k8": view("k8", n8, torch.int8, (lh, T, 128)),
            "v8": view("v8", n8, torch.float8_e4m3fn, (lh, 128, T)),
            "qs": view("qs", lh * (T // 32) * 4, torch.float32, (lh, T // 32)),
            "ks": view("ks", lh * (T // 64) * 4, torch.float32, (lh, T // 64)),
        }
        I["recv"] = R
        I["vs_mine"] = new((lh, 128), torch.float32)
        I["attend"] = DenseInt8Fp8AttentionKernel(
            DenseInt8Fp8AttentionArguments(
                desc(R["q8"]), desc(R["k8"]), desc(R["v8"]), desc(R["qs"]), desc(R["ks"]), desc(I["vs_mine"]),
                desc(I["attended"]), T, lh, T, 32, 64,
            )
        )
        # (rows, row bytes, head stride, pitch, offset of this rank's tokens) of each pushed tensor
        r = self.rank
        I["moves"] = {
            "q8": (Tl, 128, T * 128, 128, r * Tl * 128),
            "k8": (Tl, 128, T * 128, 128, r * Tl * 128),
            "v8": (128, Tl, 128 * T, T, r * Tl),
            "qs": (1, Tl // 8, T // 8, T // 8, r * Tl // 8),
            "ks": (1, Tl // 16, T // 16, T // 16, r * Tl // 16),
        }
        I["qz"] = qz
        self._int8 = I

    def dense_int8_fp8(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor) -> None:
        """Dense int8-QK / fp8-PV attention on sequence-sharded bf16 input, quantised BEFORE the exchange: every rank
        quantises its token shard for all heads, the int8 / e4m3 bytes and their scales (3.2 bytes per element of
        Q, K, V instead of 6) are stored into the peers' receive areas, and the attended rows go back to their owners.

        The two statistics that span the whole sequence are agreed first: the per-channel K mean (the ranks' shard
        means are gathered and averaged in rank order on every rank, so all ranks centre with identical bits; the
        summation order differs from one GPU's, so a centred value that sits on a rounding boundary may quantise one
        step apart) and the per-channel V scale (maximum over the ranks' scales: exact, the scale is monotonic in
        the absolute maximum).  Q bytes and scales, V bytes and scales equal the single-GPU quantisers' bit for bit."""
        from nano_omni_b200.core import TensorDesc

        lib = self._lib
        for t in (q, k, v, out):
            assert t.shape == (self.local_tokens, self.heads, 128) and t.is_contiguous()
        if getattr(self, "_int8", None) is None:
            self._prepare_int8()
        I = self._int8
        qz = I["qz"]
        Tl, H, lh, T = self.local_tokens, self.heads, self.local_heads, self.num_tokens
        desc = TensorDesc.from_torch
        flat = lambda t: desc(t.view(Tl, H * 128))  # noqa: E731
        # statistics over the whole sequence
        qz.TokenGroupMeanKernel(qz.TokenGroupMeanArguments(flat(k), desc(I["mean_local"]), Tl, False, desc(I["partial"]))).submit()
        dist.all_gather_into_tensor(I["means"], I["mean_local"], group=self.group)
        mean = I["means"][0].clone()
        for r in range(1, self.world):
            mean += I["means"][r]
        I["mean"].copy_((mean / self.world).view(1, -1))
        qz.Int8Fp8ValueScaleKernel(qz.Int8Fp8ValueScaleArguments(flat(v), desc(I["vs"]), H)).submit()
        dist.all_reduce(I["vs"], op=dist.ReduceOp.MAX, group=self.group)
        I["vs_mine"].copy_(I["vs"][self.rank * lh : (self.rank + 1) * lh])
        # quantise the shard
        qz.Int8Fp8QuantizeQKKernel(qz.Int8Fp8QuantizeQKArguments(flat(q), desc(I["mean"]), desc(I["q8"]), desc(I["qs"]), H, 32, False)).submit()
        qz.Int8Fp8QuantizeQKKernel(qz.Int8Fp8QuantizeQKArguments(flat(k), desc(I["mean"]), desc(I["k8"]), desc(I["ks"]), H, 64, True)).submit()
        qz.Int8Fp8QuantizeValueKernel(qz.Int8Fp8QuantizeValueArguments(flat(v), desc(I["vs"]), desc(I["v8"]), H)).submit()
        # exchange bytes and scales
        stream = ctypes.c_void_p(lib.current_stream())
        push = lib.symbol("nob200_ulysses_push_blocks")
        ll = ctypes.c_longlong
        for name, (rows, row_bytes, head_stride, pitch, offset) in I["moves"].items():
            self._check(
                push(lib.ptr(I[name]), I["peer"][name], ctypes.c_int(H), ctypes.c_int(self.world), ctypes.c_int(rows),
                     ll(row_bytes), ll(head_stride), ll(pitch), ll(offset), stream)
            )
        self.barrier()  # every rank's bytes have landed here
        I["attend"].submit(stream.value)
        self._check(
            lib.symbol("nob200_ulysses_push_output")(
                lib.ptr(I["attended"]), self.peer_out, ctypes.c_int(T), ctypes.c_int(lh), ctypes.c_int(H),
                ctypes.c_int(self.world), ctypes.c_int(self.rank), stream,
            )
        )
        self.barrier()  # every rank's output rows have landed here; peers are done reading our pushes
        out.copy_(self.out_local)

    def sol_bf16(
        self,
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        out: torch.Tensor,
        num_protected_blocks: int,
        tau: float = 1.0,
        block: int = 128,
        topk_fraction: float = 0.0,
    ) -> torch.Tensor:
        """sol block-sparse attention on sequence-sharded input.  Routing (pool, stats, select) runs
        after the reshard, per head on the full sequence, so the masks equal the single-GPU masks.
        Returns this rank's mask u8 [blocks, heads/world, blocks]."""
        import math

        lib = self._lib
        nb = -(-self.num_tokens // block)
        lh = self.local_heads
        key = (block, topk_fraction > 0)
        if getattr(self, "_sol_key", None) != key:
            dev = self.buffer.device
            self._sol_key = key
            self._pooled = torch.empty(2, lh, nb, 128, dtype=torch.bfloat16, device=dev)
            self._stats = torch.empty(lh, 2, 128, device=dev)
            self._mask = torch.empty(nb, lh, nb, dtype=torch.uint8, device=dev)
            self._scores = torch.empty(nb * nb * lh * 4 if topk_fraction > 0 else 1, dtype=torch.uint8, device=dev)
        stream = ctypes.c_void_p(lib.current_stream())
        ci = ctypes.c_int
        self._check(
            self._push(lib.ptr(q), lib.ptr(k), lib.ptr(v), self.peer_recv, ci(self.local_tokens), ci(self.heads),
                       ci(self.world), ci(self.rank), stream)
        )
        self.barrier()
        self._check(
            lib.symbol("nob200_sol_pool")(ci(self.num_tokens), lib.ptr(self.k), lib.ptr(self.v), ctypes.c_void_p(0),
                                          lib.ptr(self._pooled), ci(lh), ci(block), stream)
        )
        self._check(lib.symbol("nob200_sol_stats")(lib.ptr(self._pooled), lib.ptr(self._stats), ci(lh), ci(nb), stream))
        topk_blocks = min(nb, math.ceil(topk_fraction * nb)) if topk_fraction > 0 else 0
        self._check(
            lib.symbol("nob200_sol_select")(
                ci(self.num_tokens), ci(num_protected_blocks), lib.ptr(self.q), lib.ptr(self._pooled), lib.ptr(self._stats),
                lib.ptr(self._mask), ci(lh), ctypes.c_float(tau), ci(block), ci(topk_blocks), lib.ptr(self._scores),
                ctypes.c_size_t(self._scores.numel()), stream,
            )
        )
        self._check(
            lib.symbol("nob200_sol_attention_d128_scatter")(
                ci(self.num_tokens), ci(self.rank * lh), lib.ptr(self.q), lib.ptr(self.k), lib.ptr(self.v),
                lib.ptr(self._pooled), lib.ptr(self._mask), self.peer_out, ci(self.world), ci(lh), ci(self.heads),
                ci(block), ci(2), stream,
            )
        )
        self.barrier()
        out.copy_(self.out_local)
        return self._mask

    def sol_quantised(self, q, k, v, out, precision: str, protected_tokens: int, tau: float = 1.0) -> None:
        """int8-fp8 or nvfp4 sol attention on sequence-sharded input: push reshard, then this rank's heads go through the
        single-GPU operator (quantisers, pools, statistics, router, exact stage) into a local numerator, and the finalize
        kernel stores every output row into its owner's tensor."""
        from nano_omni_b200 import ops
        from nano_omni_b200.core import TensorDesc

        lib = self._lib
        lh, T = self.local_heads, self.num_tokens
        key = ("quantised", precision, protected_tokens, tau)
        if getattr(self, "_sol_key", None) != key:
            self._sol_key = key
            dev = self.buffer.device
            self._attended = torch.empty(T, lh, 128, dtype=torch.bfloat16, device=dev)
            flat = lambda t: TensorDesc.from_torch(t.view(T, lh * 128))  # noqa: E731
            cls = ops.ATTENTION_OPS[("sol", precision)]
            op = cls(flat(self.q), flat(self.k), flat(self.v), total_heads=lh, protected_tokens=protected_tokens, tau=tau)
            op.to(TensorDesc.from_torch(self._attended))
            self._scratch = torch.empty(op.prepare()[1] + 256, dtype=torch.uint8, device=dev)
            base = self._scratch.data_ptr() + (-self._scratch.data_ptr()) % 256
            self._calls = op.bind(base)
        stream = ctypes.c_void_p(lib.current_stream())
        ci = ctypes.c_int
        self._check(
            self._push(lib.ptr(q), lib.ptr(k), lib.ptr(v), self.peer_recv, ci(self.local_tokens), ci(self.heads),
                       ci(self.world), ci(self.rank), stream)
        )
        self.barrier()
        for call in self._calls[:-1]:
            call.submit(stream.value)
        final = self._calls[-1].arguments  # finalize: query, pooled, selected, exact, state, output, head_offset
        self._check(
            lib.symbol("nob200_sol_nvfp4_finalize_scatter")(
                ci(T), ci(self.rank * lh), lib.ptr(final.query), lib.ptr(final.pooled), lib.ptr(final.selected),
                lib.ptr(final.exact), lib.ptr(final.state), self.peer_out, ci(self.world), ci(lh), ci(self.heads), ci(64), stream,
            )
        )
        self.barrier()
        out.copy_(self.out_local)


def make_plan(
    num_tokens: int,
    heads: int,
    world: int,
    rank: int,
    device: torch.device | str = "cuda",
    transport: str = "auto",
    group=None,
    p2p_factory=None,
    nccl_factory=None,
):
    """``p2p`` (peer-memory stores), ``nccl`` (batched NCCL point-to-point), or ``auto``: p2p when EVERY rank
    can map the others' memory, NCCL otherwise.  Returns (plan, transport used).

    With ``auto`` the ranks agree before anyone uses a plan: each reports whether its peer-memory plan could
    be built and the minimum over the group decides, so a rank whose symmetric allocation or rendezvous failed
    cannot end up on NCCL while the others wait for it at the flag barrier.  ``p2p_factory`` / ``nccl_factory``
    replace the constructors of the two plans (tests inject a failing one and CPU stand-ins).
    """
    p2p_factory = p2p_factory or (lambda: UlyssesAttentionP2P(num_tokens, heads, world, rank, device, group))
    nccl_factory = nccl_factory or (lambda: UlyssesAttention(num_tokens, heads, world, rank, device, group=group))
    if transport == "p2p":
        return p2p_factory(), "p2p"
    if transport == "auto":
        try:
            plan = p2p_factory()
        except Exception:
            plan = None
        if world > 1:
            on_gpu = dist.get_backend(group) == "nccl"
            mine = torch.tensor([0 if plan is None else 1], dtype=torch.int32, device=device if on_gpu else "cpu")
            dist.all_reduce(mine, op=dist.ReduceOp.MIN, group=group)
            if int(mine.item()) == 0:
                plan = None  # some rank could not: everybody takes the collective path
        if plan is not None:
            return plan, "p2p"
    return nccl_factory(), "nccl"
