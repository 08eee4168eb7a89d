"""Generate golden vectors by running the UNMODIFIED reference ``ref_program``s on CPU.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/nano-omni

It imports the reference package from ``<reference>/src``, points its tensor
descriptors at CPU torch tensors (the reference's ``TensorDesc.as_torch`` only
builds CUDA views) and redirects ``device="cuda"`` in the few ``ref_program``s
that hard-code it, then stores seeded inputs and the reference outputs as
``tests/golden/*.npz``.  The fixtures travel with the repository; this script
does not need to run again unless cases are added.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def to_numpy(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().copy()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def install_cpu_backend():
    """Make reference descriptors resolve to CPU tensors."""
    from nano_omni.core import tensor as ref_tensor

    registry: dict[int, torch.Tensor] = {}
    counter = [1 << 20]

    def desc(dtype, value: torch.Tensor):
        key = counter[0]
        counter[0] += 1 << 20
        registry[key] = value
        return ref_tensor.TensorDesc(dtype, tuple(value.shape), ref_tensor.TensorKind.DEVICE, (key, 0))

    def as_torch(self):
        return registry[self.info[0]]

    ref_tensor.TensorDesc.as_torch = as_torch

    # ref_programs that say device="cuda" (sol pool/select/int8 sol): build on CPU instead
    for name in ("full", "arange", "tensor", "zeros", "ones", "empty"):
        original = getattr(torch, name)

        def wrapped(*args, _original=original, **kwargs):
            if kwargs.get("device") == "cuda":
                kwargs["device"] = "cpu"
            return _original(*args, **kwargs)

        setattr(torch, name, wrapped)
    return desc


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="path of the nano-omni checkout")
    args = parser.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    desc = install_cpu_backend()

    from nano_omni.core.tensor import DType
    from nano_omni.kernels.attention.dense_bf16 import DenseBf16AttentionArguments, DenseBf16AttentionKernel
    from nano_omni.kernels.attention.dense_nvfp4 import DenseNvfp4Arguments, DenseNvfp4Kernel
    from nano_omni.kernels.attention.int8_fp8.dense import (
        DenseInt8Fp8AttentionArguments,
        DenseInt8Fp8AttentionKernel,
    )
    from nano_omni.kernels.attention.int8_fp8.quantize_qk import (
        Int8Fp8QuantizeQKArguments,
        Int8Fp8QuantizeQKKernel,
    )
    from nano_omni.kernels.attention.int8_fp8.quantize_value import (
        Int8Fp8QuantizeValueArguments,
        Int8Fp8QuantizeValueKernel,
    )
    from nano_omni.kernels.attention.int8_fp8.value_scale import (
        Int8Fp8ValueScaleArguments,
        Int8Fp8ValueScaleKernel,
    )
    from nano_omni.kernels.attention.nvfp4_prepare import Nvfp4PrepareArguments, Nvfp4PrepareKernel
    from nano_omni.kernels.normalization.token_group_mean import (
        TokenGroupMeanArguments,
        TokenGroupMeanKernel,
    )
    from nano_omni.kernels.quantization.quantize_fp4 import QuantizeFp4Arguments, QuantizeFp4Kernel

    def randn(seed, *shape, outlier=False):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(*shape, generator=g)
        if outlier:
            x[..., 5] *= 16
        return x.bfloat16()

    out: dict[str, np.ndarray] = {}

    for T, h in ((130, 2), (500, 3)):
        tag = f"T{T}_h{h}"
        src = randn(T * 7 + h, T, h * 128, outlier=True)
        out[f"src_{tag}"] = to_numpy(src)

        # column mean over all tokens (the K-centring vector) and over 64-token groups
        for tpb, pad in ((T, False), (64, False), (64, True)):
            nb = -(-T // tpb)
            res = torch.empty(nb, h * 128)
            TokenGroupMeanKernel.ref_program(
                TokenGroupMeanArguments(desc(DType.BF16, src), desc(DType.F32, res), tpb, pad)
            )
            out[f"mean_{tag}_tpb{tpb}_pad{int(pad)}"] = to_numpy(res)
        mean = torch.from_numpy(out[f"mean_{tag}_tpb{T}_pad0"]).clone()

        for tpb, center in ((32, False), (64, True), (128, True)):
            padded = -(-T // tpb) * tpb
            q = torch.empty(h, padded, 128, dtype=torch.int8)
            s = torch.empty(h, padded // tpb)
            # the reference program rejects 128 only inside the TileLang body; its ref_program is generic
            Int8Fp8QuantizeQKKernel.ref_program(
                Int8Fp8QuantizeQKArguments(
                    desc(DType.BF16, src), desc(DType.F32, mean), desc(DType.I8, q), desc(DType.F32, s), h, tpb, center
                )
            )
            out[f"qk_q_{tag}_tpb{tpb}_c{int(center)}"] = to_numpy(q)
            out[f"qk_s_{tag}_tpb{tpb}_c{int(center)}"] = to_numpy(s)

        vs = torch.empty(h, 128)
        Int8Fp8ValueScaleKernel.ref_program(Int8Fp8ValueScaleArguments(desc(DType.BF16, src), desc(DType.F32, vs), h))
        out[f"vscale_{tag}"] = to_numpy(vs)
        padded64 = -(-T // 64) * 64
        v8 = torch.empty(h, 128, padded64, dtype=torch.float8_e4m3fn)
        Int8Fp8QuantizeValueKernel.ref_program(
            Int8Fp8QuantizeValueArguments(desc(DType.BF16, src), desc(DType.F32, vs), desc(DType.FP8_E4M3, v8), h)
        )
        out[f"v8_{tag}"] = to_numpy(v8)

        padded128 = -(-T // 128) * 128
        mean_h = mean.reshape(h, 128).contiguous()
        for transpose in (False, True):
            for center in (False, True):
                rows, cols = (128, padded128) if transpose else (padded128, 128)
                packed = torch.empty(h, rows, cols // 2, dtype=torch.uint8)
                sf = torch.empty(h, rows, cols // 16, dtype=torch.float8_e4m3fn)
                Nvfp4PrepareKernel.ref_program(
                    Nvfp4PrepareArguments(
                        desc(DType.BF16, src),
                        desc(DType.F32, mean_h) if center else None,
                        desc(DType.U8, packed),
                        desc(DType.FP8_UE4M3, sf),
                        h,
                        transpose,
                    )
                )
                out[f"fp4_q_{tag}_t{int(transpose)}_c{int(center)}"] = to_numpy(packed)
                out[f"fp4_s_{tag}_t{int(transpose)}_c{int(center)}"] = to_numpy(sf)

    # global-scale NVFP4 arithmetic (linear-layer quantiser), one head-sized matrix
    T = 130
    src = randn(99, T, 128)
    out["gfp4_src"] = to_numpy(src)
    gscale = torch.tensor([0.75])
    packed = torch.empty(T, 64, dtype=torch.uint8)
    sf = torch.empty(256, 8, dtype=torch.float8_e4m3fn)
    QuantizeFp4Kernel.ref_program(
        QuantizeFp4Arguments(
            desc(DType.BF16, src), None, None, desc(DType.U8, packed), desc(DType.FP8_UE4M3, sf), desc(DType.F32, gscale)
        )
    )
    out["gfp4_q"] = to_numpy(packed)
    out["gfp4_s"] = to_numpy(sf)

    # attention outputs
    T, h = 200, 2
    q, k, v = (randn(1000 + i, T, h, 128) for i in range(3))
    for name, t in (("q", q), ("k", k), ("v", v)):
        out[f"att_{name}"] = to_numpy(t)
    o = torch.zeros(T, 3, 128, dtype=torch.bfloat16)
    DenseBf16AttentionKernel.ref_program(
        DenseBf16AttentionArguments(*(desc(DType.BF16, t) for t in (q, k, v)), desc(DType.BF16, o), 1)
    )
    out["att_bf16_out"] = to_numpy(o)

    # int8-fp8 attention on quantised operands produced by the reference quantisers
    def flat(t):
        return t.reshape(T, h * 128).contiguous()

    kmean = torch.empty(1, h * 128)
    TokenGroupMeanKernel.ref_program(TokenGroupMeanArguments(desc(DType.BF16, flat(k)), desc(DType.F32, kmean), T, False))
    q8 = torch.empty(h, -(-T // 32) * 32, 128, dtype=torch.int8)
    qs = torch.empty(h, -(-T // 32))
    k8 = torch.empty(h, -(-T // 64) * 64, 128, dtype=torch.int8)
    ks = torch.empty(h, -(-T // 64))
    Int8Fp8QuantizeQKKernel.ref_program(
        Int8Fp8QuantizeQKArguments(
            desc(DType.BF16, flat(q)), desc(DType.F32, kmean), desc(DType.I8, q8), desc(DType.F32, qs), h, 32, False
        )
    )
    Int8Fp8QuantizeQKKernel.ref_program(
        Int8Fp8QuantizeQKArguments(
            desc(DType.BF16, flat(k)), desc(DType.F32, kmean), desc(DType.I8, k8), desc(DType.F32, ks), h, 64, True
        )
    )
    vs = torch.empty(h, 128)
    Int8Fp8ValueScaleKernel.ref_program(Int8Fp8ValueScaleArguments(desc(DType.BF16, flat(v)), desc(DType.F32, vs), h))
    v8 = torch.empty(h, 128, -(-T // 64) * 64, dtype=torch.float8_e4m3fn)
    Int8Fp8QuantizeValueKernel.ref_program(
        Int8Fp8QuantizeValueArguments(desc(DType.BF16, flat(v)), desc(DType.F32, vs), desc(DType.FP8_E4M3, v8), h)
    )
    o8 = torch.zeros(T, h * 128, dtype=torch.bfloat16)
    DenseInt8Fp8AttentionKernel.ref_program(
        DenseInt8Fp8AttentionArguments(
            desc(DType.I8, q8),
            desc(DType.I8, k8),
            desc(DType.FP8_E4M3, v8),
            desc(DType.F32, qs),
            desc(DType.F32, ks),
            desc(DType.F32, vs),
            desc(DType.BF16, o8),
            T,
            h,
            T,
        )
    )
    out["att_int8_out"] = to_numpy(o8)

    # nvfp4 attention on operands from the reference nvfp4 quantiser
    P = -(-T // 128) * 128
    kmean_h = kmean.reshape(h, 128).contiguous()

    def prep(t, mean, transpose):
        rows, cols = (128, P) if transpose else (P, 128)
        packed = torch.empty(h, rows, cols // 2, dtype=torch.uint8)
        sf = torch.empty(h, rows, cols // 16, dtype=torch.float8_e4m3fn)
        Nvfp4PrepareKernel.ref_program(
            Nvfp4PrepareArguments(
                desc(DType.BF16, flat(t)),
                desc(DType.F32, mean) if mean is not None else None,
                desc(DType.U8, packed),
                desc(DType.FP8_UE4M3, sf),
                h,
                transpose,
            )
        )
        return packed, sf

    q4, qsf = prep(q, None, False)
    k4, ksf = prep(k, kmean_h, False)
    v4, vsf = prep(v, None, True)
    o4 = torch.zeros(T, h, 128, dtype=torch.bfloat16)
    DenseNvfp4Kernel.ref_program(
        DenseNvfp4Arguments(
            desc(DType.U8, q4),
            desc(DType.U8, k4),
            desc(DType.U8, v4),
            desc(DType.FP8_UE4M3, qsf),
            desc(DType.FP8_UE4M3, ksf),
            desc(DType.FP8_UE4M3, vsf),
            desc(DType.BF16, o4),
            T,
            T,
            0,
        )
    )
    out["att_nvfp4_out"] = to_numpy(o4)

    path = os.path.join(HERE, "dense_path.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1e6:.2f} MB")
    make_sol(desc, randn)
    make_norm_rope(desc, randn)
    make_matmul(desc)


def make_sol(desc, randn) -> None:
    """Fixtures of the sol routing path: pooling, statistics, routing mask, fused bf16 attention."""
    from nano_omni.core.tensor import DType
    from nano_omni.kernels.attention.int8_fp8.sol_pool import SolInt8Fp8PoolArguments, SolInt8Fp8PoolKernel
    from nano_omni.kernels.attention.nvfp4.sol_select import SolNvfp4SelectArguments, SolNvfp4SelectKernel
    from nano_omni.kernels.attention.sol.pool import SolPoolArguments, SolPoolKernel
    from nano_omni.kernels.attention.sol.stats import SolStatsArguments, SolStatsKernel
    from nano_omni.kernels.attention.sol_attention import SolAttentionArguments, SolAttentionKernel

    out: dict[str, np.ndarray] = {}
    for T, h, protected in ((300, 2, 1), (1000, 2, 2)):
        tag = f"T{T}_h{h}"
        nb = -(-T // 64)
        q, k, v = (randn(5000 + T + i, T, h, 128) for i in range(3))
        # give the keys block structure so that routing selects a non-trivial subset
        g = torch.Generator().manual_seed(T)
        centres = torch.randn(nb, h, 128, generator=g) * 1.5
        k = (k.float() + centres.repeat_interleave(64, dim=0)[:T]).bfloat16()
        for name, t in (("q", q), ("k", k), ("v", v)):
            out[f"{name}_{tag}"] = to_numpy(t)
        pooled = torch.empty(2, h, nb, 128, dtype=torch.bfloat16)
        SolPoolKernel.ref_program(SolPoolArguments(desc(DType.BF16, k), desc(DType.BF16, v), desc(DType.BF16, pooled)))
        out[f"pooled_{tag}"] = to_numpy(pooled)
        kmean = k.float().mean(0).contiguous()  # [h, 128]
        out[f"kmean_{tag}"] = to_numpy(kmean)
        pooled3 = torch.empty(3, h, nb, 128, dtype=torch.bfloat16)
        SolInt8Fp8PoolKernel.ref_program(
            SolInt8Fp8PoolArguments(desc(DType.BF16, k), desc(DType.BF16, v), desc(DType.F32, kmean), desc(DType.BF16, pooled3))
        )
        out[f"pooled3_{tag}"] = to_numpy(pooled3)
        stats = torch.empty(h, 2, 128)
        SolStatsKernel.ref_program(SolStatsArguments(desc(DType.BF16, pooled), desc(DType.F32, stats)))
        out[f"stats_{tag}"] = to_numpy(stats)
        mask = torch.empty(nb, h, nb, dtype=torch.uint8)
        SolNvfp4SelectKernel.ref_program(
            SolNvfp4SelectArguments(
                desc(DType.BF16, q), desc(DType.BF16, pooled[0].contiguous()), desc(DType.F32, stats), desc(DType.U8, mask), 1.0, protected
            )
        )
        out[f"mask_{tag}"] = to_numpy(mask)
        o = torch.zeros(T, h, 128, dtype=torch.bfloat16)
        SolAttentionKernel.ref_program(
            SolAttentionArguments(
                desc(DType.BF16, q), desc(DType.BF16, k), desc(DType.BF16, v), desc(DType.BF16, pooled), desc(DType.F32, stats),
                desc(DType.BF16, o), 1.0, 0, protected,
            )
        )
        out[f"sol_out_{tag}"] = to_numpy(o)
        out[f"protected_{tag}"] = np.array(protected)
    make_sol_quantised(desc, randn, out)
    path = os.path.join(HERE, "sol_path.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1e6:.2f} MB")



def make_sol_quantised(desc, randn, out) -> None:
    """int8-fp8 and nvfp4 sol: reference exact stage (numerator + state) followed by the shared finalize."""
    from nano_omni.core.tensor import DType
    from nano_omni.kernels.attention.int8_fp8.quantize_qk import Int8Fp8QuantizeQKArguments, Int8Fp8QuantizeQKKernel
    from nano_omni.kernels.attention.int8_fp8.quantize_value import (
        Int8Fp8QuantizeValueArguments,
        Int8Fp8QuantizeValueKernel,
    )
    from nano_omni.kernels.attention.int8_fp8.sol import SolInt8Fp8AttentionArguments, SolInt8Fp8AttentionKernel
    from nano_omni.kernels.attention.int8_fp8.sol_pool import SolInt8Fp8PoolArguments, SolInt8Fp8PoolKernel
    from nano_omni.kernels.attention.int8_fp8.value_scale import Int8Fp8ValueScaleArguments, Int8Fp8ValueScaleKernel
    from nano_omni.kernels.attention.nvfp4.sol_finalize import SolNvfp4FinalizeArguments, SolNvfp4FinalizeKernel
    from nano_omni.kernels.attention.nvfp4.sol_select import SolNvfp4SelectArguments, SolNvfp4SelectKernel
    from nano_omni.kernels.attention.nvfp4_prepare import Nvfp4PrepareArguments, Nvfp4PrepareKernel
    from nano_omni.kernels.attention.sol.stats import SolStatsArguments, SolStatsKernel
    from nano_omni.kernels.attention.sol_nvfp4 import SolNvfp4Arguments, SolNvfp4Kernel
    from nano_omni.kernels.normalization.token_group_mean import TokenGroupMeanArguments, TokenGroupMeanKernel

    T, h, protected = 300, 2, 1
    tag = f"T{T}_h{h}"
    nb = -(-T // 64)
    q, k, v = (bf16_from(out[f"{n}_{tag}"]) for n in "qkv")
    flat = lambda t: t.reshape(T, h * 128).contiguous()  # noqa: E731
    kmean = torch.empty(1, h * 128)
    TokenGroupMeanKernel.ref_program(TokenGroupMeanArguments(desc(DType.BF16, flat(k)), desc(DType.F32, kmean), T, False))
    kmean_h = kmean.reshape(h, 128).contiguous()
    pooled3 = torch.empty(3, h, nb, 128, dtype=torch.bfloat16)
    SolInt8Fp8PoolKernel.ref_program(
        SolInt8Fp8PoolArguments(desc(DType.BF16, k), desc(DType.BF16, v), desc(DType.F32, kmean_h), desc(DType.BF16, pooled3))
    )
    stats = torch.empty(h, 2, 128)
    # statistics and routing read plane 0 (the uncentred block means), as the reference op binds them
    SolStatsKernel.ref_program(SolStatsArguments(desc(DType.BF16, pooled3[0:2].contiguous()), desc(DType.F32, stats)))
    mask = torch.empty(nb, h, nb, dtype=torch.uint8)
    SolNvfp4SelectKernel.ref_program(
        SolNvfp4SelectArguments(
            desc(DType.BF16, q), desc(DType.BF16, pooled3[0].contiguous()), desc(DType.F32, stats), desc(DType.U8, mask), 1.0, protected
        )
    )
    out[f"q_kmean_{tag}"] = to_numpy(kmean)
    out[f"q_pooled3_{tag}"] = to_numpy(pooled3)
    out[f"q_stats_{tag}"] = to_numpy(stats)
    out[f"q_mask_{tag}"] = to_numpy(mask)

    # ---- int8-fp8
    q8 = torch.empty(h, -(-T // 32) * 32, 128, dtype=torch.int8)
    qs = torch.empty(h, -(-T // 32))
    k8 = torch.empty(h, nb * 64, 128, dtype=torch.int8)
    ks = torch.empty(h, nb)
    Int8Fp8QuantizeQKKernel.ref_program(
        Int8Fp8QuantizeQKArguments(desc(DType.BF16, flat(q)), desc(DType.F32, kmean), desc(DType.I8, q8), desc(DType.F32, qs), h, 32, False)
    )
    Int8Fp8QuantizeQKKernel.ref_program(
        Int8Fp8QuantizeQKArguments(desc(DType.BF16, flat(k)), desc(DType.F32, kmean), desc(DType.I8, k8), desc(DType.F32, ks), h, 64, True)
    )
    vs = torch.empty(h, 128)
    Int8Fp8ValueScaleKernel.ref_program(Int8Fp8ValueScaleArguments(desc(DType.BF16, flat(v)), desc(DType.F32, vs), h))
    v8 = torch.empty(h, 128, nb * 64, dtype=torch.float8_e4m3fn)
    Int8Fp8QuantizeValueKernel.ref_program(
        Int8Fp8QuantizeValueArguments(desc(DType.BF16, flat(v)), desc(DType.F32, vs), desc(DType.FP8_E4M3, v8), h)
    )
    exact = torch.zeros(T, h, 128, dtype=torch.bfloat16)
    state = torch.zeros(T, h, 2)
    SolInt8Fp8AttentionKernel.ref_program(
        SolInt8Fp8AttentionArguments(
            desc(DType.I8, q8), desc(DType.I8, k8), desc(DType.FP8_E4M3, v8), desc(DType.F32, qs), desc(DType.F32, ks),
            desc(DType.F32, vs), desc(DType.U8, mask), desc(DType.BF16, exact), desc(DType.F32, state), T, 0, 1.0, protected,
        )
    )
    out[f"i8_exact_{tag}"] = to_numpy(exact)
    out[f"i8_state_{tag}"] = to_numpy(state)
    final = torch.zeros(T, h, 128, dtype=torch.bfloat16)
    SolNvfp4FinalizeKernel.ref_program(
        SolNvfp4FinalizeArguments(
            desc(DType.BF16, q), desc(DType.BF16, pooled3), desc(DType.U8, mask), desc(DType.BF16, exact), desc(DType.F32, state),
            desc(DType.BF16, final), 0,
        )
    )
    out[f"i8_final_{tag}"] = to_numpy(final)

    # ---- nvfp4
    P = -(-T // 128) * 128

    def prep(t, mean, transpose):
        rows, cols = (128, P) if transpose else (P, 128)
        packed = torch.empty(h, rows, cols // 2, dtype=torch.uint8)
        sf = torch.empty(h, rows, cols // 16, dtype=torch.float8_e4m3fn)
        Nvfp4PrepareKernel.ref_program(
            Nvfp4PrepareArguments(
                desc(DType.BF16, flat(t)), desc(DType.F32, mean) if mean is not None else None, desc(DType.U8, packed),
                desc(DType.FP8_UE4M3, sf), h, transpose,
            )
        )
        return packed, sf

    q4, qsf = prep(q, None, False)
    k4, ksf = prep(k, kmean_h, False)
    v4, vsf = prep(v, None, True)
    exact4 = torch.zeros(T, h, 128, dtype=torch.bfloat16)
    state4 = torch.zeros(T, h, 2)
    SolNvfp4Kernel.ref_program(
        SolNvfp4Arguments(
            desc(DType.U8, q4), desc(DType.U8, k4), desc(DType.U8, v4), desc(DType.FP8_UE4M3, qsf), desc(DType.FP8_UE4M3, ksf),
            desc(DType.FP8_UE4M3, vsf), desc(DType.U8, mask), desc(DType.BF16, exact4), desc(DType.F32, state4), T, T, 0, 1.0,
            protected,
        )
    )
    out[f"f4_exact_{tag}"] = to_numpy(exact4)
    out[f"f4_state_{tag}"] = to_numpy(state4)
    final4 = torch.zeros(T, h, 128, dtype=torch.bfloat16)
    SolNvfp4FinalizeKernel.ref_program(
        SolNvfp4FinalizeArguments(
            desc(DType.BF16, q), desc(DType.BF16, pooled3), desc(DType.U8, mask), desc(DType.BF16, exact4), desc(DType.F32, state4),
            desc(DType.BF16, final4), 0,
        )
    )
    out[f"f4_final_{tag}"] = to_numpy(final4)


def bf16_from(array):
    return torch.from_numpy(array.copy()).view(torch.bfloat16)


def make_norm_rope(desc, randn) -> None:
    """Per-head RMS norm + split-half RoPE, alone and fused with the int8 query quantiser."""
    from nano_omni.core.tensor import DType
    from nano_omni.kernels.specialized.h3_head_norm_rope import H3HeadNormRopeArguments, H3HeadNormRopeKernel
    from nano_omni.kernels.specialized.h3_query_prepare import H3QueryPrepareArguments, H3QueryPrepareKernel

    out: dict[str, np.ndarray] = {}
    T, h = 130, 3
    g = torch.Generator().manual_seed(77)
    source = (torch.randn(T, h, 128, generator=g) * 2).bfloat16()
    weight = (1 + 0.1 * torch.randn(128, generator=g)).bfloat16()
    angle = torch.rand(T, 48, generator=g) * 6.2831853
    cosines, sines = torch.cos(angle).contiguous(), torch.sin(angle).contiguous()
    out["source"], out["weight"] = to_numpy(source), to_numpy(weight)
    out["cosines"], out["sines"] = to_numpy(cosines), to_numpy(sines)
    for rope in (False, True):
        result = torch.empty(T, h, 128, dtype=torch.bfloat16)
        H3HeadNormRopeKernel.ref_program(
            H3HeadNormRopeArguments(
                desc(DType.BF16, source), desc(DType.BF16, weight), desc(DType.F32, cosines) if rope else None,
                desc(DType.F32, sines) if rope else None, desc(DType.BF16, result),
            )
        )
        out[f"head_norm_rope_{int(rope)}"] = to_numpy(result)
        rows = -(-T // 32) * 32
        q8 = torch.empty(h, rows, 128, dtype=torch.int8)
        scales = torch.empty(h, rows // 32)
        H3QueryPrepareKernel.ref_program(
            H3QueryPrepareArguments(
                desc(DType.BF16, source.reshape(T, h * 128)), desc(DType.BF16, weight),
                desc(DType.F32, cosines) if rope else None, desc(DType.F32, sines) if rope else None,
                desc(DType.I8, q8), desc(DType.F32, scales),
            )
        )
        out[f"query_q_{int(rope)}"] = to_numpy(q8)
        out[f"query_s_{int(rope)}"] = to_numpy(scales)
    # row-wise int8 of the projection inputs, plain and with the 256-column group rotation
    from nano_omni.kernels.quantization.convrot_int8 import ConvRotInt8Arguments, ConvRotInt8Kernel
    from nano_omni.kernels.quantization.int8_rowwise import Int8RowwiseArguments, Int8RowwiseKernel

    rows, columns = 37, 768
    activations = (torch.randn(rows, columns, generator=g) * 1.7).bfloat16()
    activations[:, 300] *= 9
    out["rowwise_src"] = to_numpy(activations)
    for name, kernel, arguments in (
        ("rowwise", Int8RowwiseKernel, Int8RowwiseArguments),
        ("convrot", ConvRotInt8Kernel, ConvRotInt8Arguments),
    ):
        q8 = torch.empty(rows, columns, dtype=torch.int8)
        sc = torch.empty(rows)
        kernel.ref_program(arguments(desc(DType.BF16, activations), desc(DType.I8, q8), desc(DType.F32, sc)))
        out[f"{name}_q"], out[f"{name}_s"] = to_numpy(q8), to_numpy(sc)
    path = os.path.join(HERE, "norm_rope.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1e6:.2f} MB")


def make_matmul(desc) -> None:
    """The projection GEMMs with their fused epilogues: int8 (scales) and bf16 (output scale)."""
    from nano_omni.core.tensor import DType
    from nano_omni.kernels.matmul.matmul_bf16 import MatmulBf16Arguments, MatmulBf16Kernel
    from nano_omni.kernels.matmul.matmul_int8 import MatmulInt8Arguments, MatmulInt8Kernel

    out: dict[str, np.ndarray] = {}
    g = torch.Generator().manual_seed(91)
    M, N, K = 37, 40, 144
    x8 = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    w8 = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    ws = (torch.rand(N, 1, generator=g) * 2e-4 + 1e-5).contiguous()
    xs = (torch.rand(M, generator=g) * 0.05 + 0.001).contiguous()
    xb = torch.randn(M, K, generator=g).bfloat16()
    wb = (torch.randn(N, K, generator=g) * K**-0.5).bfloat16()
    bias = (torch.randn(N, generator=g) * 0.5).bfloat16()
    residual = torch.randn(M, N, generator=g).bfloat16()
    multiply = torch.randn(M, N, generator=g).bfloat16()
    for name, tensor in (("x8", x8), ("w8", w8), ("ws", ws), ("xs", xs), ("xb", xb), ("wb", wb), ("bias", bias),
                         ("residual", residual), ("multiply", multiply)):  # fmt: skip
        out[name] = to_numpy(tensor)
    bf = lambda t: desc(DType.BF16, t)  # noqa: E731
    for tag, (b, r, m, silu) in {"plain": (None, None, None, False), "bias_res": (bias, residual, None, False),
                                 "all": (bias, residual, multiply, True)}.items():  # fmt: skip
        opt = lambda t: bf(t) if t is not None else None  # noqa: E731
        result = torch.empty(M, N, dtype=torch.bfloat16)
        MatmulInt8Kernel.ref_program(
            MatmulInt8Arguments(desc(DType.I8, x8), desc(DType.I8, w8), opt(b), opt(r), opt(m), bf(result),
                                desc(DType.F32, ws), desc(DType.F32, xs), silu)
        )  # fmt: skip
        out[f"int8_{tag}"] = to_numpy(result)
        result = torch.empty(M, N, dtype=torch.bfloat16)
        MatmulBf16Kernel.ref_program(MatmulBf16Arguments(bf(xb), bf(wb), opt(b), opt(r), opt(m), bf(result), 0.75, silu))
        out[f"bf16_{tag}"] = to_numpy(result)
    path = os.path.join(HERE, "matmul.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
