"""Headline benchmark: dense bf16 DiT attention, S=32768, 24 heads, head_dim 128.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One "step" is one pass of the attention hot path over one batch of synthetic
Q/K/V (seed 1, N(0,1) bf16, 1 % of K's channels x16, 512 text + 32256 video
tokens).  At N=1 the whole problem runs on one GPU.  At N>1 the sequence is
sharded over the ranks, resharded to heads by an NCCL all-to-all, attended
locally and resharded back (both exchanges inside the timed region); the
problem size is fixed, so scaling is "strong".

Rank 0 prints ONE JSON line.  `value` is whole-job attention TFLOP/s with the
inputs resident in HBM; `e2e` is the same metric through the public Kernel API
starting from pinned host buffers (H2D of Q/K/V and D2H of O inside the timed
region); `roofline` rates the attention kernel against the measured bf16
tensor peak; `cpu_baseline` times the CPU oracle (fp32 SDPA) on a bounded
sample.  `--impl reference` times that CPU path alone, with all host threads.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SEQ, HEADS, DIM = 32768, 24, 128
TEXT_TOKENS = 512
WORKLOAD = "dense_bf16_attention S=32768 (512 text + 32256 video) H=24 D=128 batch 1, non-causal"
FALLBACK_BF16_TFLOPS = 1590.0
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of a kernel from an ncu capture, with the
# shape it was captured at; a launch at another shape is scaled by tokens x heads (traffic grows in proportion
# because K and V of a head stay in L2 while its query tiles are processed).
NCU_TRAFFIC = {
    "fa_fwd_bf16_kernel": {"bytes": 201.97e6 + 49.16e6, "tokens": 16384, "heads": 16},
}
# Issue-rate peaks of tcgen05.mma per operand kind on this GPU (`python -m nano_omni_b200.peaks`: back-to-back
# 128 x 128 x K MMAs on all SMs, T(FL)OP/s at the clock of a short burst), the denominators for the precisions that
# have no library GEMM figure.
ISSUE_RATE_PEAKS = {"bf16": 2227.0, "int8_fp8": (4575.0 + 4449.0) / 2, "nvfp4": 8908.0}


def ncu_traffic(kernel: str, tokens: int, heads: int) -> int | None:
    entry = NCU_TRAFFIC.get(kernel)
    if entry is None:
        return None
    return int(entry["bytes"] * (tokens * heads) / (entry["tokens"] * entry["heads"]))


def attention_flops(heads: int, tq: int, tk: int) -> int:
    return 4 * heads * tq * tk * DIM


def make_inputs(seq: int, heads: int, seed: int = 1):
    """Config-2 recipe: N(0,1) bf16; one of the 128 K channels (1 %) per head multiplied by 16."""
    import torch

    g = torch.Generator().manual_seed(seed)
    q = torch.randn(seq, heads, DIM, generator=g).bfloat16()
    k = torch.randn(seq, heads, DIM, generator=g)
    v = torch.randn(seq, heads, DIM, generator=g).bfloat16()
    channel = torch.randint(0, DIM, (heads,), generator=g)
    k[:, torch.arange(heads), channel] *= 16
    return q, k.bfloat16(), v


def peak_bf16_tflops() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except Exception:
        return FALLBACK_BF16_TFLOPS, "fallback"


def sustained_bf16_tflops() -> float | None:
    """The library GEMM's rate in a seconds-long loop under the power cap (the state the timed steps run in)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _loop(self) -> None:
        nv = self._nvml
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        s = sorted(self.samples)
        return {
            "sm_mhz": s[len(s) // 2] if s else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(s),
        }


class CpuSdpaSample:
    """The CPU oracle (fp32 SDPA) on `heads` x `queries` rows against all SEQ keys."""

    def __init__(self, heads: int, queries: int, threads: int) -> None:
        import torch

        from oracle import reference_math as rm

        torch.set_num_threads(threads)
        g = torch.Generator().manual_seed(1)
        self.rm = rm
        self.heads, self.queries, self.threads = heads, queries, threads
        self.q = torch.randn(queries, heads, DIM, generator=g).bfloat16()
        self.k = torch.randn(SEQ, heads, DIM, generator=g).bfloat16()
        self.v = torch.randn(SEQ, heads, DIM, generator=g).bfloat16()
        self.flops = attention_flops(heads, queries, SEQ)
        self.text = f"{heads} heads x {queries} queries x {SEQ} keys per pass, fp32 SDPA (torch CPU oracle)"

    def once(self) -> float:
        t0 = time.perf_counter()
        self.rm.dense_attention_fp32(self.q, self.k, self.v)
        return time.perf_counter() - t0


def run_reference(args) -> None:
    """The reference arm: the reference math for this path on the host cores (CPU oracle)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample = CpuSdpaSample(2, 2048, threads)
    for _ in range(max(args.warmup, 1)):
        sample.once()
    elapsed = sum(sample.once() for _ in range(args.steps))
    value = sample.flops * args.steps / elapsed / 1e12
    line = {
        "impl": "reference",
        "metric": "dit_attention_tflops",
        "value": value,
        "unit": "TFLOP/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample.text},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample.text},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


_INPUT_CACHE: dict = {}


def device_inputs(seq: int, seed: int):
    """Q, K, V of the benchmark recipe on the GPU; one set is kept so that workloads of one shape share it."""
    key = (seq, seed)
    if key not in _INPUT_CACHE:
        _INPUT_CACHE.clear()
        _INPUT_CACHE[key] = tuple(t.cuda() for t in make_inputs(seq, HEADS, seed=seed))
    return _INPUT_CACHE[key]


def measure_workload(workload: str, steps: int, warmup: int, seq: int = 0) -> dict:
    """Single-GPU timing of one precision / routing through its operator of ``nano_omni_b200.ops``.

    ``value`` counts preparation (quantisers or pooling + routing) and attention, ``attention_only_tflops`` the
    attention kernels alone.  The quantised sol workloads run the reference's chain (threshold routing over
    64-token blocks, exact stage with state, finalize).
    """
    import torch

    from nano_omni_b200 import _lib, ops
    from nano_omni_b200.core import TensorDesc

    torch.cuda.set_device(0)
    sol_case = workload.startswith("sol_")
    seq = seq or (131072 if sol_case else SEQ)
    q, k, v = device_inputs(seq, 2 if sol_case else 1)
    flat = lambda t: t.view(seq, HEADS * DIM)  # noqa: E731
    out = torch.empty(seq, HEADS, DIM, dtype=torch.bfloat16, device="cuda")
    stream = _lib.current_stream()
    note = {}
    if workload == "dense_bf16":
        op = ops.DenseBf16Attention(*(TensorDesc.from_torch(flat(t)) for t in (q, k, v)), total_heads=HEADS)
    elif workload == "sol_bf16":
        # the benchmark's sol configuration: 128-token blocks, top 25 % of key blocks per query block, 512 text tokens
        op = ops.SolAttention(
            *(TensorDesc.from_torch(flat(t)) for t in (q, k, v)), total_heads=HEADS, protected_tokens=512,
            block=128, topk_fraction=0.25,
        )  # fmt: skip
        note = {"block": 128, "topk_fraction": 0.25, "protected_tokens": 512}
    else:
        extra = {"protected_tokens": 512} if sol_case else {}
        # "_rotated": the operands quantised as the benchmark states them (Walsh-Hadamard rotation; int8 scales per
        # 128 tokens; one global NVFP4 scale per tensor)
        rotated = workload.endswith("_rotated")
        kind, precision = workload.removesuffix("_rotated").split("_", 1)
        cls = ops.ATTENTION_OPS[(kind, precision)]
        if cls is ops.DenseInt8Fp8Attention:
            op = cls(*(TensorDesc.from_torch(flat(t)) for t in (q, k, v)), hadamard=rotated)
            out = out.view(seq, HEADS * DIM)
        elif rotated:
            from nano_omni_b200.kernels.quantize import hadamard128_rows

            scales = tuple(float(hadamard128_rows(t.clone()).abs().max()) / (6 * 448) for t in (q, k, v))
            op = cls(*(TensorDesc.from_torch(flat(t)) for t in (q, k, v)), total_heads=HEADS, global_scales=scales)
            note = {"global_scales": scales}
        else:
            op = cls(*(TensorDesc.from_torch(flat(t)) for t in (q, k, v)), total_heads=HEADS, **extra)
        if sol_case:
            note = {"block": 64, "routing": "threshold tau=1", "protected_tokens": 512}
    op.to(TensorDesc.from_torch(out))
    _, scratch_bytes = op.prepare()
    scratch = torch.empty(scratch_bytes + 256, dtype=torch.uint8, device="cuda")
    base = scratch.data_ptr() + (-scratch.data_ptr()) % 256
    calls = op.bind(base)
    attention_names = {
        "dense_bf16_attention_d128", "dense_int8_fp8_d128", "dense_nvfp4_attention_d128", "sol_attention_d128",
        "sol_int8_fp8_attention_d128", "sol_nvfp4_attention_d128", "sol_nvfp4_finalize",
    }  # fmt: skip
    attention = [c for c in calls if type(c).name in attention_names]
    prepare = [c for c in calls if type(c).name not in attention_names]

    def timed(kernels, count):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(count):
            for kernel in kernels:
                kernel.submit(stream)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / count

    for _ in range(warmup):
        for kernel in calls:
            kernel.submit(stream)
    torch.cuda.synchronize()
    if _lib.read_status():
        raise RuntimeError("device status set during warm-up")
    with ClockSampler(0) as clocks:
        ms_all = timed(calls, steps)
        ms_att = timed(attention, steps)
        ms_prep = timed(prepare, steps) if prepare else 0.0
    if _lib.read_status():
        raise RuntimeError("device status set during the timed region")
    flops = attention_flops(HEADS, seq, seq)
    peak, which = peak_bf16_tflops()
    if sol_case:
        mask = next(c.arguments.mask if hasattr(c.arguments, "mask") else c.arguments.selected for c in attention)
        nb = mask.shape[0]
        at = mask.data_ptr() - scratch.data_ptr()
        selected = float(scratch[at : at + mask.num_bytes].float().mean())
        note["selected_fraction"] = selected
        note["blocks"] = nb
    return {
        "metric": "dit_attention_tflops",
        "value": flops / (ms_all * 1e-3) / 1e12,
        "unit": "TFLOP/s (dense-equivalent flops 4*H*S*S*128 over prepare + attention time)",
        "n_gpus": 1,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": ms_all,
        "ms_attention": ms_att,
        "ms_prepare": ms_prep,
        "attention_only_tflops": flops / (ms_att * 1e-3) / 1e12,
        "higher_is_better": True,
        "data": "synthetic",
        "config": {"workload": workload, "seq_len": seq, "heads": HEADS, "head_dim": DIM, **note},
        "kernels": [type(c).name for c in calls],
        "gpu_launches": len(calls) * steps,
        "scratch_bytes": scratch_bytes,
        "peak_bf16_tflops": peak,
        "peak_source": which,
        "clocks": clocks.summary(),
    }


def run_other_workload(args) -> None:
    """One of the other configurations alone, in the headline's JSON shape."""
    assert args.gpus == 1, "the extra workloads are single-GPU measurements"
    print(json.dumps(measure_workload(args.workload, args.steps, args.warmup, args.seq)))


def extra_workloads(steps: int, warmup: int) -> dict:
    """The other precisions and the sol routing, measured in the same process after the headline: dense int8-fp8 and
    nvfp4 at the headline shape (with bf16 through the same operator path as their reference), sol bf16 / int8-fp8 /
    nvfp4 at S = 131072.  Per workload: time with and without the preparation kernels, throughput in dense-equivalent
    flops, the ratio to bf16 (attention kernels only, same shape), and the attention kernels' rate against the
    tcgen05 issue-rate peak of their operand kind."""
    import torch

    out: dict = {}
    reference_ms: dict[int, float] = {}
    for workload in ("dense_bf16", "dense_int8_fp8", "dense_nvfp4", "sol_bf16", "sol_int8_fp8", "sol_nvfp4"):
        m = measure_workload(workload, steps, warmup)
        seq = m["config"]["seq_len"]
        precision = workload.split("_", 1)[1]
        if workload == "dense_bf16":
            reference_ms[seq] = m["ms_attention"]
        entry = {
            "seq_len": seq,
            "ms_per_step": m["ms_per_step"],
            "ms_attention": m["ms_attention"],
            "ms_prepare": m["ms_prepare"],
            "tflops": m["value"],
            "attention_only_tflops": m["attention_only_tflops"],
            "kernels": m["kernels"],
            "clocks": m["clocks"],
        }
        if workload.startswith("dense_"):
            entry["ratio_to_bf16"] = reference_ms[seq] / m["ms_attention"]
            peak = ISSUE_RATE_PEAKS[precision]
            entry["roofline"] = {
                "bound": "tensor", "achieved": m["attention_only_tflops"], "peak": peak, "unit": "T(FL)OP/s",
                "frac": m["attention_only_tflops"] / peak, "peak_source": "tcgen05 issue rate of this operand kind",
            }  # fmt: skip
        else:
            entry["selected_fraction"] = m["config"].get("selected_fraction")
            entry["routing"] = {k: m["config"][k] for k in ("block", "topk_fraction", "routing") if k in m["config"]}
            # dense bf16 at this length is 16 x the headline's work; its time is extrapolated from the headline shape
            entry["speedup_over_dense_bf16_extrapolated"] = reference_ms[SEQ] * (seq / SEQ) ** 2 / m["ms_attention"]
        out[workload] = entry
    _INPUT_CACHE.clear()
    torch.cuda.empty_cache()
    return out


def run_sol_distributed(args) -> None:
    """sol attention on sequence-sharded input over N GPUs: push reshard, routing per head on the full sequence,
    block-sparse attention whose epilogue scatters the rows to their owners.  bf16: 128-token blocks, top 25 %;
    int8-fp8 / nvfp4: the reference's chain (64-token blocks, threshold routing, exact stage + finalize).
    Also the dense int8-fp8 path that quantises on the token shards before the exchange (S = 32768 by default).
    Strong scaling."""
    import torch
    import torch.distributed as dist

    from nano_omni_b200 import _lib, ulysses

    world, rank, local_rank = (int(os.environ[k]) for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"))
    assert world == args.gpus
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    seq = args.seq or (SEQ if args.workload == "dense_int8_fp8" else 131072)
    assert HEADS % world == 0 and seq % (world * 256) == 0
    shard = seq // world
    q, k, v = (t[rank * shard : (rank + 1) * shard].contiguous().cuda() for t in make_inputs(seq, HEADS, seed=2))
    out = torch.empty(shard, HEADS, DIM, dtype=torch.bfloat16, device="cuda")
    plan, transport = ulysses.make_plan(seq, HEADS, world, rank, transport=os.environ.get("NOB200_ULYSSES", "auto"))
    assert hasattr(plan, "sol_bf16"), "the sol path needs the peer-memory transport"

    if args.workload == "dense_int8_fp8":
        routing = {"exchange": "int8 / e4m3 bytes and scales, quantised on the token shards; K mean gathered, V scale max-reduced"}

        def step():
            plan.dense_int8_fp8(q, k, v, out)
    elif args.workload == "sol_bf16":
        routing = {"block": 128, "topk_fraction": 0.25}

        def step():
            plan.sol_bf16(q, k, v, out, TEXT_TOKENS // 128, block=128, topk_fraction=0.25)
    else:
        precision = args.workload.split("_", 1)[1]
        routing = {"block": 64, "routing": "threshold tau=1"}
        assert hasattr(plan, "sol_quantised")

        def step():
            plan.sol_quantised(q, k, v, out, precision, TEXT_TOKENS)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    assert _lib.read_status() == 0
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        barrier()
    assert _lib.read_status() == 0
    t = torch.tensor([start.elapsed_time(stop)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    if rank == 0:
        flops = attention_flops(HEADS, seq, seq)
        print(
            json.dumps(
                {
                    "metric": "dit_attention_tflops",
                    "value": flops * args.steps / (total_ms * 1e-3) / 1e12,
                    "unit": "TFLOP/s (dense-equivalent flops 4*H*S*S*128 over reshard + routing + attention time)",
                    "n_gpus": world,
                    "steps": args.steps,
                    "warmup": args.warmup,
                    "ms_per_step": total_ms / args.steps,
                    "higher_is_better": True,
                    "scaling": "strong",
                    "data": "synthetic",
                    "config": {"workload": args.workload, "seq_len": seq, "heads": HEADS, "head_dim": DIM, **routing,
                               "protected_tokens": TEXT_TOKENS, "transport": transport,
                               "parallelism": f"ulysses{world}"},
                    "clocks": clocks.summary(),
                }
            )
        )  # fmt: skip
    dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument(
        "--workload",
        default="dense_bf16",
        choices=["dense_bf16", "dense_int8_fp8", "dense_nvfp4", "sol_bf16", "sol_int8_fp8", "sol_nvfp4",
                 "dense_int8_fp8_rotated", "dense_nvfp4_rotated"],
        help="dense_bf16 is the headline configuration (its line also carries the others under `extra`); naming "
        "another one measures it alone in the same format",
    )
    parser.add_argument("--seq", type=int, default=0, help="sequence length override (a multiple of 256 x gpus)")
    parser.add_argument("--no-extra", action="store_true", help="skip the other precisions / sol workloads (N=1 only)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
        return
    if (args.workload.startswith("sol_") or args.workload == "dense_int8_fp8") and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        run_sol_distributed(args)
        return
    if args.workload != "dense_bf16":
        run_other_workload(args)
        return

    import torch

    from nano_omni_b200 import _lib
    from nano_omni_b200.core import TensorDesc
    from nano_omni_b200.kernels.dense_bf16 import DenseBf16AttentionArguments, DenseBf16AttentionKernel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    _lib.library()  # no fallback: fail here when the extension is missing
    desc = TensorDesc.from_torch
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        from nano_omni_b200 import ulysses

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    seq = args.seq or SEQ
    assert HEADS % world == 0 and seq % (world * 256) == 0, "sequence must be a multiple of 256 x gpus"
    workload_name = WORKLOAD if seq == SEQ else WORKLOAD.replace("S=32768 (512 text + 32256 video)", f"S={seq}")

    q_cpu, k_cpu, v_cpu = make_inputs(seq, HEADS)
    shard = seq // world
    lo, hi = rank * shard, (rank + 1) * shard
    q_host, k_host, v_host = (t[lo:hi].contiguous().pin_memory() for t in (q_cpu, k_cpu, v_cpu))
    del q_cpu, k_cpu, v_cpu
    q, k, v = (t.cuda(non_blocking=True) for t in (q_host, k_host, v_host))
    out = torch.empty(shard, HEADS, DIM, dtype=torch.bfloat16, device="cuda")
    out_host = torch.empty(shard, HEADS, DIM, dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream()

    if distributed:
        plan, transport = ulysses.make_plan(seq, HEADS, world, rank, transport=os.environ.get("NOB200_ULYSSES", "auto"))
        # NOB200_ULYSSES_GROUPS=g: push head group i + 1 while group i is attended (peer-memory transport only)
        groups = int(os.environ.get("NOB200_ULYSSES_GROUPS", "0")) if transport == "p2p" else 0
        if groups:
            plan._prepare_groups(groups)
        launches_per_step = plan.launches_per_step

        def step(qd, kd, vd, od):
            if groups:
                plan.dense_bf16_pipelined(qd, kd, vd, od, groups)
            else:
                plan.dense_bf16(qd, kd, vd, od)
    else:
        launches_per_step, groups = 1, 0

        def step(qd, kd, vd, od):
            DenseBf16AttentionKernel(DenseBf16AttentionArguments(desc(qd), desc(kd), desc(vd), desc(od), 0)).submit()

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for _ in range(args.warmup):
        step(q, k, v, out)
    barrier()
    assert _lib.read_status() == 0, "attention kernel reported a wait timeout during warm-up"
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        barrier()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for a, b in events:
            a.record(stream)
            step(q, k, v, out)
            b.record(stream)
        stop.record(stream)
        barrier()
    total_ms = start.elapsed_time(stop)
    kernel_ms = sum(a.elapsed_time(b) for a, b in events) / args.steps
    assert _lib.read_status() == 0, "attention kernel reported a wait timeout"

    # ---- end to end through the public API: pinned host -> device -> kernel -> pinned host, every step;
    # uploads, attention and downloads of consecutive steps overlap on three streams
    from nano_omni_b200.host_pipeline import HostAttentionPipeline

    pipeline = HostAttentionPipeline((shard, HEADS, DIM), step)
    e2e_steps = args.steps
    for _ in range(2):
        pipeline.submit(q_host, k_host, v_host, out_host)
    pipeline.finish()
    barrier()
    e2e_start = torch.cuda.Event(enable_timing=True)
    e2e_stop = torch.cuda.Event(enable_timing=True)
    e2e_start.record(pipeline.h2d)
    for _ in range(e2e_steps):
        pipeline.submit(q_host, k_host, v_host, out_host)
    pipeline.d2h.wait_stream(pipeline.compute)
    pipeline.d2h.wait_stream(pipeline.h2d)
    e2e_stop.record(pipeline.d2h)
    pipeline.finish()
    barrier()
    e2e_ms = e2e_start.elapsed_time(e2e_stop)

    if distributed:
        t = torch.tensor([total_ms, kernel_ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, kernel_ms, e2e_ms = t.tolist()

    check = None
    if distributed:
        # Results, not only speed: two heads of the sharded output against the single-GPU kernel on the gathered
        # operands, on rank 0.  A mismatch ends the run.
        heads_checked = 2
        gathered = []
        for t in (q, k, v):
            part = t[:, :heads_checked].contiguous()
            whole = torch.empty(seq, heads_checked, DIM, dtype=torch.bfloat16, device="cuda")
            dist.all_gather_into_tensor(whole, part)
            gathered.append(whole)
        if rank == 0:
            single = torch.empty(seq, heads_checked, DIM, dtype=torch.bfloat16, device="cuda")
            DenseBf16AttentionKernel(
                DenseBf16AttentionArguments(desc(gathered[0]), desc(gathered[1]), desc(gathered[2]), desc(single), 0)
            ).submit()
            torch.cuda.synchronize()
            mine = out[:, :heads_checked].float()
            want = single[lo:hi].float()
            worst = float((mine - want).abs().max())
            # the sharded run may split the keys differently (fewer heads per GPU): bf16 rounding of the shares
            if not torch.allclose(mine, want, rtol=2**-6, atol=2**-8):
                raise RuntimeError(f"sharded attention differs from the single-GPU kernel: max |diff| {worst}")
            check = {"rows": shard, "heads": heads_checked, "max_abs_diff_vs_single_gpu": worst}
        del gathered

    flops = attention_flops(HEADS, seq, seq)
    value = flops * args.steps / (total_ms * 1e-3) / 1e12
    e2e_value = flops * e2e_steps / (e2e_ms * 1e-3) / 1e12
    peak, peak_source = peak_bf16_tflops()
    per_gpu_flops = flops / world
    achieved = per_gpu_flops / (kernel_ms * 1e-3) / 1e12

    if rank == 0:
        line = {
            "metric": "dit_attention_tflops",
            "value": value,
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": workload_name,
                "seq_len": seq,
                "heads": HEADS,
                "head_dim": DIM,
                "text_tokens": TEXT_TOKENS,
                "parallelism": "single GPU" if world == 1 else f"ulysses seq<->head reshard x{world} over {transport}" + (f", {groups} head groups pipelined" if groups else ""),
                "l2": f"inputs ({3 * seq * HEADS * DIM * 2 // 1000000} MB) larger than L2; no flush",
                "flop_convention": "4*H*S*S*128",
            },
            "tflops_per_gpu": value / world,
            "e2e": {
                "value": e2e_value,
                "unit": "TFLOP/s",
                "h2d_bytes_per_step": 3 * q_host.numel() * 2 * world,
                "d2h_bytes_per_step": out_host.numel() * 2 * world,
                "steps": e2e_steps,
            },
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "roofline": {
                "bound": "tensor",
                "kernel": "fa_fwd_bf16_kernel" if world == 1 else "ulysses step (pack + all-to-all + fa_fwd_bf16_kernel)",
                "achieved": achieved,
                "peak": peak,
                "unit": "TFLOP/s",
                "frac": achieved / peak,
                "peak_source": peak_source,
                # for context: the same GEMM run back to back for seconds settles lower under the 1000 W cap, which is
                # also where the timed steps run (see "clocks")
                "frac_of_sustained_peak": (achieved / sustained_bf16_tflops()) if sustained_bf16_tflops() else None,
                # one GPU: the attention kernel's DRAM bytes (ncu, scaled to this shape); several: that kernel's
                # share plus the rows this rank sends and receives in the two reshards (3 inputs out, 1 output in)
                "traffic": ncu_traffic("fa_fwd_bf16_kernel", seq, HEADS)
                if world == 1
                else ncu_traffic("fa_fwd_bf16_kernel", seq, HEADS // world) + 4 * shard * HEADS * DIM * 2 * (world - 1) // world,
                "ms_per_launch": kernel_ms,
            },
        }
        if check is not None:
            line["check"] = check
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            sample = CpuSdpaSample(2, 4096, threads)
            sample.once()
            seconds = min(sample.once() for _ in range(3))
            line["cpu_baseline"] = {
                "value": sample.flops / seconds / 1e12,
                "unit": "TFLOP/s",
                "cores": threads,
                "kind": "port",
                "sample": f"{sample.text}, best of 3, {seconds:.2f} s per pass",
            }
        if world == 1 and not args.no_extra:
            del q, k, v, out, q_host, k_host, v_host, out_host, pipeline
            torch.cuda.empty_cache()
            line["extra"] = extra_workloads(steps=3, warmup=3)
        print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
