"""Tensor-pipe peaks of this GPU for the operand kinds of the attention kernels.

    python -m nano_omni_b200.peaks

Launches ``nob200_mma_issue_rate`` (one CTA per SM, back-to-back ``tcgen05.mma`` 128 x 128 x K from shared memory)
for bf16, int8, e4m3 and block-scaled nvfp4, times each launch with CUDA events and prints one JSON line: T(FL)OP/s over all SMs,
SM cycles per MMA, and the SM clock implied by cycles / time.  The bf16 figure can be read against the library GEMM
peak in ``MEASURED_PEAKS.json``; the int8 / fp8 / nvfp4 figures are the denominators for those precisions.
"""

from __future__ import annotations

import ctypes
import json

import torch

from nano_omni_b200 import _lib

KINDS = {"bf16": (0, 16), "int8": (1, 32), "fp8_e4m3": (2, 32), "nvfp4_block_scaled": (3, 64)}


def measure(count: int = 1 << 16, repeats: int = 3) -> dict:
    torch.cuda.set_device(0)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    cycles = torch.zeros(sms, dtype=torch.int64, device="cuda")
    function = _lib.symbol("nob200_mma_issue_rate")
    stream = ctypes.c_void_p(_lib.current_stream())
    result = {"sms": sms, "mmas_per_cta": count}
    for name, (kind, k) in KINDS.items():
        best = None
        for _ in range(repeats + 1):  # first launch is the warm-up
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            code = function(ctypes.c_int(kind), ctypes.c_int(count), ctypes.c_int(sms), _lib.ptr(cycles), stream)
            stop.record()
            if code != 0:
                raise RuntimeError(_lib.last_error())
            torch.cuda.synchronize()
            ms = start.elapsed_time(stop)
            best = ms if best is None else min(best, ms)
        if _lib.read_status() or int(cycles.min()) < 0:
            raise RuntimeError("a bounded wait gave up")
        worst = int(cycles.max())
        ops = 2 * 128 * 128 * k * count * sms
        result[name] = {
            "tera_ops_per_s": ops / (best * 1e-3) / 1e12,
            "cycles_per_mma": worst / count,
            "sm_mhz_implied": worst / (best * 1e-3) / 1e6,
            "ms": best,
        }
    return result


PIPE_OPS = {"ex2": 0, "cvt_e4m3x2": 1, "cvt_e2m1x2": 2, "cvt_bf16x2": 3, "fma": 4, "max3": 5, "integer_add": 6}


def measure_pipes(iters: int = 2000) -> dict:
    """Lanes per clock and SM of the softmax warps' instruction kinds, for 1, 2 and 4 warps per scheduler
    (``nob200_pipe_issue_rate``: 16 independent instructions per round).  The exponential's 16 lanes per clock are
    what bounds the attention kernels beside the tensor pipe: 128 x 128 scores cost 1024 cycles of one SM's MUFU."""
    torch.cuda.set_device(0)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    cycles = torch.zeros(sms * 32, dtype=torch.int64, device="cuda")
    sink = torch.zeros(1024, device="cuda")
    function = _lib.symbol("nob200_pipe_issue_rate")
    stream = ctypes.c_void_p(_lib.current_stream())
    result = {"sms": sms, "rounds_of_16": iters}
    for name, op in PIPE_OPS.items():
        row = {}
        for warps in (4, 8, 16):
            for _ in range(2):  # the first launch is the warm-up
                code = function(ctypes.c_int(op), ctypes.c_int(warps), ctypes.c_int(iters), ctypes.c_int(sms),
                                _lib.ptr(cycles), _lib.ptr(sink), stream)
                if code != 0:
                    raise RuntimeError(_lib.last_error())
                torch.cuda.synchronize()
            worst = int(cycles[:warps].max())  # warps of CTA 0
            per_scheduler = worst / (iters * 16) / (warps / 4)  # cycles per warp instruction on one scheduler
            row[f"{warps // 4}_warps_per_scheduler"] = {
                "cycles_per_warp_instruction": round(per_scheduler, 3),
                "lanes_per_clock_per_sm": round(128 / per_scheduler, 1),
            }
        result[name] = row
    return result


if __name__ == "__main__":
    import sys

    print(json.dumps(measure_pipes() if "--pipes" in sys.argv else measure()))
