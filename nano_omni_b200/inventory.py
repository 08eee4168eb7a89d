"""Kernel inventory in the reference's CSV schema (scripts/update.py:49-60):

    model,kernel,percent,latency,launch,mem%,ncu%,tops,workload,config

    python -m nano_omni_b200.inventory --tokens 32768 --heads 24 > inventory.csv

Every kernel class of the registry is launched alone at the given shape on seeded random tensors
(``nano_omni_b200.tune``), timed with CUDA events, and reported with

* ``latency``  median milliseconds of one launch;
* ``percent``  its share of the sum over the listed kernels;
* ``mem%``     bytes of its tensor arguments (scratch excluded) / latency, as a percentage of the measured HBM
               copy bandwidth (``MEASURED_PEAKS.json`` ``hbm_gbs``, 6650 GB/s when the file is absent);
* ``tops``     ``Kernel.tops`` / latency in T(FL)OP/s, empty for kernels without tensor-core work;
* ``ncu%``     left empty: profiler captures are taken separately, one kernel at a time.
"""

from __future__ import annotations

import argparse
import csv
import json
import os
import sys

import torch

from nano_omni_b200 import kernels, tune
from nano_omni_b200.core import TensorDesc

FIELDS = ("model", "kernel", "percent", "latency", "launch", "mem%", "ncu%", "tops", "workload", "config")


def canonical(value) -> str:
    return json.dumps(value, sort_keys=True, separators=(",", ":"))


def workloads(tokens: int, heads: int) -> list[tuple[str, dict, dict]]:
    """(kernel name, Workload fields, tune options) of the attention path at one shape."""
    t, h = tokens, heads
    sparse = {"mask_density": 0.16}
    return [
        # the projections around attention at the reference's widths (model 5376, 56 heads x 128 = 7168)
        ("int8_rowwise", {"num_tokens": t, "columns": 5376}, {}),
        ("convrot_int8", {"num_tokens": t, "columns": 5376, "group": 256}, {}),
        ("matmul_int8", {"num_tokens": t, "n": 7168, "k": 5376}, {}),
        ("matmul_int8", {"num_tokens": t, "n": 5376, "k": 7168, "use_residual": True}, {}),
        # a LoRA pair of rank 64 beside the QKV projection: compress, then update through the residual chain
        ("matmul_bf16", {"num_tokens": t, "n": 64, "k": 5376}, {}),
        ("matmul_bf16", {"num_tokens": t, "n": 7168, "k": 64, "use_residual": True, "output_scale": 0.5}, {}),
        ("h3_head_norm_rope", {"tokens": t, "heads": h, "use_rope": True}, {}),
        ("h3_qk_norm_rope", {"tokens": t, "heads": h, "use_rope": True}, {}),
        ("h3_query_prepare", {"tokens": t, "heads": h, "use_rope": True}, {}),
        ("token_group_mean", {"num_tokens": t, "columns": h * 128, "tokens_per_block": t, "include_padding": False}, {}),
        ("int8_fp8_quantize_qk", {"num_tokens": t, "heads": h, "tokens_per_block": 32, "center": False}, {}),
        ("int8_fp8_quantize_qk", {"num_tokens": t, "heads": h, "tokens_per_block": 64, "center": True}, {}),
        ("int8_fp8_value_scale", {"num_tokens": t, "heads": h}, {}),
        ("int8_fp8_quantize_value", {"num_tokens": t, "heads": h}, {}),
        ("nvfp4_prepare", {"num_tokens": t, "heads": h, "transpose": False, "center": True}, {}),
        ("nvfp4_prepare", {"num_tokens": t, "heads": h, "transpose": True, "center": False}, {}),
        ("sol_pool", {"num_tokens": t, "heads": h, "block": 64}, {}),
        ("sol_int8_fp8_pool", {"num_tokens": t, "heads": h, "block": 64}, {}),
        ("sol_stats", {"heads": h, "num_blocks": -(-t // 64)}, {}),
        ("sol_nvfp4_select", {"num_tokens": t, "heads": h, "tau": 1.0, "block": 64}, {}),
        ("dense_bf16_attention_d128", {"num_tokens": t, "heads": h, "total_heads": h}, {}),
        ("dense_int8_fp8_d128", {"num_query_tokens": t, "num_kv_tokens": t, "heads": h}, {}),
        ("dense_nvfp4_attention_d128", {"num_query_tokens": t, "num_kv_tokens": t, "heads": h, "total_heads": h}, {}),
        ("sol_attention_d128", {"num_tokens": t, "heads": h, "total_heads": h, "block": 128, "topk_fraction": 0.25}, {}),
        ("sol_int8_fp8_attention_d128", {"num_tokens": t, "heads": h, "total_heads": h}, sparse),
        ("sol_nvfp4_attention_d128", {"num_query_tokens": t, "num_kv_tokens": t, "heads": h, "total_heads": h}, sparse),
        ("sol_nvfp4_finalize", {"num_tokens": t, "heads": h, "total_heads": h}, sparse),
    ]


def hbm_peak_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6650.0


def argument_bytes(arguments) -> int:
    total = 0
    for name in arguments.__dataclass_fields__:
        value = getattr(arguments, name)
        if isinstance(value, TensorDesc) and name != "workspace":
            total += value.num_bytes
    return total


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--tokens", type=int, default=32768)
    parser.add_argument("--heads", type=int, default=24)
    parser.add_argument("--repeat", type=int, default=5)
    parser.add_argument("--only", default="", help="comma-separated kernel names")
    args = parser.parse_args()
    only = set(filter(None, args.only.split(",")))
    peak = hbm_peak_gbs()
    rows = []
    for name, fields, options in workloads(args.tokens, args.heads):
        if only and name not in only:
            continue
        cls = kernels.classes()[name]
        workload = tune.workload_of(cls, fields)
        arguments = tune.address(cls.make_arguments(workload))
        if "mask_density" in options:
            tune.fill_mask(arguments, options["mask_density"])
        kernel = cls(arguments)
        times = tune.measure(kernel, args.repeat, 2)
        latency = sorted(times)[len(times) // 2]
        tops = cls.tops(kernel.arguments)
        rows.append(
            {
                "model": "h3-attention-path",
                "kernel": name,
                "latency": latency,
                "launch": 1,
                "mem%": round(100.0 * argument_bytes(arguments) / (latency * 1e-3) / 1e9 / peak, 2),
                "ncu%": "",
                "tops": round(sum(tops.values()) / (latency * 1e-3) / 1e12, 1) if tops else "",
                "workload": canonical(kernel.workload.model_dump(mode="json")),
                "config": canonical(kernel.config.model_dump(mode="json")),
            }
        )
        del kernel, arguments
        torch.cuda.empty_cache()
    total = sum(row["latency"] for row in rows)
    writer = csv.DictWriter(sys.stdout, fieldnames=FIELDS)
    writer.writeheader()
    for row in rows:
        row["percent"] = round(100.0 * row["latency"] / total, 2)
        row["latency"] = round(row["latency"], 4)
        writer.writerow(row)


if __name__ == "__main__":
    main()
