"""Isolated kernel launcher and timer (the role of the reference's scripts/tune.py:228-280).

    python -m nano_omni_b200.tune --kernel dense_bf16_attention_d128 \
        --workload '{"num_tokens": 16384, "heads": 16, "total_heads": 16}' --repeat 5

Builds the kernel's arguments from its Workload with seeded random CUDA tensors
(floats N(0,1)*scale, int8 in [-3,3], bytes uniform, e4m3 scales in [0.125,1.125)),
launches it through the C ABI and reports CUDA-event times.  It is the command
that profiler captures are taken from; correctness is checked by the test suite,
not here.
"""

from __future__ import annotations

import argparse
import dataclasses
import json

import torch

from nano_omni_b200 import _lib, kernels
from nano_omni_b200.core import DType, TensorDesc, TensorKind


def _fill(desc: TensorDesc, generator: torch.Generator, scale: float) -> TensorDesc:
    shape = desc.shape
    if desc.dtype == DType.BF16:
        t = (torch.randn(shape, generator=generator, device="cuda") * scale).bfloat16()
    elif desc.dtype == DType.F32:
        t = torch.rand(shape, generator=generator, device="cuda") * 0.1 + 0.01
    elif desc.dtype == DType.I8:
        t = torch.randint(-3, 4, shape, generator=generator, device="cuda", dtype=torch.int8)
    elif desc.dtype == DType.FP8_UE4M3:
        t = (torch.rand(shape, generator=generator, device="cuda") + 0.125).to(torch.float8_e4m3fn)
    elif desc.dtype == DType.FP8_E4M3:
        t = torch.randn(shape, generator=generator, device="cuda").to(torch.float8_e4m3fn)
    else:
        t = torch.randint(0, 256, shape, generator=generator, device="cuda", dtype=torch.uint8)
    return TensorDesc.from_torch(t, desc.dtype)


def address(arguments, seed: int = 0, scale: float = 1.0):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    return arguments.map(lambda d: _fill(d, generator, scale) if d.kind == TensorKind.EMPTY else d)


def measure(kernel, repeat: int, warmup: int) -> list[float]:
    stream = torch.cuda.current_stream()
    for _ in range(warmup):
        kernel.submit()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeat):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        kernel.submit()
        b.record(stream)
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    status = _lib.read_status()
    if status:
        raise RuntimeError(f"device status {status:#x}: a bounded wait gave up")
    return times


def workload_of(cls, fields: dict):
    """Instance of the Workload type that ``cls.make_workload`` returns, built from ``fields``."""
    wanted = cls.make_workload.__annotations__.get("return")
    for candidate in vars(__import__(cls.__module__, fromlist=["x"])).values():
        if isinstance(candidate, type) and candidate.__name__ == wanted:
            return candidate(**fields)
    raise LookupError(f"cannot find workload type {wanted}")


def fill_mask(arguments, density: float) -> None:
    """Routing mask argument (``selected`` / ``mask``): ones at ``density`` plus the three-block band and block 0."""
    for name in ("selected", "mask"):
        tensor = getattr(arguments, name, None)
        if tensor is None:
            continue
        generator = torch.Generator(device="cuda").manual_seed(1)
        mask = tensor.as_torch()
        mask.copy_((torch.rand(mask.shape, generator=generator, device="cuda") < density).to(mask.dtype))
        blocks = torch.arange(mask.shape[0], device="cuda")
        band = (blocks[:, None] - torch.arange(mask.shape[2], device="cuda")[None, :]).abs() <= 1
        mask.masked_fill_(band[:, None, :], 1)
        mask[..., 0] = 1


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--kernel", required=True)
    parser.add_argument("--workload", required=True, help="JSON object with the Workload fields")
    parser.add_argument("--overrides", default="{}", help="JSON object of scalar Arguments fields to replace")
    parser.add_argument("--repeat", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=1)
    parser.add_argument("--scale", type=float, default=1.0)
    parser.add_argument(
        "--mask-density",
        type=float,
        default=None,
        help="fill a routing mask argument (`selected` / `mask`) with ones at this density plus the three-block band",
    )
    args = parser.parse_args()

    cls = kernels.classes()[args.kernel]
    arguments = cls.make_arguments(workload_of(cls, json.loads(args.workload)))
    overrides = json.loads(args.overrides)
    if overrides:
        arguments = dataclasses.replace(arguments, **overrides)
    arguments = address(arguments, scale=args.scale)
    if args.mask_density is not None:
        fill_mask(arguments, args.mask_density)
    kernel = cls(arguments)
    times = measure(kernel, args.repeat, args.warmup)
    result = {
        "kernel": args.kernel,
        "workload": kernel.workload.model_dump(),
        "ms": times,
        "ms_median": sorted(times)[len(times) // 2],
    }
    tops = cls.tops(kernel.arguments)
    if tops:
        ops = sum(tops.values())
        result["tops_per_s"] = ops / (result["ms_median"] * 1e-3) / 1e12
    print(json.dumps(result))


if __name__ == "__main__":
    main()
