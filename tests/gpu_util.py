"""Helpers shared by the GPU parity tests."""

from __future__ import annotations

import torch

from nano_omni_b200 import _lib
from nano_omni_b200.core import DType, TensorDesc


def desc(tensor: torch.Tensor, dtype: DType | None = None) -> TensorDesc:
    return TensorDesc.from_torch(tensor, dtype)


def randn_bf16(seed: int, *shape: int, outlier: bool = False, device: str = "cuda") -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g)
    if outlier:
        x[..., 5] *= 16
    return x.bfloat16().to(device)


def run(kernel) -> None:
    """Launch, synchronise and fail on a device status (bounded-wait timeout)."""
    kernel.submit()
    status = _lib.read_status()
    assert status == 0, f"{type(kernel).symbol}: device status {status:#x}"
