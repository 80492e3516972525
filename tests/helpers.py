"""Helpers shared by the GPU parity tests: error metrics and a single-rank layer driver."""
from __future__ import annotations

import numpy as np
import torch


def rel_l2(ref: torch.Tensor, got: torch.Tensor) -> float:
    ref, got = ref.double().cpu(), got.double().cpu()
    denom = ref.norm().item()
    return (ref - got).norm().item() / (denom if denom > 0 else 1.0)


def bf16_from_u16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def to_bytes(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.uint8).cpu().numpy()


BF16_REL_L2 = 1e-2    # tolerance the task states for the BF16 path
MXFP8_REL_L2 = 3e-2   # tolerance the task states for the MXFP8 path
