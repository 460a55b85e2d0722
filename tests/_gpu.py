"""Small torch helpers for the GPU tests: host arrays <-> device tensors."""
from __future__ import annotations

import numpy as np
import torch

DEV = "cuda:0"


def dev(a: np.ndarray) -> torch.Tensor:
    """Copy a NumPy array to the device keeping its bytes (uint16/uint8 stay integer tensors)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def host(t: torch.Tensor, dtype=None) -> np.ndarray:
    a = t.detach().cpu().contiguous()
    if a.dtype == torch.bfloat16:
        a = a.view(torch.int16)
    out = a.numpy()
    return out.view(dtype) if dtype is not None else out


def bf16_dev(a_f32: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a_f32, dtype=np.float32)).to(DEV).to(torch.bfloat16)


def within(out: np.ndarray, ref: np.ndarray, tol: float = 2e-3):
    """max|out-ref| <= tol * RMS(ref): the attention parity bar."""
    ref64 = ref.astype(np.float64)
    rms = float(np.sqrt(np.mean(ref64 * ref64)))
    err = float(np.max(np.abs(out.astype(np.float64) - ref64)))
    return err <= tol * rms, err / max(rms, 1e-30)
