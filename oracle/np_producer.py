"""CPU restatement (test infrastructure only) of the reference's K/V/Q producer epilogue.

After the K/V/Q projections the reference runs, per layer and token
(lib/gemma4_layer.mojo:326-340):
  V-norm   gpu_rmsnorm_no_weight_mojo   lib/ops_gpu_mojo_reductions.mojo:353-417
  QK-norm  gpu_qk_norm_mojo             lib/ops_gpu_mojo_reductions.mojo:422-485
  RoPE     gpu_rope_mojo / batched      lib/ops_gpu_mojo.mojo:310-368
and then the quantising append.  The functions here follow those kernels' arithmetic in
float64 (the reference computes in float32; the order of its parallel sums is not
reproducible, so parity for this step is a tolerance, see `rope_tolerance`).

Not pinned by any golden vector of the reference (it has none for these kernels): parity
unpinned; the formulas are anchored on the cited lines only.
"""
from __future__ import annotations

import numpy as np

EPS_RMSNORM = 1e-6                       # ops_gpu_mojo_reductions.mojo:31
LN_THETA_DEFAULT = 9.21034037            # ln(10000), ops_gpu_mojo.mojo:335
LN_THETA_1E6 = 13.81551056               # used when theta == 1000000.0, ops_gpu_mojo.mojo:336-337


def rms_inv(x: np.ndarray) -> np.ndarray:
    """1 / sqrt(mean(x^2) + eps) per row (last axis), ops_gpu_mojo_reductions.mojo:395-396."""
    x = np.asarray(x, np.float64)
    return 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + EPS_RMSNORM)


def rmsnorm_no_weight(x: np.ndarray) -> np.ndarray:
    """V-norm: x * rms_inv per head row."""
    return np.asarray(x, np.float64) * rms_inv(x)


def qk_norm(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """Per-head RMSNorm with a weight vector shared by the heads: x * rms_inv * w[j]."""
    return np.asarray(x, np.float64) * rms_inv(x) * np.asarray(w, np.float64)


def ln_theta(theta: float) -> float:
    """The reference keys the logarithm on equality with 1e6 and otherwise uses ln(10000)."""
    return LN_THETA_1E6 if float(theta) == 1000000.0 else LN_THETA_DEFAULT


def rope_angles(pos: np.ndarray, hd: int, theta: float, rope_dim: int) -> np.ndarray:
    """angle[s, i] = pos[s] * exp(-(2 i / hd) * ln_theta) for the rope_dim/2 rotated pairs."""
    i = np.arange(rope_dim // 2, dtype=np.float64)
    inv_freq = np.exp(-(2.0 * i / float(hd)) * ln_theta(theta))
    return np.asarray(pos, np.float64)[:, None] * inv_freq[None, :]


def rope(x: np.ndarray, base_pos: int, theta: float, rope_dim: int) -> np.ndarray:
    """x [S, H, hd]; token s sits at position base_pos + s.  Pairs are (i, i + hd/2) for
    i < rope_dim/2 (rotate-half split at hd/2 even when rope_dim < hd), the frequency
    denominator is hd:  a' = a cos - b sin,  b' = a sin + b cos."""
    x = np.array(x, np.float64, copy=True)
    S, _, hd = x.shape
    half, n = hd // 2, rope_dim // 2
    ang = rope_angles(base_pos + np.arange(S), hd, theta, rope_dim)      # [S, n]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[:, :, :n].copy(), x[:, :, half:half + n].copy()
    x[:, :, :n] = a * c - b * s
    x[:, :, half:half + n] = a * s + b * c
    return x


def rope_tolerance(x_normed: np.ndarray, base_pos: int, theta: float, rope_dim: int) -> np.ndarray:
    """Per-element bound for an implementation that does this step in float32: 2e-6 of the
    row maximum for the normalisation, plus the rotation error of an angle that carries
    ~2.5 float32 roundings (frequency, product with the position, range reduction):
    3e-7 * angle * hypot(a, b)."""
    x = np.asarray(x_normed, np.float64)
    S, _, hd = x.shape
    half, n = hd // 2, rope_dim // 2
    tol = np.broadcast_to(2e-6 * np.max(np.abs(x), axis=-1, keepdims=True) + 1e-7, x.shape).copy()
    if n:
        ang = np.abs(rope_angles(base_pos + np.arange(S), hd, theta, rope_dim))[:, None, :]
        mag = np.hypot(x[:, :, :n], x[:, :, half:half + n])
        tol[:, :, :n] += 3e-7 * ang * mag + 2e-6 * mag
        tol[:, :, half:half + n] += 3e-7 * ang * mag + 2e-6 * mag
    return tol
