"""NumPy restatement of the KV-cache quantizers, independent of ``nomos_oracle.c``.

TEST INFRASTRUCTURE ONLY ("parity unpinned" at the byte level, see
``nomos_oracle.c``).  Two restatements written separately (scalar C loops and
vectorised NumPy) must agree bit-for-bit before either is trusted as the checker
for the CUDA kernels; ``tests/test_oracle_codecs.py`` enforces that.

All arithmetic is done on ``np.float32`` arrays so every add/mul/div rounds to
binary32 exactly once, as the reference's Float32 expressions do
(lib/kv_cache_quant.mojo:33-40, 170-193, 338-365, 536-578).
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def round_away_clamp(x: np.ndarray, lim: int) -> np.ndarray:
    """trunc(x +- 0.5f) computed in binary32, clamped to [-lim, lim]
    (lib/kv_cache_quant.mojo:33-40, 301-308)."""
    x = x.astype(F32, copy=False)
    y = np.where(x >= F32(0), x + F32(0.5), x - F32(0.5)).astype(F32)
    return np.clip(np.trunc(y).astype(np.int32), -lim, lim)


def quant_rows_i8(x: np.ndarray):
    """x [rows, l_hd] fp32 -> (codes int8 [rows, l_hd], scale fp32 [rows]).
    scale = amax/127 (0 -> 1); code = round_away(x * (1/scale)).  :170-193."""
    x = x.astype(F32, copy=False)
    amax = np.max(np.abs(x), axis=-1).astype(F32)
    scale = (amax / F32(127.0)).astype(F32)
    scale = np.where(scale == 0, F32(1.0), scale).astype(F32)
    inv = (F32(1.0) / scale).astype(F32)
    codes = round_away_clamp((x * inv[..., None]).astype(F32), 127).astype(np.int8)
    return codes, scale


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """codes [..., 2n] in [-8,7] -> bytes [..., n]; even element in the low
    nibble, odd element in the high nibble, two's complement (:364)."""
    c = codes.astype(np.int32) & 0xF
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    """bytes [..., n] -> signed codes [..., 2n] (:761-763)."""
    b = packed.astype(np.int32)
    lo, hi = b & 0xF, (b >> 4) & 0xF
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.int32)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return np.where(out >= 8, out - 16, out).astype(np.int8)


def quant_rows_i4(x: np.ndarray):
    """Row-scale int4: scale = amax/7 (0 -> 1), reciprocal multiply, clamp +-7 (:338-365).
    Returns (codes int8 [rows, l_hd], scale fp32 [rows])."""
    x = x.astype(F32, copy=False)
    amax = np.max(np.abs(x), axis=-1).astype(F32)
    scale = (amax / F32(7.0)).astype(F32)
    scale = np.where(scale == 0, F32(1.0), scale).astype(F32)
    inv = (F32(1.0) / scale).astype(F32)
    codes = round_away_clamp((x * inv[..., None]).astype(F32), 7).astype(np.int8)
    return codes, scale


def quant_rows_i4_block32(x: np.ndarray):
    """Block-32 int4 (:536-578).  x [rows, l_hd] with l_hd a multiple of 32.
    Returns (codes int8 [rows, l_hd], block scales fp16 [rows, nblocks],
    q8 row scale fp32 [rows])."""
    x = x.astype(F32, copy=False)
    rows, l_hd = x.shape
    assert l_hd % 32 == 0
    nb = l_hd // 32
    xb = x.reshape(rows, nb, 32)
    a = np.max(np.abs(xb), axis=-1).astype(F32)
    s = np.where(a > 0, (a / F32(7.0)).astype(F32), F32(1.0)).astype(F32)
    s16 = s.astype(np.float16)                # RNE narrowing
    sf = s16.astype(F32)
    codes = round_away_clamp((xb / sf[..., None]).astype(F32), 7).astype(np.int8).reshape(rows, l_hd)
    recon = np.max((sf * F32(7.0)).astype(F32), axis=-1).astype(F32)
    q8s = np.where(recon > 0, (recon / F32(127.0)).astype(F32), F32(1.0)).astype(F32)
    return codes, s16, q8s


def block32_to_q8(codes: np.ndarray, s16: np.ndarray, q8s: np.ndarray) -> np.ndarray:
    """int8 view of a block-32 row: round_away((q4 * sf) / q8s) (:687, :734)."""
    rows, l_hd = codes.shape
    sf = np.repeat(s16.astype(F32), 32, axis=-1)[:, :l_hd]
    v = ((codes.astype(F32) * sf).astype(F32) / q8s[:, None]).astype(F32)
    return round_away_clamp(v, 127).astype(np.int8)


def ring_rows(nkv: int, cache_cap: int, base_pos: int, n_s: int) -> np.ndarray:
    """Cache row index [n_s, nkv] of (token s, head h): h*cache_cap + (base_pos+s) % cache_cap (:167)."""
    s = (base_pos + np.arange(n_s)) % cache_cap
    return (np.arange(nkv)[None, :] * cache_cap + s[:, None]).astype(np.int64)
