"""Seeded synthetic inputs shared by the CPU and GPU tests and by the benchmark.

No public dataset is involved: tensors stand in for one layer's attention state at
the shapes the benchmark configurations name.  Values are N(0,1) drawn in fp32,
rounded to bf16 and widened back, as the configurations specify.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle as orc


def bf16_normal(rng: np.random.Generator, shape) -> np.ndarray:
    return orc.bf16_round(rng.standard_normal(shape, dtype=np.float32))


def k_with_outliers(rng: np.random.Generator, T: int, nkv: int, hd: int, n_out: int = 4, gain: float = 8.0):
    """K [T, nkv, hd]; per KV head `n_out` channels scaled by `gain` (configuration 2)."""
    k = rng.standard_normal((T, nkv, hd), dtype=np.float32)
    for h in range(nkv):
        ch = rng.choice(hd, n_out, replace=False)
        k[:, h, ch] *= gain
    return orc.bf16_round(k)


def ref_probe_rows(n_rows: int, kvd: int, layer: int, base_pos: int):
    """Deterministic K/V source rows of the reference's append A/B probe
    (nomos_ffi.mojo:1052-1059): row gains (s+1)^2 so that any cross-row leakage of
    quantisation statistics changes the bytes."""
    j = np.arange(kvd)[None, :]
    s = np.arange(n_rows)[:, None]
    raw = ((j * 37 + s * 101 + layer * 17 + base_pos * 13) % 257) - 128
    gain = ((s + 1) * (s + 1)).astype(np.float32)
    x = ((raw.astype(np.float32) / np.float32(17.0)).astype(np.float32) * gain).astype(np.float32)
    v = ((x * np.float32(0.73)).astype(np.float32)
         + ((s + 1).astype(np.float32) * np.float32(0.19)).astype(np.float32)).astype(np.float32)
    return np.ascontiguousarray(x), np.ascontiguousarray(v)


def ref_q8_probe_row(kvd: int, layer: int):
    """Single deterministic row of the block-32 q8-view probe (nomos_ffi.mojo:875-879)."""
    i = np.arange(kvd)
    raw = ((i * 37 + layer * 17) % 257) - 128
    x = (raw.astype(np.float32) / np.float32(17.0)).astype(np.float32)
    v = ((x * np.float32(0.73)).astype(np.float32) + np.float32(0.19)).astype(np.float32)
    return np.ascontiguousarray(x[None, :]), np.ascontiguousarray(v[None, :])


class KVCache:
    """Host-side packed KV cache in the reference's layouts.

    fmt: 'i8' (int8 + fp32 row scale), 'i4' (int4 + fp32 row scale),
    'i4b32' (int4 + fp16 scale per 32 + cached fp32 q8 row scale)."""

    def __init__(self, fmt: str, nkv: int, cache_cap: int, l_hd: int, cache_hd: int | None = None):
        self.fmt, self.nkv, self.cache_cap, self.l_hd = fmt, nkv, cache_cap, l_hd
        self.cache_hd = cache_hd or l_hd
        self.scale_blocks = (l_hd + 31) // 32 if fmt == "i4b32" else 1
        row_bytes = self.cache_hd if fmt == "i8" else self.cache_hd // 2
        dt = np.int8 if fmt == "i8" else np.uint8
        self.k = np.zeros((nkv, cache_cap, row_bytes), dtype=dt)
        self.v = np.zeros((nkv, cache_cap, row_bytes), dtype=dt)
        nbytes = orc.scale_buffer_bytes(nkv, cache_cap, l_hd, self.scale_blocks)
        self.ks = np.zeros(nbytes, dtype=np.uint8)
        self.vs = np.zeros(nbytes, dtype=np.uint8)

    @property
    def kv_fmt(self) -> int:
        return {"i8": orc.KV_I8, "i4": orc.KV_I4, "i4b32": orc.KV_I4B32}[self.fmt]

    def append(self, k_rows: np.ndarray, v_rows: np.ndarray, base_pos: int):
        """k_rows/v_rows [n_s, nkv, l_hd] fp32."""
        n_s = k_rows.shape[0]
        k_rows = np.ascontiguousarray(k_rows, dtype=np.float32)
        v_rows = np.ascontiguousarray(v_rows, dtype=np.float32)
        l_kvd = self.nkv * self.l_hd
        if self.fmt == "i8":
            orc.append_quant_kv_i8(k_rows, v_rows, self.k, self.v, self.ks, self.vs,
                                   n_s, self.nkv, self.l_hd, l_kvd, self.cache_cap, self.cache_hd, base_pos)
        else:
            orc.append_quant_kv_i4(k_rows, v_rows, self.k, self.v, self.ks, self.vs,
                                   n_s, self.nkv, self.l_hd, l_kvd, self.cache_cap, self.cache_hd, base_pos,
                                   self.scale_blocks)

    def row_scales_f32(self, which: str) -> np.ndarray:
        buf = self.ks if which == "k" else self.vs
        assert self.fmt != "i4b32"
        return buf.view(np.float32).reshape(self.nkv, self.cache_cap)
