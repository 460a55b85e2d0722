"""Generates the golden fixtures in this folder from the CPU oracle.

    python tests/golden/gen_golden.py

The reference itself (Mojo GPU kernels) cannot run where this repository is built
and publishes no golden bytes for this path, so these vectors pin the ORACLE's
current behaviour (its arithmetic is a restatement of the reference, see
oracle/nomos_oracle.c): a change to either the oracle or the CUDA kernels that
alters a byte shows up against them.  Inputs are stored with the outputs, so the
fixtures do not depend on a random-number generator's stream.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import oracle as orc  # noqa: E402
from tests._cases import KVCache, bf16_normal, k_with_outliers, ref_probe_rows  # noqa: E402


def codec_case(fmt: str, seed: int):
    """9 probe rows (the reference's own generator) + random rows through a wrapping ring of 16."""
    nkv, hd, cap = 4, 128, 16
    rng = np.random.default_rng(seed)
    k1, v1 = ref_probe_rows(9, nkv * hd, 3, 11)
    k2, v2 = bf16_normal(rng, (6, nkv, hd)), bf16_normal(rng, (6, nkv, hd))
    c = KVCache(fmt, nkv, cap, hd)
    c.append(k1.reshape(9, nkv, hd), v1.reshape(9, nkv, hd), 11)      # slots 11..15, 0..3
    c.append(k2, v2, 20)                                              # slots 4..9
    return dict(k1=k1, v1=v1, k2=k2, v2=v2, cache_k=c.k, cache_v=c.v, scales_k=c.ks, scales_v=c.vs)


def attn_case(fmt: str, seed: int, nh, nkv, hd, T, cap, S=1, window=0, scale=1.0, outliers=False):
    rng = np.random.default_rng(seed)
    k = k_with_outliers(rng, T, nkv, hd) if outliers else bf16_normal(rng, (T, nkv, hd))
    v = bf16_normal(rng, (T, nkv, hd))
    q = bf16_normal(rng, (S, nh, hd))
    c = KVCache(fmt, nkv, cap, hd)
    c.append(k, v, 0)
    klen = min(T, cap)
    out = orc.attn_exact(q, c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, cap, S=S, window=window,
                         query_base_pos=T - S, win_lo=T - klen, softmax_scale=scale)
    return dict(q=q, cache_k=c.k, cache_v=c.v, scales_k=c.ks, scales_v=c.vs, out=out,
                meta=np.array([nh, nkv, hd, T, cap, S, window], np.int64), scale=np.array([scale], np.float64))


def producer_case(seed: int):
    """Producer epilogue (V-norm, QK-norm, RoPE): 3 tokens from position 1022, 8 q / 4 kv heads x 128,
    full rotary with theta 1e4, and the partial-rotary / theta 1e6 variant on the same inputs."""
    from oracle import np_producer as npp
    rng = np.random.default_rng(seed)
    n_s, nh, nkv, hd, base = 3, 8, 4, 128, 1022
    q = (rng.standard_normal((n_s, nh, hd)) * 3.0).astype(np.float32)
    k = (rng.standard_normal((n_s, nkv, hd)) * 2.0).astype(np.float32)
    v = (rng.standard_normal((n_s, nkv, hd)) * 0.7).astype(np.float32)
    qw = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kw = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    out = dict(q=q, k=k, v=v, qw=qw, kw=kw, meta=np.array([n_s, nh, nkv, hd, base], np.int64),
               v_out=npp.rmsnorm_no_weight(v))
    for tag, theta, rdim in (("sliding", 10000.0, hd), ("full", 1000000.0, hd // 4)):
        out[f"k_out_{tag}"] = npp.rope(npp.qk_norm(k, kw), base, theta, rdim)
        out[f"q_out_{tag}"] = npp.rope(npp.qk_norm(q, qw), base, theta, rdim)
    return out


def main():
    orc.build()
    np.savez_compressed(HERE / "producer.npz", **producer_case(1010))
    for fmt in ("i8", "i4", "i4b32"):
        np.savez_compressed(HERE / f"codec_{fmt}.npz", **codec_case(fmt, 7))
    # configuration 1 (8/4 heads, hd 128, 512 keys, scale 1/sqrt(128)), int8
    np.savez_compressed(HERE / "attn_c1_i8.npz", **attn_case("i8", 1001, 8, 4, 128, 512, 512, scale=1 / np.sqrt(128.0)))
    # wrapped ring, int8: 700 positions through 256 slots
    np.savez_compressed(HERE / "attn_ring_i8.npz", **attn_case("i8", 1003, 8, 4, 128, 700, 256, scale=0.2))
    # verify rows: S = 9 over 300 keys
    np.savez_compressed(HERE / "attn_verify_i8.npz", **attn_case("i8", 1004, 8, 4, 128, 300, 512, S=9, scale=0.15))
    # int4 layouts (ring of 256 wrapped)
    for fmt in ("i4", "i4b32"):
        np.savez_compressed(HERE / f"attn_ring_{fmt}.npz", **attn_case(fmt, 1005, 8, 4, 128, 700, 256, scale=0.2))
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
