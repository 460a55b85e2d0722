"""The oracle reproduces the committed golden fixtures (CPU only).
Fixtures and their generator live in tests/golden/."""
from pathlib import Path

import numpy as np
import pytest

from tests._cases import KVCache

GOLD = Path(__file__).resolve().parent / "golden"
FMT_ID = {"i8": 0, "i4": 1, "i4b32": 2}


def load(name):
    return dict(np.load(GOLD / name))


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
def test_codec_golden(oracle, fmt):
    g = load(f"codec_{fmt}.npz")
    nkv, hd, cap = 4, 128, 16
    c = KVCache(fmt, nkv, cap, hd)
    c.append(g["k1"].reshape(9, nkv, hd), g["v1"].reshape(9, nkv, hd), 11)
    c.append(g["k2"], g["v2"], 20)
    assert np.array_equal(c.k, g["cache_k"]) and np.array_equal(c.v, g["cache_v"])
    assert np.array_equal(c.ks, g["scales_k"]) and np.array_equal(c.vs, g["scales_v"])


@pytest.mark.parametrize("name,fmt", [("attn_c1_i8", "i8"), ("attn_ring_i8", "i8"), ("attn_verify_i8", "i8"),
                                      ("attn_ring_i4", "i4"), ("attn_ring_i4b32", "i4b32")])
def test_attention_golden(oracle, name, fmt):
    g = load(name + ".npz")
    nh, nkv, hd, T, cap, S, window = (int(x) for x in g["meta"])
    klen = min(T, cap)
    out = oracle.attn_exact(g["q"], g["cache_k"], g["cache_v"], g["scales_k"], g["scales_v"], FMT_ID[fmt], nh, nkv, hd, hd,
                            cap, S=S, window=window, query_base_pos=T - S, win_lo=T - klen, softmax_scale=float(g["scale"][0]))
    assert np.allclose(out, g["out"], rtol=0, atol=1e-6)


def test_producer_golden():
    from oracle import np_producer as npp
    g = load("producer.npz")
    n_s, nh, nkv, hd, base = (int(x) for x in g["meta"])
    assert np.allclose(npp.rmsnorm_no_weight(g["v"]), g["v_out"], rtol=0, atol=1e-12)
    for tag, theta, rdim in (("sliding", 10000.0, hd), ("full", 1000000.0, hd // 4)):
        assert np.allclose(npp.rope(npp.qk_norm(g["k"], g["kw"]), base, theta, rdim), g[f"k_out_{tag}"], rtol=0, atol=1e-12)
        assert np.allclose(npp.rope(npp.qk_norm(g["q"], g["qw"]), base, theta, rdim), g[f"q_out_{tag}"], rtol=0, atol=1e-12)
