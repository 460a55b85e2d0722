"""The CUDA library against the committed golden fixtures (tests/golden/), through the C ABI:
cache bytes and scales bit-exact, attention within 2e-3 x RMS of the stored exact output."""
from pathlib import Path

import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._gpu import DEV, dev, host, within

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
FMT_ID = {"i8": ops.KV_I8, "i4": ops.KV_I4, "i4b32": ops.KV_I4B32}


def load(name):
    return dict(np.load(GOLD / name))


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
def test_codec_golden(fmt):
    g = load(f"codec_{fmt}.npz")
    nkv, hd, cap = 4, 128, 16
    dk = torch.zeros(g["cache_k"].shape, dtype=torch.uint8, device=DEV); dv = torch.zeros_like(dk)
    dks = torch.zeros(g["scales_k"].shape, dtype=torch.uint8, device=DEV); dvs = torch.zeros_like(dks)
    for k, v, n, base in ((g["k1"], g["v1"], 9, 11), (g["k2"], g["v2"], 6, 20)):
        if fmt == "i8":
            ops.gpu_append_quant_kv_i8(None, dev(k), dev(v), dk, dv, dks, dvs, n, nkv, hd, nkv * hd, cap, hd, base)
        else:
            ops.gpu_append_quant_kv_i4(None, dev(k), dev(v), dk, dv, dks, dvs, n, nkv, hd, nkv * hd, cap, hd, base,
                                       4 if fmt == "i4b32" else 1)
    torch.cuda.synchronize()
    assert np.array_equal(host(dk), g["cache_k"].view(np.uint8)) and np.array_equal(host(dv), g["cache_v"].view(np.uint8))
    assert np.array_equal(host(dks), g["scales_k"]) and np.array_equal(host(dvs), g["scales_v"])


@pytest.mark.parametrize("name,fmt", [("attn_c1_i8", "i8"), ("attn_ring_i8", "i8"), ("attn_verify_i8", "i8"),
                                      ("attn_ring_i4", "i4"), ("attn_ring_i4b32", "i4b32")])
def test_attention_golden(name, fmt):
    g = load(name + ".npz")
    nh, nkv, hd, T, cap, S, window = (int(x) for x in g["meta"])
    klen = min(T, cap)
    out = torch.full((S, nh, hd), -1e30, dtype=torch.float32, device=DEV)
    keep = [dev(g[k]) for k in ("q", "cache_k", "cache_v", "scales_k", "scales_v")]
    a = ops.make_args(q=keep[0], k_cache=keep[1], v_cache=keep[2], k_scales=keep[3], v_scales=keep[4], out=out,
                      kv_fmt=FMT_ID[fmt], S=S, nh=nh, nkv=nkv, kvg=nh // nkv, l_hd=hd, cache_hd=hd, cache_cap=cap,
                      win_start=T - klen, klen=klen, window=window, softmax_scale=float(g["scale"][0]))
    ws = torch.empty(max(ops.attn_workspace_bytes(a), 16), dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = ws.data_ptr(), ws.numel()
    ops.attn_fused(None, a)
    torch.cuda.synchronize()
    got = host(out)
    for r in range(S):
        ok, rel = within(got[r], g["out"][r], 2e-3)
        assert ok, f"{name} row {r}: {rel:.2e} x RMS"


@pytest.mark.parametrize("tag,theta,rdim_div", [("sliding", 10000.0, 1), ("full", 1000000.0, 4)])
def test_producer_golden(tag, theta, rdim_div):
    """Producer epilogue against the stored float64 rows, within the float32 bound of oracle/np_producer.py."""
    from oracle import np_producer as npp
    g = load("producer.npz")
    n_s, nh, nkv, hd, base = (int(x) for x in g["meta"])
    rdim = hd // rdim_div
    dq = dev(g["q"])
    ko = torch.zeros((n_s, nkv, hd), dtype=torch.float32, device=DEV); vo = torch.zeros_like(ko)
    ops.kv_norm_rope_append(None, dq, dev(g["qw"]), dev(g["k"]), dev(g["v"]), dev(g["kw"]), None, None, None, None,
                            n_s=n_s, nh=nh, nkv=nkv, l_hd=hd, l_kvd=nkv * hd, cache_cap=0, cache_hd=hd, base_pos=base,
                            theta=theta, rope_dim=rdim, kv_fmt=-1, k_out=ko, v_out=vo)
    torch.cuda.synchronize()
    assert np.all(np.abs(host(vo) - g["v_out"]) <= 2e-6 * np.max(np.abs(g["v_out"]), axis=-1, keepdims=True) + 1e-7)
    assert np.all(np.abs(host(ko) - g[f"k_out_{tag}"]) <= npp.rope_tolerance(npp.qk_norm(g["k"], g["kw"]), base, theta, rdim))
    assert np.all(np.abs(host(dq) - g[f"q_out_{tag}"]) <= npp.rope_tolerance(npp.qk_norm(g["q"], g["qw"]), base, theta, rdim))
