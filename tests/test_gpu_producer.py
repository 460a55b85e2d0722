"""GPU parity of the fused producer epilogue (V-norm, QK-norm, RoPE, quantize-on-write), through
the C ABI.

Two gates.  (1) The normalised / rotated fp32 rows (Q in place, K and V through k_out / v_out)
against the float64 restatement of the reference kernels, within `np_producer.rope_tolerance`
(float32 roundings of the norm plus the angle error a float32 frequency x position product
carries).  (2) The cache bytes and scales must equal, bit for bit, what the oracle's append
codec makes of exactly those fp32 rows."""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from oracle import np_producer as npp
from tests._cases import KVCache, bf16_normal
from tests._gpu import DEV, dev, host

pytestmark = pytest.mark.gpu


def run_case(fmt, hd, nh, nkv, n_s, base_pos, cap, theta, rope_dim, seed, with_q=True, l_kvd=None):
    rng = np.random.default_rng(seed)
    l_kvd = l_kvd or nkv * hd
    q = (rng.standard_normal((n_s, nh, hd)) * 3.0).astype(np.float32)
    k = np.zeros((n_s, l_kvd), np.float32); v = np.zeros((n_s, l_kvd), np.float32)
    k[:, :nkv * hd] = (rng.standard_normal((n_s, nkv * hd)) * 2.0).astype(np.float32)
    v[:, :nkv * hd] = (rng.standard_normal((n_s, nkv * hd)) * 0.7).astype(np.float32)
    qw = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kw = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    c = KVCache(fmt, nkv, cap, hd)
    dq, dk, dv, dqw, dkw = dev(q), dev(k), dev(v), dev(qw), dev(kw)
    ck, cv, cks, cvs = dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)
    ko = torch.full((n_s, nkv, hd), -1e30, dtype=torch.float32, device=DEV); vo = torch.full_like(ko, -1e30)
    ops.kv_norm_rope_append(None, dq if with_q else None, dqw if with_q else None, dk, dv, dkw, ck, cv, cks, cvs,
                            n_s=n_s, nh=nh, nkv=nkv, l_hd=hd, l_kvd=l_kvd, cache_cap=cap, cache_hd=hd, base_pos=base_pos,
                            theta=theta, rope_dim=rope_dim, kv_fmt=c.kv_fmt, k_out=ko, v_out=vo)
    torch.cuda.synchronize()
    k3 = k[:, :nkv * hd].reshape(n_s, nkv, hd); v3 = v[:, :nkv * hd].reshape(n_s, nkv, hd)
    # gate 1: values
    want_v = npp.rmsnorm_no_weight(v3)
    kn = npp.qk_norm(k3, kw)
    want_k = npp.rope(kn, base_pos, theta, rope_dim)
    got_k, got_v = host(ko), host(vo)
    assert np.all(np.abs(got_v - want_v) <= 2e-6 * np.max(np.abs(want_v), axis=-1, keepdims=True) + 1e-7), "V-norm"
    assert np.all(np.abs(got_k - want_k) <= npp.rope_tolerance(kn, base_pos, theta, rope_dim)), "K norm + rope"
    if with_q:
        qn = npp.qk_norm(q, qw)
        want_q = npp.rope(qn, base_pos, theta, rope_dim)
        assert np.all(np.abs(host(dq) - want_q) <= npp.rope_tolerance(qn, base_pos, theta, rope_dim)), "Q norm + rope"
    else:
        assert np.array_equal(host(dq), q)
    assert np.array_equal(host(dk), k) and np.array_equal(host(dv), v), "sources must not be modified"
    # gate 2: bytes and scales are the codec's, bit for bit, on exactly those rows
    c.append(got_k, got_v, base_pos)
    assert np.array_equal(host(ck), c.k) and np.array_equal(host(cv), c.v), "cache bytes"
    assert np.array_equal(host(cks), c.ks) and np.array_equal(host(cvs), c.vs), "scales"


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
def test_decode_token_sliding_layer_geometry(fmt):
    """One token, rope over the whole head (rope_dim = head_dim, theta 1e4), ring slot pos % cap."""
    run_case(fmt, hd=256, nh=32, nkv=16, n_s=1, base_pos=8191, cap=1024, theta=10000.0, rope_dim=256, seed=11)


@pytest.mark.parametrize("fmt", ["i8", "i4b32"])
def test_decode_token_full_layer_geometry(fmt):
    """Full-attention layers: head_dim 512, partial rotary (head_dim / 4), theta 1e6."""
    run_case(fmt, hd=512, nh=32, nkv=4, n_s=1, base_pos=12345, cap=16384, theta=1000000.0, rope_dim=128, seed=12)


@pytest.mark.parametrize("fmt,hd", [("i8", 128), ("i4", 128), ("i4b32", 128), ("i8", 64)])
def test_batched_tokens_positions_and_ring_wrap(fmt, hd):
    """n_s tokens at positions base_pos + s, wrapping the ring, with a padded token stride."""
    run_case(fmt, hd=hd, nh=8, nkv=4, n_s=9, base_pos=1020, cap=1024, theta=10000.0, rope_dim=hd, seed=13,
             l_kvd=4 * hd + 64)


def test_without_query_rows_and_position_zero():
    run_case("i8", hd=128, nh=8, nkv=4, n_s=3, base_pos=0, cap=64, theta=10000.0, rope_dim=128, seed=14, with_q=False)


def test_norm_and_rope_only_leaves_the_cache_alone():
    rng = np.random.default_rng(15)
    n_s, nkv, hd = 2, 4, 128
    k = rng.standard_normal((n_s, nkv, hd)).astype(np.float32); v = rng.standard_normal((n_s, nkv, hd)).astype(np.float32)
    kw = np.ones(hd, np.float32)
    ko = torch.zeros((n_s, nkv, hd), dtype=torch.float32, device=DEV); vo = torch.zeros_like(ko)
    ops.kv_norm_rope_append(None, None, None, dev(k), dev(v), dev(kw), None, None, None, None,
                            n_s=n_s, nh=0, nkv=nkv, l_hd=hd, l_kvd=nkv * hd, cache_cap=0, cache_hd=hd, base_pos=5,
                            theta=10000.0, rope_dim=128, kv_fmt=-1, k_out=ko, v_out=vo)
    torch.cuda.synchronize()
    kn = npp.qk_norm(k, kw)
    assert np.all(np.abs(host(ko) - npp.rope(kn, 5, 10000.0, 128)) <= npp.rope_tolerance(kn, 5, 10000.0, 128))
    assert np.allclose(host(vo), npp.rmsnorm_no_weight(v), rtol=0, atol=1e-5)


def test_produced_rows_feed_the_attention_call(oracle):
    """End of the chain: rows written by the producer are read by the fused attention kernel."""
    rng = np.random.default_rng(16)
    nh, nkv, hd, T = 8, 4, 128, 300
    c = KVCache("i8", nkv, T, hd)
    ck, cv, cks, cvs = dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)
    kw = np.ones(hd, np.float32); qw = np.ones(hd, np.float32)
    k = rng.standard_normal((T, nkv, hd)).astype(np.float32); v = rng.standard_normal((T, nkv, hd)).astype(np.float32)
    q = rng.standard_normal((1, nh, hd)).astype(np.float32)
    dq = dev(q)
    ko = torch.zeros((T, nkv, hd), dtype=torch.float32, device=DEV); vo = torch.zeros_like(ko)
    ops.kv_norm_rope_append(None, None, None, dev(k), dev(v), dev(kw), ck, cv, cks, cvs, n_s=T, nh=0, nkv=nkv, l_hd=hd,
                            l_kvd=nkv * hd, cache_cap=T, cache_hd=hd, base_pos=0, theta=10000.0, rope_dim=hd, kv_fmt=ops.KV_I8,
                            k_out=ko, v_out=vo)
    ops.kv_norm_rope_append(None, dq, dev(qw), dev(k[:1]), dev(v[:1]), dev(kw), None, None, None, None, n_s=1, nh=nh, nkv=nkv,
                            l_hd=hd, l_kvd=nkv * hd, cache_cap=0, cache_hd=hd, base_pos=T - 1, theta=10000.0, rope_dim=hd, kv_fmt=-1)
    out = torch.zeros((1, nh, hd), dtype=torch.float32, device=DEV)
    a = ops.make_args(q=dq, k_cache=ck, v_cache=cv, k_scales=cks, v_scales=cvs, out=out, kv_fmt=ops.KV_I8, nh=nh, nkv=nkv,
                      kvg=2, l_hd=hd, cache_hd=hd, cache_cap=T, klen=T, softmax_scale=0.05)
    ws = torch.empty(max(ops.attn_workspace_bytes(a), 16), dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = ws.data_ptr(), ws.numel()
    ops.attn_fused(None, a)
    torch.cuda.synchronize()
    c.append(host(ko), host(vo), 0)
    want = oracle.attn_exact(host(dq), c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, T, S=1, window=0,
                             query_base_pos=T - 1, win_lo=0, softmax_scale=0.05)
    err = np.max(np.abs(host(out) - want)) / np.sqrt(np.mean(want ** 2))
    assert err <= 2e-3, f"{err:.2e} x RMS"
