"""Back-to-back launch chains on one stream, without host synchronisation in between.

The attention kernels are launched with programmatic stream serialization: a grid may be set up, run its
warming pass over the query and request settled cache rows while its stream predecessor is still writing.
These tests put real producers in front of it and check every step of the chain against the oracle:
  * the producer epilogue rewrites the query IN PLACE and appends the newest rows, then the tcgen05 kernel
    (and the mma.sync kernel) reads them -- one query buffer reused by every step;
  * a decode loop on ONE cache where every step's attention call carries its own fused append and sets
    NOMOS_ATTN_SETTLED_CACHE, so step i+1 must not stream the row step i is still storing.
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import KVCache, bf16_normal
from tests._gpu import DEV, dev, host, within

pytestmark = pytest.mark.gpu
TOL = 2e-3
PATHS = {"auto": 0, "mma_sync": ops.NO_TCGEN05, "tcgen05": ops.TCGEN05_ALWAYS}


@pytest.mark.parametrize("path", ["mma_sync", "tcgen05"])
@pytest.mark.parametrize("n_s", [1, 9])
def test_producer_rewrites_the_query_in_place_then_attention_reads_it(oracle, path, n_s):
    rng = np.random.default_rng(160 + n_s)
    nh, nkv, hd, T0, steps = 8, 4, 128, 3000, 6
    cap = T0 + steps * n_s
    c = KVCache("i8", nkv, cap, hd)
    k0, v0 = bf16_normal(rng, (T0, nkv, hd)), bf16_normal(rng, (T0, nkv, hd))
    c.append(k0, v0, 0)
    ck, cv, cks, cvs = dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)
    qw = dev((1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)); kw = dev(np.ones(hd, np.float32))
    raw_q = dev(rng.standard_normal((steps, n_s, nh, hd)).astype(np.float32) * np.float32(3.0))
    raw_k = dev(rng.standard_normal((steps, n_s, nkv, hd)).astype(np.float32))
    raw_v = dev(rng.standard_normal((steps, n_s, nkv, hd)).astype(np.float32))
    dq = torch.zeros((n_s, nh, hd), dtype=torch.float32, device=DEV)           # ONE query buffer for every step
    outs = torch.full((steps, n_s, nh, hd), -1e30, dtype=torch.float32, device=DEV)
    k_used = torch.zeros((steps, n_s, nkv, hd), dtype=torch.float32, device=DEV); v_used = torch.zeros_like(k_used)
    args = []
    for i in range(steps):
        klen = T0 + (i + 1) * n_s
        a = ops.make_args(q=dq, k_cache=ck, v_cache=cv, k_scales=cks, v_scales=cvs, out=outs[i], kv_fmt=ops.KV_I8, S=n_s,
                          nh=nh, nkv=nkv, kvg=nh // nkv, l_hd=hd, cache_hd=hd, cache_cap=cap, klen=klen, softmax_scale=0.09,
                          flags=PATHS[path] | ops.SETTLED_CACHE)
        args.append(a)
    need = max(ops.attn_workspace_bytes(a) for a in args)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    for a in args:
        a.workspace, a.ws_bytes = ws.data_ptr(), need
    torch.cuda.synchronize()
    for i in range(steps):                                                     # no synchronisation inside the loop
        dq.copy_(raw_q[i])
        ops.kv_norm_rope_append(None, dq, qw, raw_k[i], raw_v[i], kw, ck, cv, cks, cvs, n_s=n_s, nh=nh, nkv=nkv, l_hd=hd,
                                l_kvd=nkv * hd, cache_cap=cap, cache_hd=hd, base_pos=T0 + i * n_s, theta=10000.0, rope_dim=hd,
                                kv_fmt=ops.KV_I8, k_out=k_used[i], v_out=v_used[i])
        ops.attn_fused(None, args[i])
    torch.cuda.synchronize()
    # what the producer made of each step's query: the same kernel run alone on a copy (it is deterministic)
    q_used = []
    for i in range(steps):
        t = raw_q[i].clone()
        ops.kv_norm_rope_append(None, t, qw, raw_k[i], raw_v[i], kw, None, None, None, None, n_s=n_s, nh=nh, nkv=nkv, l_hd=hd,
                                l_kvd=nkv * hd, cache_cap=0, cache_hd=hd, base_pos=T0 + i * n_s, theta=10000.0, rope_dim=hd,
                                kv_fmt=-1)
        torch.cuda.synchronize()
        q_used.append(host(t))
    got = host(outs)
    for i in range(steps):
        c.append(host(k_used[i]), host(v_used[i]), T0 + i * n_s)
        klen = T0 + (i + 1) * n_s
        want = oracle.attn_exact(q_used[i], c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, cap, S=n_s, window=0,
                                 query_base_pos=klen - n_s, win_lo=0, softmax_scale=0.09)
        for r in range(n_s):
            ok, rel = within(got[i][r], want[r], TOL)
            assert ok, f"step {i} row {r}: {rel:.2e} x RMS"
    assert np.array_equal(host(ck).view(np.uint8), c.k.view(np.uint8)) and np.array_equal(host(cks), c.ks)


@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("n_new", [1, 4])
def test_single_cache_fused_append_loop_with_settled_cache_flag(oracle, path, n_new):
    """Every step appends its own rows inside the attention launch and declares the older rows settled; the next
    step's early reads must leave out the rows this step is still storing."""
    rng = np.random.default_rng(170 + n_new)
    nh, nkv, hd, steps = 8, 4, 128, 10
    T0 = 128 * 9 - 3                       # the appended rows cross a tile boundary during the loop
    cap = T0 + steps * n_new
    c = KVCache("i8", nkv, cap, hd)
    c.append(bf16_normal(rng, (T0, nkv, hd)), bf16_normal(rng, (T0, nkv, hd)), 0)
    ck, cv, cks, cvs = dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)
    q = bf16_normal(rng, (steps, n_new, nh, hd))
    nk = bf16_normal(rng, (steps, n_new, nkv, hd)); nv = bf16_normal(rng, (steps, n_new, nkv, hd))
    dq, dnk, dnv = dev(q), dev(nk), dev(nv)
    outs = torch.full((steps, n_new, nh, hd), -1e30, dtype=torch.float32, device=DEV)
    args = []
    for i in range(steps):
        klen = T0 + (i + 1) * n_new
        args.append(ops.make_args(q=dq[i], k_cache=ck, v_cache=cv, k_scales=cks, v_scales=cvs, out=outs[i], kv_fmt=ops.KV_I8,
                                  S=n_new, nh=nh, nkv=nkv, kvg=nh // nkv, l_hd=hd, cache_hd=hd, cache_cap=cap, klen=klen,
                                  softmax_scale=0.1, new_k=dnk[i], new_v=dnv[i], n_new=n_new, new_base_pos=klen - n_new,
                                  flags=PATHS[path] | ops.SETTLED_CACHE))
    need = max(ops.attn_workspace_bytes(a) for a in args)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    for a in args:
        a.workspace, a.ws_bytes = ws.data_ptr(), need
    torch.cuda.synchronize()
    for a in args:
        ops.attn_fused(None, a)
    torch.cuda.synchronize()
    got = host(outs)
    for i in range(steps):
        c.append(nk[i], nv[i], T0 + i * n_new)
        klen = T0 + (i + 1) * n_new
        want = oracle.attn_exact(q[i], c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, cap, S=n_new, window=0,
                                 query_base_pos=klen - n_new, win_lo=0, softmax_scale=0.1)
        for r in range(n_new):
            ok, rel = within(got[i][r], want[r], TOL)
            assert ok, f"step {i} row {r}: {rel:.2e} x RMS"
    assert np.array_equal(host(ck).view(np.uint8), c.k.view(np.uint8)) and np.array_equal(host(cks), c.ks)
