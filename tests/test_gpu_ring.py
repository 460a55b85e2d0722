"""Verify and decode over a sliding-window ring with slack, driven by the ring bookkeeping API:
batches of draft rows are appended and attended in one fused call, some are rejected and later
overwritten, and every output row must equal exact sliding-window attention over the LINEAR
history of accepted rows (the combination the reference refuses, lib/engine_prefill.mojo:87-88)."""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import KVCache, bf16_normal
from tests._gpu import DEV, dev, host, within

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["i8", "i4b32"])
def test_verify_over_ring_with_rollback(oracle, fmt):
    rng = np.random.default_rng(91)
    nh, nkv, hd, W, VB = 8, 4, 128, 64, 5
    cap = W + VB - 1
    ring = ops.KvRing(cache_cap=cap, window=W, max_rows=VB)
    c = KVCache(fmt, nkv, cap, hd)
    dk, dv, dks, dvs = dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)
    hist_k = np.zeros((0, nkv, hd), np.float32); hist_v = np.zeros((0, nkv, hd), np.float32)
    for step_no in range(110):
        n = 1 if step_no % 3 == 0 else int(rng.integers(2, VB + 1))
        st = ring.plan(n)
        L = int(st.base_pos)
        assert L == hist_k.shape[0]
        new_k, new_v = bf16_normal(rng, (n, nkv, hd)), bf16_normal(rng, (n, nkv, hd))
        q = bf16_normal(rng, (n, nh, hd))
        dq, dnk, dnv = dev(np.ascontiguousarray(q, np.float32)), dev(new_k), dev(new_v)
        out = torch.full((n, nh, hd), -1e30, dtype=torch.float32, device=DEV)
        a = ops.make_args(q=dq, k_cache=dk, v_cache=dv, k_scales=dks, v_scales=dvs, out=out, kv_fmt=c.kv_fmt, nh=nh, nkv=nkv,
                          kvg=nh // nkv, l_hd=hd, cache_hd=hd, cache_cap=1, klen=1, softmax_scale=0.1,
                          new_k=dnk.data_ptr(), new_v=dnv.data_ptr())
        ring.fill_args(st, a)
        ws = torch.empty(max(ops.attn_workspace_bytes(a), 16), dtype=torch.uint8, device=DEV)
        a.workspace, a.ws_bytes = ws.data_ptr(), ws.numel()
        ops.attn_fused(None, a)
        torch.cuda.synchronize()
        # oracle: a linear cache holding the accepted history and the staged rows
        lin = KVCache(fmt, nkv, L + n, hd)
        if L:
            lin.append(hist_k, hist_v, 0)
        lin.append(new_k, new_v, L)
        klen = int(st.klen)
        want = oracle.attn_exact(q, lin.k, lin.v, lin.ks, lin.vs, lin.kv_fmt, nh, nkv, hd, hd, L + n, S=n, window=W,
                                 query_base_pos=L, win_lo=L + n - klen, softmax_scale=0.1)
        ok, rel = within(host(out), want, 2e-3)
        assert ok, f"step {step_no} (L={L}, n={n}): {rel:.2e} x RMS"
        accepted = n if n == 1 else int(rng.integers(0, n + 1))
        ring.commit(accepted)
        hist_k = np.concatenate([hist_k, new_k[:accepted]]); hist_v = np.concatenate([hist_v, new_v[:accepted]])
    assert ring.len == hist_k.shape[0] and ring.len > cap        # the ring wrapped
