"""GPU parity of the prefill attention (many query rows, causal + sliding-window masks, no S x key_len scratch).

int8 caches at head_dim 128 run on the query-major tcgen05 kernel (128 query rows per CTA); int4 / block-32 caches,
wider heads and wrapped rings run as row groups of the mma.sync kernel.  Both are checked against the oracle's fp64
attention over the same cache bytes, every query row against its own RMS (2e-3), through the fused entry point and
through the reference's square / prefix operators (lib/attention_gpu_int8.mojo:804-887).
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import bf16_normal
from tests._gpu import DEV, bf16_dev, dev, host, within
from tests.test_gpu_attn import build_cache

pytestmark = pytest.mark.gpu
TOL = 2e-3
SENTINEL = -1.0e30


def run_fused(c, q, *, S, klen, win_start=0, window=0, scale, flags=0, q_type=ops.F32, out_type=ops.F32, batch=1):
    nh = q.shape[-2]
    dq = bf16_dev(q) if q_type == ops.BF16 else dev(np.ascontiguousarray(q, np.float32))
    out = torch.full((batch, S, nh, c.l_hd), SENTINEL, dtype=torch.bfloat16 if out_type == ops.BF16 else torch.float32, device=DEV)
    keep = [dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)]
    a = ops.make_args(q=dq, k_cache=keep[0], v_cache=keep[1], k_scales=keep[2], v_scales=keep[3], out=out, kv_fmt=c.kv_fmt,
                      q_type=q_type, out_type=out_type, batch=batch, S=S, nh=nh, nkv=c.nkv, kvg=nh // c.nkv, l_hd=c.l_hd,
                      cache_hd=c.cache_hd, cache_cap=c.cache_cap, win_start=win_start, klen=klen, window=window,
                      softmax_scale=scale, flags=flags)
    choice = ops.attn_kernel_choice(a)
    need = ops.attn_workspace_bytes(a)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = ws.data_ptr(), need
    ops.attn_fused(None, a)
    torch.cuda.synchronize()
    return host(out.float()), choice


def check_rows(got, want, S, tol=TOL, what=""):
    worst = 0.0
    for r in range(S):
        ok, rel = within(got[r], want[r], tol)
        worst = max(worst, rel)
        assert ok, f"{what} row {r}: {rel:.2e} x RMS"
    return worst


@pytest.mark.parametrize("fmt", ["i8", "i4b32"])
@pytest.mark.parametrize("S,window", [(1, 0), (17, 0), (128, 0), (128, 40), (1000, 0), (1000, 300), (2900, 0), (2900, 1024)])
def test_square_prefill_sizes_and_windows(oracle, fmt, S, window):
    """S query rows over the S keys at 0..S-1 (what a prompt of S tokens does), with and without a sliding window."""
    rng = np.random.default_rng(S + window + (7 if fmt == "i8" else 11))
    nh, nkv, hd = 4, 2, 128
    c = build_cache(fmt, rng, S, nkv, hd)
    q = bf16_normal(rng, (S, nh, hd))
    scale = 1.0 / np.sqrt(hd)
    want = oracle.attn_exact(q, c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, S, S=S, window=window, query_base_pos=0,
                             win_lo=0, softmax_scale=scale)
    got, choice = run_fused(c, q, S=S, klen=S, window=window, scale=scale)
    assert choice == (2 if fmt == "i8" and S * 2 > 24 else choice)
    assert not np.any(got == SENTINEL)
    check_rows(got[0], want, S, what=f"{fmt} S={S} W={window}")


@pytest.mark.parametrize("kvg", [1, 2, 4, 8])
def test_prefill_group_sizes_and_a_prefix_already_in_the_cache(oracle, kvg):
    """A chunk of S rows appended behind T0 cached keys (chunked prefill), for every GQA group size; the tcgen05
    prefill kernel and the mma.sync row-group path must both pass, and agree with each other loosely."""
    rng = np.random.default_rng(50 + kvg)
    nkv, hd, T0, S = 2, 128, 700, 333
    nh = nkv * kvg
    c = build_cache("i8", rng, T0 + S, nkv, hd, cap=T0 + S + 9)
    q = bf16_normal(rng, (S, nh, hd))
    scale = 1.0 / np.sqrt(hd)
    want = oracle.attn_exact(q, c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, c.cache_cap, S=S, window=0, query_base_pos=T0,
                             win_lo=0, softmax_scale=scale)
    got, choice = run_fused(c, q, S=S, klen=T0 + S, scale=scale)
    assert choice == 2
    check_rows(got[0], want, S, what=f"kvg={kvg} prefill kernel")
    got2, choice2 = run_fused(c, q, S=S, klen=T0 + S, scale=scale, flags=ops.NO_TCGEN05)
    assert choice2 == 0
    check_rows(got2[0], want, S, what=f"kvg={kvg} mma.sync row groups")


def test_prefill_bf16_in_and_out_batched_with_window_start(oracle):
    """bf16 query and output, two sequences in one call, a window that starts inside a larger ring (no wrap)."""
    rng = np.random.default_rng(77)
    nh, nkv, hd, S, start, cap, B = 8, 4, 128, 200, 150, 512, 2
    caches = [build_cache("i8", rng, S, nkv, hd, cap=cap, start=start) for _ in range(B)]
    q = bf16_normal(rng, (B, S, nh, hd))
    scale = 1.0 / np.sqrt(hd)
    class Both:                                   # the two sequences' caches stacked along the batch dimension
        pass
    c = Both()
    c.k = np.stack([x.k for x in caches]); c.v = np.stack([x.v for x in caches])
    c.ks = np.stack([x.ks for x in caches]); c.vs = np.stack([x.vs for x in caches])
    c.kv_fmt, c.nkv, c.l_hd, c.cache_hd, c.cache_cap = caches[0].kv_fmt, nkv, hd, hd, cap
    got, choice = run_fused(c, q, S=S, klen=S, win_start=start, window=64, scale=scale, q_type=ops.BF16, out_type=ops.BF16, batch=B)
    assert choice == 2
    for b in range(B):
        want = oracle.attn_exact(q[b], caches[b].k, caches[b].v, caches[b].ks, caches[b].vs, caches[b].kv_fmt, nh, nkv, hd, hd, cap,
                                 S=S, window=64, query_base_pos=start, win_lo=start, softmax_scale=scale)
        for r in range(S):
            wb = oracle.bf16_round(want[r])
            tol = np.abs(wb) * 2.0 ** -7 + 1e-6 + TOL * np.sqrt(np.mean(want[r] ** 2))
            assert np.all(np.abs(got[b][r] - wb) <= tol), f"sequence {b} row {r}"


@pytest.mark.parametrize("S,key_len,window,qbase,kbase", [
    (100, 140, 0, 100, 70),      # the key array ends before the last query rows: they all see up to key 139
    (60, 200, 0, 10, 33),        # the first rows sit before the first key: no key, zero output
    (300, 64, 0, 0, 0),          # far more queries than keys
    (90, 150, 50, 100, 40),      # windowed, clipped at both ends
])
def test_prefix_operator_ranges_only_the_prefill_kernel_expresses(oracle, S, key_len, window, qbase, kbase):
    """attention_prefill_prefix_batched_int8 with key arrays that do not end at the last query row
    (lib/batched_attn_gpu.mojo:314-326 bounds; empty ranges give all-zero rows)."""
    rng = np.random.default_rng(S + key_len + window)
    nh, nkv, hd, max_seq = 8, 4, 128, key_len + 5
    c = build_cache("i8", rng, key_len, nkv, hd, cap=max_seq)
    q = bf16_normal(rng, (S, nh, hd)) * np.float32(0.3)
    scores = torch.empty(16, dtype=torch.float32, device=DEV)
    out = torch.full((S, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    ops.attention_prefill_prefix_batched_int8(None, dev(q), 0, scores, 0, out, dev(c.k), dev(c.v), dev(c.ks).view(torch.float32),
                                              dev(c.vs).view(torch.float32), nh, nkv, hd, hd, max_seq, S, key_len, nh // nkv, window,
                                              qbase, kbase)
    torch.cuda.synchronize()
    got = host(out)
    assert not np.any(got == SENTINEL)
    for s in range(S):
        q_abs = qbase + s
        hi = min(q_abs - kbase, key_len - 1)
        lo = max(0, (max(0, q_abs - window + 1) if window > 0 else 0) - kbase)
        if hi < lo:
            assert np.all(got[s] == 0.0), f"row {s}: empty key range must give zeros"
            continue
        want = oracle.attn_exact(q[s:s + 1], c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, max_seq, S=1, window=0,
                                 query_base_pos=hi, win_lo=lo)
        ok, rel = within(got[s], want[0], TOL)
        assert ok, f"row {s} keys [{lo},{hi}]: {rel:.2e} x RMS"


def test_prefill_back_to_back_launches_reuse_everything(oracle):
    """Several prefill launches in a row without host synchronisation (tensor memory, barriers and the programmatic
    dependency chain are set up again by every CTA)."""
    rng = np.random.default_rng(91)
    nh, nkv, hd, S = 8, 4, 128, 500
    c = build_cache("i8", rng, S, nkv, hd)
    q = bf16_normal(rng, (S, nh, hd))
    scale = 1.0 / np.sqrt(hd)
    want = oracle.attn_exact(q, c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, S, S=S, window=0, query_base_pos=0, win_lo=0,
                             softmax_scale=scale)
    keep = [dev(np.ascontiguousarray(q, np.float32)), dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)]
    outs = [torch.full((S, nh, hd), SENTINEL, dtype=torch.float32, device=DEV) for _ in range(4)]
    for o in outs:
        a = ops.make_args(q=keep[0], k_cache=keep[1], v_cache=keep[2], k_scales=keep[3], v_scales=keep[4], out=o, kv_fmt=ops.KV_I8,
                          S=S, nh=nh, nkv=nkv, kvg=2, l_hd=hd, cache_hd=hd, cache_cap=S, klen=S, softmax_scale=scale)
        ops.attn_fused(None, a)
    torch.cuda.synchronize()
    for o in outs:
        check_rows(host(o), want, S)
    assert ops.device_faults() == 0
