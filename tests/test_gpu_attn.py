"""GPU parity of the attention kernels against the CPU oracle, through the C ABI.

Gate (the parity bar for a re-ordered floating-point reduction): on the fp32
output, max|out - exact| <= 2e-3 * RMS(exact), where `exact` is the oracle's
fp64 attention over the bit-identical quantised cache.  Deviations from the
reference's own lossy realisation (int8 re-quantised Q/P per 32-block) is bounded
loosely in the thin-entry-point tests below, not gated at 2e-3.
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import KVCache, bf16_normal, k_with_outliers, orc
from tests._gpu import DEV, bf16_dev, dev, host, within

pytestmark = pytest.mark.gpu
TOL = 2e-3
SENTINEL = -1.0e30


# Every test that goes through fused() runs three times: on the kernel the library picks, pinned
# to the mma.sync kernel, and on the tcgen05 kernel wherever it supports the call (int8 KV,
# head_dim 128, with or without fused append).
EXTRA_FLAGS = 0


@pytest.fixture(autouse=True, params=["auto", "mma_sync", "tcgen05"])
def kernel_path(request):
    global EXTRA_FLAGS
    EXTRA_FLAGS = {"auto": 0, "mma_sync": ops.NO_TCGEN05, "tcgen05": ops.TCGEN05_ALWAYS}[request.param]
    yield request.param
    EXTRA_FLAGS = 0


def build_cache(fmt, rng, T, nkv, hd, cap=None, outliers=False, cache_hd=None, start=0):
    cap = cap or T
    k = k_with_outliers(rng, T, nkv, hd) if outliers else bf16_normal(rng, (T, nkv, hd))
    v = bf16_normal(rng, (T, nkv, hd))
    c = KVCache(fmt, nkv, cap, hd, cache_hd)
    step = 4096
    for b in range(0, T, step):
        c.append(k[b:b + step], v[b:b + step], start + b)
    return c


def fused(c: KVCache, q, *, S=1, klen, win_start=0, window=0, scale=1.0, q_type=ops.F32, out_type=ops.F32,
          force_splits=0, partial=False, new_k=None, new_v=None, new_base_pos=0):
    nkv, hd = c.nkv, c.l_hd
    nh = q.shape[-2]
    dq = bf16_dev(q) if q_type == ops.BF16 else dev(np.ascontiguousarray(q, np.float32))
    out = torch.full((S, nh, hd), SENTINEL, dtype=torch.bfloat16 if out_type == ops.BF16 else torch.float32, device=DEV)
    part = torch.full((S * nh, hd + 2), SENTINEL, dtype=torch.float32, device=DEV) if partial else None
    dk, dv, dks, dvs = dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)
    a = ops.make_args(q=dq, k_cache=dk, v_cache=dv, k_scales=dks, v_scales=dvs, out=out, partial_out=part,
                      kv_fmt=c.kv_fmt, q_type=q_type, out_type=out_type, S=S, nh=nh, nkv=nkv, kvg=nh // nkv,
                      l_hd=hd, cache_hd=c.cache_hd, cache_cap=c.cache_cap, win_start=win_start, klen=klen,
                      window=window, softmax_scale=scale, force_splits=force_splits, flags=EXTRA_FLAGS)
    if new_k is not None:
        keep = (dev(np.ascontiguousarray(new_k, np.float32)), dev(np.ascontiguousarray(new_v, np.float32)))
        a.new_k, a.new_v, a.n_new, a.new_base_pos = keep[0].data_ptr(), keep[1].data_ptr(), new_k.shape[0], new_base_pos
    ws_bytes = ops.attn_workspace_bytes(a)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = ws.data_ptr(), ws_bytes
    ops.attn_fused(None, a)
    torch.cuda.synchronize()
    res = host(part) if partial else host(out.float())
    caches = (host(dk), host(dv), host(dks), host(dvs))
    return res, caches


def exact(oracle, c: KVCache, q, *, S=1, klen, win_start=0, window=0, scale=1.0, want_partial=False):
    nh = q.shape[-2]
    return oracle.attn_exact(q, c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, c.nkv, c.l_hd, c.cache_hd, c.cache_cap,
                             S=S, window=window, query_base_pos=win_start + klen - S, win_lo=win_start,
                             softmax_scale=scale, want_partial=want_partial)


# ------------------------------------------------------------------ int8 decode

def test_config1_decode_i8(oracle):
    """Configuration 1: 8 q heads / 4 kv heads, hd 128, 512 keys, scale 1/sqrt(128), bf16 Q and output."""
    rng = np.random.default_rng(1001)
    nh, nkv, hd, T = 8, 4, 128, 512
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (1, nh, hd))
    scale = 1.0 / np.sqrt(128.0)
    want = exact(oracle, c, q, klen=T, scale=scale)
    got, _ = fused(c, q, klen=T, scale=scale)
    ok, rel = within(got, want, TOL)
    assert ok, f"fp32 output off by {rel:.2e} x RMS"
    got_bf, _ = fused(c, q, klen=T, scale=scale, q_type=ops.BF16, out_type=ops.BF16)
    want_bf = oracle.bf16_round(want)
    ulp = np.abs(want_bf) * 2.0 ** -7 + 1e-6            # one bf16 ulp of the reference value, generously
    assert np.all(np.abs(got_bf - want_bf) <= ulp + TOL * np.sqrt(np.mean(want ** 2)))


@pytest.mark.parametrize("T", [1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 1023, 1024, 1025, 4097])
def test_decode_i8_lengths(oracle, T):
    rng = np.random.default_rng(T)
    nh, nkv, hd = 8, 4, 128
    c = build_cache("i8", rng, T, nkv, hd, cap=T + 3)
    q = bf16_normal(rng, (1, nh, hd)) * np.float32(0.3)
    want = exact(oracle, c, q, klen=T)
    got, _ = fused(c, q, klen=T)
    ok, rel = within(got, want, TOL)
    assert ok, f"T={T}: {rel:.2e} x RMS"
    assert not np.any(got == SENTINEL), "output not fully written"


def test_decode_i8_many_tiles_per_cta_back_to_back(oracle):
    """One CTA walks 100 tiles of 128 keys (every pipeline stage and barrier phase is reused many
    times), launched several times in a row without a host synchronisation in between."""
    rng = np.random.default_rng(77)
    nh, nkv, hd, T = 4, 2, 128, 12800
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (1, nh, hd)) * np.float32(0.5)
    want = exact(oracle, c, q, klen=T)
    keep = [dev(np.ascontiguousarray(q, np.float32)), dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)]
    for splits in (1, 5):
        out = torch.full((1, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
        a = ops.make_args(q=keep[0], k_cache=keep[1], v_cache=keep[2], k_scales=keep[3], v_scales=keep[4], out=out,
                          kv_fmt=ops.KV_I8, nh=nh, nkv=nkv, kvg=2, l_hd=hd, cache_hd=hd, cache_cap=T, klen=T,
                          force_splits=splits, flags=EXTRA_FLAGS)
        ws = torch.empty(max(ops.attn_workspace_bytes(a), 16), dtype=torch.uint8, device=DEV)
        a.workspace, a.ws_bytes = ws.data_ptr(), ws.numel()
        for _ in range(6):
            ops.attn_fused(None, a)
        torch.cuda.synchronize()
        ok, rel = within(host(out), want, TOL)
        assert ok, f"splits={splits}: {rel:.2e} x RMS"


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 16])
def test_decode_i8_forced_splits_agree(oracle, splits):
    rng = np.random.default_rng(77)
    nh, nkv, hd, T = 32, 16, 128, 2048 + 17
    c = build_cache("i8", rng, T, nkv, hd, outliers=True)
    q = bf16_normal(rng, (1, nh, hd))
    scale = 1.0 / np.sqrt(128.0)
    want = exact(oracle, c, q, klen=T, scale=scale)
    got, _ = fused(c, q, klen=T, scale=scale, force_splits=splits)
    ok, rel = within(got, want, TOL)
    assert ok, f"splits={splits}: {rel:.2e} x RMS"


def test_config2_shape_decode_i8_reduced_context(oracle):
    """Configuration 2's heads and K outliers at a context the oracle finishes in seconds (8192)."""
    rng = np.random.default_rng(1002)
    nh, nkv, hd, T = 32, 16, 128, 8192
    c = build_cache("i8", rng, T, nkv, hd, outliers=True)
    q = bf16_normal(rng, (1, nh, hd))
    scale = 1.0 / np.sqrt(128.0)
    want = exact(oracle, c, q, klen=T, scale=scale)
    got, _ = fused(c, q, klen=T, scale=scale, q_type=ops.BF16)
    ok, rel = within(got, want, TOL)
    assert ok, f"{rel:.2e} x RMS"


def test_decode_i8_peaked_and_flat_softmax(oracle):
    """One dominant key (unscaled scores, sharp softmax) and near-uniform attention."""
    rng = np.random.default_rng(5)
    nh, nkv, hd, T = 8, 4, 128, 3000
    c = build_cache("i8", rng, T, nkv, hd)
    # gain 1: unscaled N(0,1) logits (std ~11, one key dominates); gain 1e-3: flat softmax.
    # gain 3 (logit std ~34) is far outside anything the model produces; there the 16-bit
    # fixed-point query (relative step 2^-15 of the row maximum) shows, so the bar is looser.
    for gain, tol in ((1.0, TOL), (1e-3, TOL), (3.0, 1e-2)):
        q = bf16_normal(rng, (1, nh, hd)) * np.float32(gain)
        want = exact(oracle, c, q, klen=T)
        got, _ = fused(c, q, klen=T)
        ok, rel = within(got, want, tol)
        assert ok, f"gain={gain}: {rel:.2e} x RMS"


def test_decode_i8_ring_window(oracle):
    """A wrapped ring: 3000 positions through 1024 slots, window = last 1024 / last 700 keys."""
    rng = np.random.default_rng(9)
    nh, nkv, hd, cap, T = 8, 4, 128, 1024, 3000
    c = build_cache("i8", rng, T, nkv, hd, cap=cap)
    q = bf16_normal(rng, (1, nh, hd))
    for klen in (1024, 700, 33):
        win_start = T - klen
        want = exact(oracle, c, q, klen=klen, win_start=win_start, scale=0.2)
        got, _ = fused(c, q, klen=klen, win_start=win_start, scale=0.2)
        ok, rel = within(got, want, TOL)
        assert ok, f"klen={klen}: {rel:.2e} x RMS"


def test_decode_i8_wide_cache_rows(oracle):
    """cache_hd (row pitch) wider than the head dim."""
    rng = np.random.default_rng(12)
    nh, nkv, hd, T = 8, 4, 128, 777
    c = build_cache("i8", rng, T, nkv, hd, cache_hd=256)
    q = bf16_normal(rng, (1, nh, hd))
    want = exact(oracle, c, q, klen=T, scale=0.1)
    got, _ = fused(c, q, klen=T, scale=0.1)
    ok, rel = within(got, want, TOL)
    assert ok, f"{rel:.2e} x RMS"


def test_decode_i8_gqa8(oracle):
    """kvg = 8 (the reference's full-attention layers use nkv 4 / kvg 8)."""
    rng = np.random.default_rng(13)
    nh, nkv, hd, T = 32, 4, 128, 1500
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (1, nh, hd))
    want = exact(oracle, c, q, klen=T, scale=0.1)
    got, _ = fused(c, q, klen=T, scale=0.1)
    ok, rel = within(got, want, TOL)
    assert ok, f"{rel:.2e} x RMS"


# ------------------------------------------------------------- thin entry points

def test_thin_decode_i8_matches_reference_signature(oracle):
    """nomos_attn_decode_i8 with the reference's argument list: pitch = max_seq, pre-offset bases."""
    rng = np.random.default_rng(21)
    nh, nkv, hd, max_seq, T, lo = 8, 4, 128, 2048, 1500, 300
    c = build_cache("i8", rng, T, nkv, hd, cap=max_seq)
    q = bf16_normal(rng, (nh, hd))
    klen = T - lo
    want = exact(oracle, c, q[None], klen=klen, win_start=lo)[0]
    dk, dv = dev(c.k), dev(c.v)
    dks, dvs = dev(c.ks).view(torch.float32), dev(c.vs).view(torch.float32)
    scratch = torch.empty(nh * klen, dtype=torch.float32, device=DEV)
    out = torch.full((nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    ops.attention_gpu_int8_dev(None, dev(q), dk.data_ptr() + lo * hd, dv.data_ptr() + lo * hd,
                               dks.data_ptr() + lo * 4, dvs.data_ptr() + lo * 4, scratch, out,
                               nh, nkv, hd, hd, max_seq, klen, nh // nkv)
    torch.cuda.synchronize()
    ok, rel = within(host(out), want, TOL)
    assert ok, f"{rel:.2e} x RMS"
    # The reference's own int8 route re-quantises Q and P to 8 bits per 32 block and sits 4-7 % of
    # RMS away from exact arithmetic on inputs like these; the library must stay at least that close to it.
    sc = np.zeros((nh, klen), np.float32); ref_out = np.zeros((nh, hd), np.float32)
    oracle.attn_decode_int8(q, c.k.reshape(-1)[lo * hd:], c.v.reshape(-1)[lo * hd:],
                            c.ks.view(np.float32)[lo:], c.vs.view(np.float32)[lo:], sc, ref_out,
                            nh, nkv, hd, hd, max_seq, klen, nh // nkv)
    assert within(host(out), ref_out, 0.15)[0]


@pytest.mark.parametrize("S,window", [(1, 0), (9, 0), (9, 1024), (17, 0), (4, 100)])
def test_thin_multirow_i8(oracle, S, window):
    """Verify rows: row r attends absolute keys [max(0,apos-window+1), apos], apos = qbase + r."""
    rng = np.random.default_rng(31 + S)
    nh, nkv, hd, max_seq, qbase = 8, 4, 128, 2048, 1200
    T = qbase + S
    c = build_cache("i8", rng, T, nkv, hd, cap=max_seq)
    q = bf16_normal(rng, (S, nh, hd)) * np.float32(0.5)
    want = exact(oracle, c, q, S=S, klen=T, window=window)
    stride = T
    scores = torch.empty(S * nh * stride, dtype=torch.float32, device=DEV)
    out = torch.full((S, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    ops.attention_decode_order_multirow_int8(None, dev(q), scores, out, dev(c.k), dev(c.v),
                                             dev(c.ks).view(torch.float32), dev(c.vs).view(torch.float32),
                                             nh, nkv, hd, hd, max_seq, S, stride, nh // nkv, window, qbase)
    torch.cuda.synchronize()
    got = host(out)
    assert not np.any(got == SENTINEL)
    for r in range(S):
        ok, rel = within(got[r], want[r], TOL)
        assert ok, f"row {r}: {rel:.2e} x RMS"


def test_config4_shape_verify_reduced_context(oracle):
    """Configuration 4: VB=9 rows x 32/16 heads, int8 KV, bf16 Q, at 4096 cached keys."""
    rng = np.random.default_rng(1004)
    nh, nkv, hd, S, T0 = 32, 16, 128, 9, 4096
    T = T0 + S
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (S, nh, hd))
    scale = 1.0 / np.sqrt(128.0)
    want = exact(oracle, c, q, S=S, klen=T, scale=scale)
    got, _ = fused(c, q, S=S, klen=T, scale=scale, q_type=ops.BF16)
    for r in range(S):
        ok, rel = within(got[r], want[r], TOL)
        assert ok, f"row {r}: {rel:.2e} x RMS"


# ------------------------------------------------------------ fused append + attend

def test_fused_append_then_attend_i8(oracle):
    rng = np.random.default_rng(41)
    nh, nkv, hd, cap, T = 8, 4, 128, 1024, 2500
    c = build_cache("i8", rng, T - 1, nkv, hd, cap=cap)
    new_k, new_v = bf16_normal(rng, (1, nkv, hd)), bf16_normal(rng, (1, nkv, hd))
    q = bf16_normal(rng, (1, nh, hd))
    klen = min(T, cap)
    got, caches = fused(c, q, klen=klen, win_start=T - klen, scale=0.1, new_k=new_k, new_v=new_v, new_base_pos=T - 1)
    c.append(new_k, new_v, T - 1)                       # oracle appends, then attends
    want = exact(oracle, c, q, klen=klen, win_start=T - klen, scale=0.1)
    ok, rel = within(got, want, TOL)
    assert ok, f"{rel:.2e} x RMS"
    assert np.array_equal(caches[0].view(np.uint8), c.k.view(np.uint8)) and np.array_equal(caches[2], c.ks)
    assert np.array_equal(caches[1].view(np.uint8), c.v.view(np.uint8)) and np.array_equal(caches[3], c.vs)


@pytest.mark.parametrize("pinned", [True, False])
def test_host_buffer_step_matches_device_call(oracle, pinned):
    """nomos_attn_fused_host: query and new rows arrive in host memory, the output lands there; the
    result and the appended cache rows equal those of the device-buffer call.  Pinned buffers are
    read and written by the kernel directly, pageable ones go through the staging copies."""
    rng = np.random.default_rng(43)
    nh, nkv, hd, cap, T = 8, 4, 128, 512, 400
    c = build_cache("i8", rng, T - 1, nkv, hd, cap=cap)
    new_k, new_v = bf16_normal(rng, (1, nkv, hd)), bf16_normal(rng, (1, nkv, hd))
    q = bf16_normal(rng, (1, nh, hd))
    qb, kb = nh * hd * 4, nkv * hd * 4
    host_in = torch.empty(qb + 2 * kb, dtype=torch.uint8)
    host_in = host_in.pin_memory() if pinned else host_in
    host_in[:qb].view(torch.float32).copy_(torch.from_numpy(np.ascontiguousarray(q, np.float32)).reshape(-1))
    host_in[qb:qb + kb].view(torch.float32).copy_(torch.from_numpy(np.ascontiguousarray(new_k, np.float32)).reshape(-1))
    host_in[qb + kb:].view(torch.float32).copy_(torch.from_numpy(np.ascontiguousarray(new_v, np.float32)).reshape(-1))
    dev_in = torch.zeros_like(host_in, device=DEV)
    host_out = torch.full((1, nh, hd), SENTINEL, dtype=torch.float32)
    host_out = host_out.pin_memory() if pinned else host_out
    dev_out = torch.zeros((1, nh, hd), dtype=torch.float32, device=DEV)
    dk, dv, dks, dvs = dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)
    a = ops.make_args(q=dev_in.data_ptr(), k_cache=dk, v_cache=dv, k_scales=dks, v_scales=dvs, out=dev_out, kv_fmt=ops.KV_I8,
                      nh=nh, nkv=nkv, kvg=2, l_hd=hd, cache_hd=hd, cache_cap=cap, klen=T, softmax_scale=0.1,
                      new_k=dev_in.data_ptr() + qb, new_v=dev_in.data_ptr() + qb + kb, n_new=1, new_base_pos=T - 1,
                      flags=EXTRA_FLAGS)
    ws = torch.empty(max(ops.attn_workspace_bytes(a), 16), dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = ws.data_ptr(), ws.numel()
    ops.attn_fused_host(None, a, host_in, dev_in, host_in.numel(), host_out, dev_out, host_out.numel() * 4)
    got = host_out.numpy().copy()                       # no synchronise here: the call returns with the data in place
    c.append(new_k, new_v, T - 1)
    want = exact(oracle, c, q, klen=T, scale=0.1)
    ok, rel = within(got, want, TOL)
    assert ok, f"{rel:.2e} x RMS"
    assert np.array_equal(host(dk).view(np.uint8), c.k.view(np.uint8)) and np.array_equal(host(dks), c.ks)


# ------------------------------------------------------- partial export and merge

def test_partials_merge_equals_full(oracle):
    """Sequence-sharded decode: G shards export (o, m, l); the merge equals full attention."""
    rng = np.random.default_rng(51)
    nh, nkv, hd, T, G = 8, 4, 128, 4000, 4
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (1, nh, hd))
    want = exact(oracle, c, q, klen=T, scale=0.15)
    chunk = T // G
    parts = []
    for g in range(G):
        # shard g owns positions [g*chunk, (g+1)*chunk): a window of the same cache
        p, _ = fused(c, q, klen=chunk, win_start=g * chunk, scale=0.15, partial=True)
        # every key of the shard is visible to the (single) query row: causal bound = shard end
        parts.append(p)
    parts = np.stack(parts)                              # [G, nh, hd+2]
    d_parts = dev(parts)
    out = torch.full((nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    ops.attn_merge_partials(None, d_parts, G, nh, hd, out)
    torch.cuda.synchronize()
    ok, rel = within(host(out)[None], want, TOL)
    assert ok, f"{rel:.2e} x RMS"
    # and the exported triples are valid against the oracle's merge
    merged = oracle.merge_partials(parts.astype(np.float64), hd)
    assert within(merged[None], want, TOL)[0]


# ---------------------------------------------------------------- error behaviour

def test_bad_arguments_return_status_not_fault():
    t = torch.zeros(1024, dtype=torch.float32, device=DEV)
    with pytest.raises(ops.NomosError) as e:
        ops.attention_gpu_int8_dev(None, t, t, t, t, t, t, t, 8, 4, 128, 128, 64, 16, 3)   # nh != nkv*kvg
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:
        ops.attention_gpu_int8_dev(None, t, t, t, t, t, t, t, 8, 4, 96, 96, 64, 16, 2)     # head_dim 96
    assert e.value.status == -2
    with pytest.raises(ops.NomosError) as e:
        ops.attention_gpu_int8_dev(None, t, 0, t, t, t, t, t, 8, 4, 128, 128, 64, 16, 2)    # null K
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:
        ops.attention_gpu_int8_dev(None, t, t, t, t, t, t, t, 8, 4, 128, 128, 64, 65, 2)    # seq_len > pitch
    assert e.value.status == -3
    ops.attention_gpu_int8_dev(None, t, t, t, t, t, t, t, 0, 4, 128, 128, 64, 16, 2)        # nh <= 0: no-op, ok
    ops.attention_gpu_int8_dev(None, t, t, t, t, t, t, t, 8, 4, 128, 128, 64, 0, 2)         # seq_len <= 0: no-op
    torch.cuda.synchronize()


def test_settled_cache_flag_gives_identical_output(oracle):
    """The flag only moves the first cache reads ahead of the stream-order wait; results are the same."""
    rng = np.random.default_rng(61)
    nh, nkv, hd, T = 32, 16, 128, 5000
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (1, nh, hd))
    keep = [dev(q), dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)]
    outs = []
    for flags in (0, ops.SETTLED_CACHE):
        out = torch.full((1, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
        a = ops.make_args(q=keep[0], k_cache=keep[1], v_cache=keep[2], k_scales=keep[3], v_scales=keep[4], out=out,
                          kv_fmt=ops.KV_I8, nh=nh, nkv=nkv, kvg=2, l_hd=hd, cache_hd=hd, cache_cap=T, klen=T,
                          softmax_scale=0.1, flags=flags)
        ws = torch.empty(max(ops.attn_workspace_bytes(a), 16), dtype=torch.uint8, device=DEV)
        a.workspace, a.ws_bytes = ws.data_ptr(), ws.numel()
        for _ in range(3):                      # back-to-back launches exercise the programmatic dependency chain
            ops.attn_fused(None, a)
        torch.cuda.synchronize()
        outs.append(host(out))
    assert np.array_equal(outs[0], outs[1])
    want = exact(oracle, c, q, klen=T, scale=0.1)
    assert within(outs[1], want, TOL)[0]


@pytest.mark.parametrize("fmt,hd,win_start", [("i8", 128, 0), ("i8", 128, 1237), ("i4", 128, 0), ("i4b32", 128, 5), ("i4", 256, 0)])
def test_tma_and_cp_async_copy_paths_agree(oracle, fmt, hd, win_start):
    """Whole tiles come by TMA tensor copies, ragged / ring-wrapping ones by cp.async; forcing
    everything onto cp.async must not change a bit.  Odd window starts make the scale rows
    miss the 16-byte rule of the bulk copy (scales then ride cp.async beside a TMA tile)."""
    rng = np.random.default_rng(600 + hd + win_start)
    nkv, kvg, T = 4, 2, 3000
    nh = nkv * kvg
    cap = 4096 if win_start else T
    c = build_cache(fmt, rng, T, nkv, hd, cap=cap, start=win_start)
    q = bf16_normal(rng, (1, nh, hd))
    keep = [dev(q), dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)]
    outs = []
    for flags in (ops.NO_TCGEN05, ops.NO_TCGEN05 | ops.NO_TMA):      # both on the mma.sync kernel
        out = torch.full((1, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
        a = ops.make_args(q=keep[0], k_cache=keep[1], v_cache=keep[2], k_scales=keep[3], v_scales=keep[4], out=out,
                          kv_fmt=c.kv_fmt, nh=nh, nkv=nkv, kvg=kvg, l_hd=hd, cache_hd=hd, cache_cap=cap, klen=T,
                          win_start=win_start, softmax_scale=0.1, flags=flags)
        ws = torch.empty(max(ops.attn_workspace_bytes(a), 16), dtype=torch.uint8, device=DEV)
        a.workspace, a.ws_bytes = ws.data_ptr(), ws.numel()
        ops.attn_fused(None, a)
        torch.cuda.synchronize()
        outs.append(host(out))
    assert np.array_equal(outs[0], outs[1])
    want = exact(oracle, c, q, klen=T, win_start=win_start, scale=0.1)
    assert within(outs[0], want, TOL)[0]


@pytest.mark.parametrize("S,kvg", [(17, 2), (9, 8), (4, 8)])
def test_many_verify_rows(oracle, S, kvg):
    """More than 24 query rows per KV head (the 24-row CTA path) and wide GQA groups."""
    rng = np.random.default_rng(S * 10 + kvg)
    nkv, hd, T = 2, 128, 900
    nh = nkv * kvg
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (S, nh, hd)) * np.float32(0.5)
    want = exact(oracle, c, q, S=S, klen=T, scale=0.2)
    got, _ = fused(c, q, S=S, klen=T, scale=0.2)
    for r in range(S):
        ok, rel = within(got[r], want[r], TOL)
        assert ok, f"row {r}: {rel:.2e} x RMS"


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8, 9, 12, 13, 17])
def test_verify_forced_splits_cover_every_merge_path(oracle, splits):
    """18 query rows per KV head merged from 1..17 splits: no merge, the barrier-free paired merge with
    capacities 4 / 8 / 12 and the staged merge (more than 12 splits); the tile counts per CTA (and per
    softmax group of the tcgen05 kernel, which takes tiles in turn) are odd, even and 1."""
    rng = np.random.default_rng(500 + splits)
    nh, nkv, hd, S, T0 = 4, 2, 128, 9, 2300
    T = T0 + S
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (S, nh, hd))
    scale = 1.0 / np.sqrt(128.0)
    want = exact(oracle, c, q, S=S, klen=T, scale=scale)
    got, _ = fused(c, q, S=S, klen=T, scale=scale, q_type=ops.BF16, force_splits=splits)
    for r in range(S):
        ok, rel = within(got[r], want[r], TOL)
        assert ok, f"row {r}: {rel:.2e} x RMS"
    gotb, _ = fused(c, q, S=S, klen=T, scale=scale, q_type=ops.BF16, out_type=ops.BF16, force_splits=splits)
    # the bf16 store of the same path: the fp32 result rounded once
    assert np.all(np.abs(gotb - got) <= np.abs(got) * 2.0 ** -8 + 1e-30)


@pytest.mark.parametrize("S,big", [(1, 30.0), (9, 30.0), (9, 1e-3), (3, 200.0)])
def test_query_rows_of_very_different_magnitude(oracle, S, big):
    """Query rows that share a CTA (the heads of a GQA group, the tokens of a verify step) but differ in
    magnitude by 30x .. 1000x: every row is quantised with its own fixed-point scale, so each must pass the
    gate separately, against its own RMS.  The softmax scale keeps the largest rows' logits moderate
    (standard deviation about 7): beyond that the 16-bit query itself limits any kernel."""
    rng = np.random.default_rng(int(S * 1000 + big))
    nh, nkv, hd, T0 = 4, 2, 128, 1500
    T = T0 + S
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (S, nh, hd))
    q[:, 0::2, :] *= np.float32(big)                          # one head of every GQA pair (and every token of it)
    if S > 1:
        q[S // 2, 1, :] *= np.float32(big)                    # and one token of the other head
    q = orc.bf16_round(q)
    scale = 0.6 / max(big, 1.0)
    want = exact(oracle, c, q, S=S, klen=T, scale=scale)
    got, _ = fused(c, q, S=S, klen=T, scale=scale)
    for r in range(S):
        for h in range(nh):
            ok, rel = within(got[r][h], want[r][h], TOL)
            assert ok, f"row {r} head {h}: {rel:.2e} x RMS"


def test_kernel_choice_follows_the_cost_model(kernel_path):
    """nomos_attn_kernel_choice: short decode calls go to the mma.sync kernel, verify and calls streaming more
    than about 330 MB to the tcgen05 kernel; the flag bits override; int4 caches have one kernel."""
    def choice(S, klen, batch=1, fmt=ops.KV_I8, flags=0, hd=128):
        a = ops.make_args(q=0x1000, k_cache=0x10000, v_cache=0x20000, k_scales=0x30000, v_scales=0x40000, out=0x50000,
                          kv_fmt=fmt, q_type=ops.BF16, out_type=ops.BF16, batch=batch, S=S, nh=32, nkv=16, kvg=2, l_hd=hd,
                          cache_hd=hd, cache_cap=klen, klen=klen, softmax_scale=0.1, flags=flags)
        return ops.attn_kernel_choice(a)
    assert choice(1, 32768) == 0
    assert choice(1, 32768, flags=ops.TCGEN05_ALWAYS) == 1
    assert choice(1, 131072) == 1
    assert choice(1, 131072, flags=ops.NO_TCGEN05) == 0
    assert choice(1, 131072, batch=8) == 1
    assert choice(9, 16393) == 1
    assert choice(9, 16393, flags=ops.NO_TCGEN05) == 0
    assert choice(1, 32768, fmt=ops.KV_I4B32) == 0
    assert choice(1, 32768, hd=256) == 0
