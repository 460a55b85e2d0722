"""GPU parity of the attention over UNQUANTISED (fp32 / bf16) KV caches, through the C ABI.

Covers the legacy KV modes of the reference: single-token decode (lib/attention_gpu.mojo:165-248), the
prefix-batched operators with their own argument lists (lib/batched_attn_gpu.mojo:499-548, 613-666) and the
square causal forms (:448-496, 558-610), including the mask rules of lib/batched_attn_gpu.mojo:285-409:
sliding windows, a key array that starts at key_base_pos > 0, key arrays that end before the last query row,
and rows whose key range is empty (their output is exactly zero).

Gate: max|out - exact| <= 2e-3 x RMS(exact) on the fp32 output, `exact` = float64 attention over the stored
values (bf16 widens exactly).  The reference's bf16 operators also narrow Q and the softmax weights to bf16
before their GEMMs; the distance of that literal restatement (the oracle's attn_*_dense with kv_is_bf16) from
exact arithmetic is printed and bounded loosely, not gated: it is a property of the reference's route, not of
this library.
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import bf16_normal, orc
from tests._gpu import DEV, dev, host, within

pytestmark = pytest.mark.gpu
TOL = 2e-3
SENTINEL = -1.0e30


def make_dense_cache(rng, nkv, max_seq, hd, cache_hd, T, bf16):
    """K, V [nkv, max_seq, cache_hd]: fp32 arrays holding the stored values, plus the device tensors."""
    k = np.zeros((nkv, max_seq, cache_hd), np.float32); v = np.zeros_like(k)
    k[:, :T, :hd] = bf16_normal(rng, (nkv, T, hd)) if bf16 else rng.standard_normal((nkv, T, hd), dtype=np.float32)
    v[:, :T, :hd] = bf16_normal(rng, (nkv, T, hd)) if bf16 else rng.standard_normal((nkv, T, hd), dtype=np.float32)
    k[:, T:, :] = 1e4; v[:, T:, :] = 1e4          # rows past the valid keys must never be read into a result
    if bf16:
        dk = torch.from_numpy(k).to(DEV).to(torch.bfloat16); dv = torch.from_numpy(v).to(DEV).to(torch.bfloat16)
    else:
        dk, dv = dev(k), dev(v)
    return k, v, dk, dv


def exact_dense(q, k, v, kvg, lo_hi):
    """float64 attention; q [S, nh, hd], k/v [nkv, T, >=hd]; lo_hi(s) -> inclusive key range of row s or None."""
    S, nh, hd = q.shape
    out = np.zeros((S, nh, hd), np.float64)
    for s in range(S):
        rng_ = lo_hi(s)
        if rng_ is None:
            continue
        lo, hi = rng_
        for h in range(nh):
            kk = k[h // kvg, lo:hi + 1, :hd].astype(np.float64); vv = v[h // kvg, lo:hi + 1, :hd].astype(np.float64)
            sc = kk @ q[s, h].astype(np.float64)
            w = np.exp(sc - sc.max())
            out[s, h] = (w / w.sum()) @ vv
    return out.astype(np.float32)


def prefix_range(S, key_len, window, qbase, kbase):
    """lib/batched_attn_gpu.mojo:314-326"""
    def f(s):
        q_abs = qbase + s
        hi = min(q_abs - kbase, key_len - 1)
        lo_abs = max(0, q_abs - window + 1) if window > 0 else 0
        lo = max(0, lo_abs - kbase)
        return (lo, hi) if hi >= lo else None
    return f


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("nh,nkv,hd,T", [(8, 4, 128, 1500), (32, 16, 128, 4097), (8, 2, 256, 700), (8, 1, 512, 333), (4, 4, 128, 1)])
def test_decode_fp32_and_bf16_caches(oracle, bf16, nh, nkv, hd, T):
    """attention_gpu_fp32_dev / attention_gpu_bf16_dev with the reference's argument lists; no softmax scale."""
    rng = np.random.default_rng(hd + T + bf16)
    max_seq, kvg = T + 5, nh // nkv
    k, v, dk, dv = make_dense_cache(rng, nkv, max_seq, hd, hd, T, bf16)
    q = (bf16_normal(rng, (nh, hd)) * np.float32(0.25)).astype(np.float32)
    scratch = torch.empty(nh * T, dtype=torch.float32, device=DEV)
    out = torch.full((nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    if bf16:
        ops.attention_gpu_bf16_dev(None, 0, dev(q), dk, dv, scratch, 0, 0, out, nh, nkv, hd, hd, max_seq, T, kvg)
    else:
        ops.attention_gpu_fp32_dev(None, 0, dev(q), dk, dv, scratch, out, nh, nkv, hd, hd, max_seq, T, kvg)
    torch.cuda.synchronize()
    got = host(out)
    assert not np.any(got == SENTINEL)
    want = exact_dense(q[None], k, v, kvg, lambda s: (0, T - 1))[0]
    ok, rel = within(got, want, TOL)
    assert ok, f"{rel:.2e} x RMS"
    # the reference's literal route (Q and P narrowed to bf16 for the bf16 cache): reported, loosely bounded
    sc = np.zeros((nh, T), np.float32); lit = np.zeros((nh, hd), np.float32)
    kk = orc.f32_to_bf16(k) if bf16 else k
    vv = orc.f32_to_bf16(v) if bf16 else v
    oracle.attn_decode_dense(q, kk, vv, sc, lit, nh, nkv, hd, hd, max_seq, T, kvg, bf16)
    _, rel_lit = within(lit, want, 1.0)
    print(f"literal {'bf16' if bf16 else 'fp32'} route vs exact: {rel_lit:.2e} x RMS; library vs exact: {rel:.2e}")
    assert within(got, lit, 5e-2)[0]


CASES = [
    # S, key_len, window, query_base_pos, key_base_pos
    (9, 1209, 0, 1200, 0),          # verify rows at the end of a linear cache
    (9, 1209, 512, 1200, 0),        # sliding window, array from position 0
    (9, 520, 512, 1200, 689),       # the engine's call above the window: pointers pre-offset by key_base
    (7, 300, 0, 0, 0),              # key array longer than the causal range (rows see [0, s])
    (16, 16, 0, 0, 0),              # square
    (16, 16, 5, 0, 0),              # square, windowed
    (12, 40, 0, 100, 70),           # key array ends before the last query rows: they all see up to key 39
    (6, 50, 0, 10, 13),             # the first rows sit before the first key: empty ranges, zero output
    (1, 64, 0, 63, 0),              # a single row
]


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("S,key_len,window,qbase,kbase", CASES)
def test_prefix_batched_fp32_and_bf16(oracle, bf16, S, key_len, window, qbase, kbase):
    """attention_prefill_prefix_batched_fp32 / _bf16: every mask rule, against float64 and the literal restatement."""
    rng = np.random.default_rng(S * 7 + key_len + window + bf16)
    nh, nkv, hd, max_seq = 8, 4, 128, key_len + 3
    kvg = nh // nkv
    k, v, dk, dv = make_dense_cache(rng, nkv, max_seq, hd, hd, key_len, bf16)
    q = (bf16_normal(rng, (S, nh, hd)) * np.float32(0.25)).astype(np.float32)
    scores = torch.empty(S * nh * key_len, dtype=torch.float32, device=DEV)
    out = torch.full((S, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    if bf16:
        ops.attention_prefill_prefix_batched_bf16(None, 0, dev(q), 0, 0, scores, 0, 0, out, dk, dv, nh, nkv, hd, hd, max_seq, S,
                                                  key_len, kvg, window, qbase, kbase)
    else:
        ops.attention_prefill_prefix_batched_fp32(None, 0, dev(q), 0, scores, 0, out, dk, dv, nh, nkv, hd, hd, max_seq, S,
                                                  key_len, kvg, window, qbase, kbase)
    torch.cuda.synchronize()
    got = host(out)
    assert not np.any(got == SENTINEL)
    f = prefix_range(S, key_len, window, qbase, kbase)
    want = exact_dense(q, k, v, kvg, f)
    for s in range(S):
        if f(s) is None:
            assert np.all(got[s] == 0.0), f"row {s}: an empty key range must give an all-zero row"
            continue
        ok, rel = within(got[s], want[s], TOL)
        assert ok, f"row {s}: {rel:.2e} x RMS"
    # literal restatement of the reference's masked softmax (scores matrix and all)
    sc = np.zeros((nkv * S * kvg, key_len), np.float32); lit = np.zeros((S, nh, hd), np.float32)
    kk = orc.f32_to_bf16(k) if bf16 else k
    vv = orc.f32_to_bf16(v) if bf16 else v
    oracle.attn_prefix_batched_dense(q, kk, vv, sc, lit, nh, nkv, hd, hd, max_seq, S, key_len, kvg, window, qbase, kbase, bf16)
    assert within(got, lit, 5e-2 if bf16 else 1e-3)[0]


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("window", [0, 33])
def test_square_batched_fp32_and_bf16(oracle, bf16, window):
    """attention_prefill_batched_fp32 / _bf16 (lib/batched_attn_gpu.mojo:448, 558): S rows over the S keys at 0..S-1."""
    rng = np.random.default_rng(90 + window + bf16)
    nh, nkv, hd, S, max_seq = 8, 2, 128, 150, 160
    kvg = nh // nkv
    k, v, dk, dv = make_dense_cache(rng, nkv, max_seq, hd, hd, S, bf16)
    q = (bf16_normal(rng, (S, nh, hd)) * np.float32(0.25)).astype(np.float32)
    scores = torch.empty(S * nh * S, dtype=torch.float32, device=DEV)
    out = torch.full((S, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    if bf16:
        ops.attention_prefill_batched_bf16(None, 0, dev(q), 0, 0, scores, 0, 0, out, dk, dv, nh, nkv, hd, hd, max_seq, S, kvg, window)
    else:
        ops.attention_prefill_batched_fp32(None, 0, dev(q), 0, scores, 0, out, dk, dv, nh, nkv, hd, hd, max_seq, S, kvg, window)
    torch.cuda.synchronize()
    want = exact_dense(q, k, v, kvg, prefix_range(S, S, window, 0, 0))
    got = host(out)
    for s in range(S):
        ok, rel = within(got[s], want[s], TOL)
        assert ok, f"row {s}: {rel:.2e} x RMS"


def test_dense_wide_cache_rows_and_bad_arguments():
    """cache_hd (row pitch) wider than the head dim; and the status codes of malformed calls."""
    rng = np.random.default_rng(3)
    nh, nkv, hd, cache_hd, T = 8, 4, 128, 192, 257
    k, v, dk, dv = make_dense_cache(rng, nkv, T, hd, cache_hd, T, False)
    k[:, :, hd:] = 1e4; v[:, :, hd:] = 1e4
    dk, dv = dev(k), dev(v)
    q = (bf16_normal(rng, (nh, hd)) * np.float32(0.25)).astype(np.float32)
    out = torch.full((nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    scratch = torch.empty(nh * T, dtype=torch.float32, device=DEV)
    ops.attention_gpu_fp32_dev(None, 0, dev(q), dk, dv, scratch, out, nh, nkv, hd, cache_hd, T, T, nh // nkv)
    torch.cuda.synchronize()
    want = exact_dense(q[None], k, v, nh // nkv, lambda s: (0, T - 1))[0]
    assert within(host(out), want, TOL)[0]
    with pytest.raises(ops.NomosError) as e:
        ops.attention_gpu_fp32_dev(None, 0, dev(q), dk, dv, scratch, out, nh, nkv, hd, cache_hd, T, T + 1, nh // nkv)   # seq_len > pitch
    assert e.value.status == -3
    with pytest.raises(ops.NomosError) as e:
        ops.attention_gpu_fp32_dev(None, 0, dev(q), dk, dv, scratch, out, nh, nkv, hd, cache_hd, T, T, 3)               # nh != nkv*kvg
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:
        ops.attention_gpu_fp32_dev(None, 0, dev(q), dk, dv, scratch, out, nh, nkv, 96, 96, T, T, nh // nkv)             # head dim 96
    assert e.value.status == -2
    ops.attention_gpu_fp32_dev(None, 0, dev(q), dk, dv, scratch, out, nh, nkv, hd, cache_hd, T, 0, nh // nkv)           # no keys: no-op
    torch.cuda.synchronize()
