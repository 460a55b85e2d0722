"""GPU parity of the int8 prefix-batched and square-batched attention operators, through the C ABI.

attention_prefill_prefix_batched_int8 (lib/attention_gpu_int8.mojo:844-887) is called by the reference's engine
with K / V / scale pointers pre-offset by `key_base` rows once the prefix is longer than a sliding layer's window
(lib/engine_prefill.mojo:926-941); attention_prefill_batched_int8 (:804-841) is the square causal prefill.  Both
are checked with exactly those argument patterns against the oracle's fp64 attention over the same cache bytes
(2e-3 x RMS per query row), and loosely against the literal restatement of the reference's own lossy route
(Q and P re-quantised to 8 bits per block of 32), which sits several percent of RMS from exact arithmetic.
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import bf16_normal
from tests._gpu import DEV, dev, host, within
from tests.test_gpu_attn import build_cache

pytestmark = pytest.mark.gpu
TOL = 2e-3
SENTINEL = -1.0e30


def engine_prefix_call(c, q, S, start_pos, window, max_seq):
    """The reference engine's call (lib/engine_prefill.mojo:926-941): key_base, key_len and pre-offset pointers."""
    nh, hd, nkv = q.shape[-2], c.l_hd, c.nkv
    key_base = start_pos - window + 1 if (window > 0 and start_pos - window + 1 > 0) else 0
    key_len = start_pos + S - key_base
    dk, dv = dev(c.k), dev(c.v)
    dks, dvs = dev(c.ks).view(torch.float32), dev(c.vs).view(torch.float32)
    scores = torch.empty(S * nh * key_len, dtype=torch.float32, device=DEV)
    out = torch.full((S, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    ops.attention_prefill_prefix_batched_int8(
        None, dev(q), 0, scores, 0, out, dk.data_ptr() + key_base * hd, dv.data_ptr() + key_base * hd,
        dks.data_ptr() + key_base * 4, dvs.data_ptr() + key_base * 4, nh, nkv, hd, hd, max_seq, S, key_len, nh // nkv,
        window, start_pos, key_base)
    torch.cuda.synchronize()
    return host(out), key_base, key_len


@pytest.mark.parametrize("S,start_pos,window", [(9, 300, 1024), (9, 1016, 1024), (9, 1500, 1024), (17, 2000, 512),
                                                (9, 1200, 0), (1, 1500, 1024), (64, 0, 1024), (40, 1000, 1024)])
def test_prefix_batched_i8_with_the_engines_arguments(oracle, S, start_pos, window):
    """start_pos below the window (key_base = 0), straddling it, and above it (key_base > 0, pointers pre-offset)."""
    rng = np.random.default_rng(S + start_pos + window)
    nh, nkv, hd, max_seq = 8, 4, 128, 2100
    T = start_pos + S
    c = build_cache("i8", rng, T, nkv, hd, cap=max_seq)
    q = bf16_normal(rng, (S, nh, hd)) * np.float32(0.5)
    got, key_base, key_len = engine_prefix_call(c, q, S, start_pos, window, max_seq)
    assert not np.any(got == SENTINEL)
    want = oracle.attn_exact(q, c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, max_seq, S=S, window=window,
                             query_base_pos=start_pos, win_lo=0)
    for r in range(S):
        ok, rel = within(got[r], want[r], TOL)
        assert ok, f"row {r} (key_base {key_base}): {rel:.2e} x RMS"
    # the literal restatement of the reference's route, on the same pre-offset arrays
    sc = np.zeros((nkv * S * (nh // nkv), key_len), np.float32); lit = np.zeros((S, nh, hd), np.float32)
    oracle.attn_prefix_batched_int8(q, sc, lit, c.k.reshape(-1)[key_base * hd:], c.v.reshape(-1)[key_base * hd:],
                                    c.ks.view(np.float32)[key_base:], c.vs.view(np.float32)[key_base:],
                                    nh, nkv, hd, hd, max_seq, S, key_len, nh // nkv, window, start_pos, key_base)
    assert within(got, lit, 0.2)[0]


@pytest.mark.parametrize("S,window", [(1, 0), (17, 0), (128, 0), (300, 0), (300, 64), (1000, 1024)])
def test_square_batched_i8(oracle, S, window):
    """attention_prefill_batched_int8: S query rows over the S keys at positions 0..S-1, causal (+ window)."""
    rng = np.random.default_rng(S * 3 + window)
    nh, nkv, hd, max_seq = 8, 4, 128, S + 7
    c = build_cache("i8", rng, S, nkv, hd, cap=max_seq)
    q = bf16_normal(rng, (S, nh, hd)) * np.float32(0.5)
    scores = torch.empty(max(nh * S * S, 16), dtype=torch.float32, device=DEV)
    out = torch.full((S, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    ops.attention_prefill_batched_int8(None, dev(q), 0, scores, 0, out, dev(c.k), dev(c.v), dev(c.ks).view(torch.float32),
                                       dev(c.vs).view(torch.float32), nh, nkv, hd, hd, max_seq, S, nh // nkv, window)
    torch.cuda.synchronize()
    got = host(out)
    assert not np.any(got == SENTINEL)
    want = oracle.attn_exact(q, c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, max_seq, S=S, window=window,
                             query_base_pos=0, win_lo=0)
    for r in range(S):
        ok, rel = within(got[r], want[r], TOL)
        assert ok, f"row {r}: {rel:.2e} x RMS"


def test_prefix_batched_i8_longer_key_array_is_cut_to_the_causal_range(oracle):
    """key_len beyond the last query row: the extra keys are never attended (they hold garbage here)."""
    rng = np.random.default_rng(5)
    nh, nkv, hd, max_seq, S, start = 8, 4, 128, 900, 9, 500
    c = build_cache("i8", rng, start + S, nkv, hd, cap=max_seq)
    c.k[:, start + S:, :] = 127
    c.ks.view(np.float32).reshape(nkv, max_seq)[:, start + S:] = 1e3      # attending any of these rows would swamp the softmax
    q = bf16_normal(rng, (S, nh, hd)) * np.float32(0.5)
    scores = torch.empty(S * nh * 700, dtype=torch.float32, device=DEV)
    out = torch.full((S, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    ops.attention_prefill_prefix_batched_int8(None, dev(q), 0, scores, 0, out, dev(c.k), dev(c.v), dev(c.ks).view(torch.float32),
                                              dev(c.vs).view(torch.float32), nh, nkv, hd, hd, max_seq, S, 700, nh // nkv, 0, start, 0)
    torch.cuda.synchronize()
    want = oracle.attn_exact(q, c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, max_seq, S=S, window=0, query_base_pos=start, win_lo=0)
    for r in range(S):
        assert within(host(out)[r], want[r], TOL)[0]
