"""GPU parity of the fused attention over the int4 cache layouts and the wider head dims,
against the oracle's exact-dequant attention (same 2e-3 x RMS bar), through the C ABI."""
import numpy as np
import pytest

from nomos_nvfp4_b200 import ops
from tests._cases import bf16_normal
from tests._gpu import within
from tests.test_gpu_attn import SENTINEL, TOL, build_cache, exact, fused

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["i4", "i4b32"])
@pytest.mark.parametrize("T", [1, 31, 32, 33, 1023, 1025])
def test_decode_int4_lengths(oracle, fmt, T):
    rng = np.random.default_rng(100 + T)
    nh, nkv, hd = 8, 4, 128
    c = build_cache(fmt, rng, T, nkv, hd, cap=T + 5)
    q = bf16_normal(rng, (1, nh, hd)) * np.float32(0.3)
    want = exact(oracle, c, q, klen=T)
    got, _ = fused(c, q, klen=T)
    ok, rel = within(got, want, TOL)
    assert ok, f"{fmt} T={T}: {rel:.2e} x RMS"
    assert not np.any(got == SENTINEL)


def test_config3_sliding_window_ring_int4_block32(oracle):
    """Configuration 3: 32/16 heads x 128, window 1024 held in a ring, current position 8191 (ring
    wrapped 7x), int4 block-32 KV, quantize-on-write of the new token fused into the call."""
    rng = np.random.default_rng(1003)
    nh, nkv, hd, cap, pos = 32, 16, 128, 1024, 8191
    c = build_cache("i4b32", rng, pos, nkv, hd, cap=cap)          # positions 0..8190 through the ring
    new_k, new_v = bf16_normal(rng, (1, nkv, hd)), bf16_normal(rng, (1, nkv, hd))
    q = bf16_normal(rng, (1, nh, hd))
    seq_len = pos + 1
    win_start = seq_len - cap                                     # 7168 -> ring slot 0
    scale = 1.0 / np.sqrt(128.0)
    got, caches = fused(c, q, klen=cap, win_start=win_start, scale=scale, q_type=ops.BF16,
                        new_k=new_k, new_v=new_v, new_base_pos=pos)
    c.append(new_k, new_v, pos)                                   # lands in slot 8191 % 1024 = 1023
    want = exact(oracle, c, q, klen=cap, win_start=win_start, scale=scale)
    ok, rel = within(got, want, TOL)
    assert ok, f"{rel:.2e} x RMS"
    assert np.array_equal(caches[0], c.k) and np.array_equal(caches[1], c.v), "fused append bytes differ"
    assert np.array_equal(caches[2], c.ks) and np.array_equal(caches[3], c.vs), "fused append scales differ"


@pytest.mark.parametrize("fmt", ["i4", "i4b32"])
def test_int4_ring_mid_wrap_and_verify_rows(oracle, fmt):
    rng = np.random.default_rng(7)
    nh, nkv, hd, cap, T = 8, 4, 128, 512, 1300
    c = build_cache(fmt, rng, T, nkv, hd, cap=cap)
    for S, klen in ((1, 512), (1, 200), (5, 300), (9, 512)):
        q = bf16_normal(rng, (S, nh, hd)) * np.float32(0.5)
        win_start = T - klen
        want = exact(oracle, c, q, S=S, klen=klen, win_start=win_start, scale=0.2)
        got, _ = fused(c, q, S=S, klen=klen, win_start=win_start, scale=0.2)
        for r in range(S):
            ok, rel = within(got[r], want[r], TOL)
            assert ok, f"{fmt} S={S} klen={klen} row {r}: {rel:.2e} x RMS"


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
@pytest.mark.parametrize("hd,nkv,kvg", [(256, 4, 2), (512, 2, 8), (256, 2, 8)])
def test_wider_heads(oracle, fmt, hd, nkv, kvg):
    """The reference model's real geometry: hd 256 / kvg 2 (sliding) and hd 512 / kvg 8 (full)."""
    rng = np.random.default_rng(hd + kvg)
    nh, T = nkv * kvg, 700
    c = build_cache(fmt, rng, T, nkv, hd)
    q = bf16_normal(rng, (1, nh, hd))
    scale = 1.0 / np.sqrt(hd)
    want = exact(oracle, c, q, klen=T, scale=scale)
    got, _ = fused(c, q, klen=T, scale=scale)
    ok, rel = within(got, want, TOL)
    assert ok, f"{fmt} hd={hd}: {rel:.2e} x RMS"


@pytest.mark.parametrize("fmt", ["i8", "i4b32"])
def test_verify_rows_wider_heads(oracle, fmt):
    rng = np.random.default_rng(3)
    nh, nkv, hd, S, T = 8, 4, 256, 9, 400
    c = build_cache(fmt, rng, T, nkv, hd)
    q = bf16_normal(rng, (S, nh, hd))
    want = exact(oracle, c, q, S=S, klen=T, scale=1 / 16.0)
    got, _ = fused(c, q, S=S, klen=T, scale=1 / 16.0)
    for r in range(S):
        ok, rel = within(got[r], want[r], TOL)
        assert ok, f"row {r}: {rel:.2e} x RMS"


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
@pytest.mark.parametrize("hd,nkv,kvg", [(512, 2, 8), (256, 4, 2)])
@pytest.mark.parametrize("T,cap,splits", [(33, 64, 0), (4097, 4100, 0), (3000, 1024, 0), (6000, 6000, 5), (2500, 2500, 1)])
def test_wider_heads_lengths_rings_and_splits(oracle, fmt, hd, nkv, kvg, T, cap, splits):
    """Head dims 256 / 512 (warps of a quad own 128-dim slices of K, V and the output and add their partial
    logits up): ragged lengths, a wrapped ring read from an odd slot, many tiles per quad, forced split counts."""
    rng = np.random.default_rng(hd + T + splits)
    nh = nkv * kvg
    c = build_cache(fmt, rng, T, nkv, hd, cap=cap)
    q = bf16_normal(rng, (1, nh, hd))
    scale = 1.0 / np.sqrt(hd)
    klen = min(T, cap) - (3 if cap < T else 0)
    win_start = T - klen
    want = exact(oracle, c, q, klen=klen, win_start=win_start, scale=scale)
    got, _ = fused(c, q, klen=klen, win_start=win_start, scale=scale, force_splits=splits)
    ok, rel = within(got, want, TOL)
    assert ok, f"{fmt} hd={hd} T={T}: {rel:.2e} x RMS"
    assert not np.any(got == SENTINEL)


@pytest.mark.parametrize("fmt,hd", [("i4b32", 512), ("i8", 256)])
def test_wider_heads_partial_export_merges_to_full(oracle, fmt, hd):
    """Two sequence shards of a wide-head cache export (o, m, l); their merge equals full attention."""
    import torch
    from tests._gpu import DEV, dev, host
    rng = np.random.default_rng(hd)
    nkv, kvg, T = 2, 4, 2048
    nh = nkv * kvg
    c = build_cache(fmt, rng, T, nkv, hd)
    q = bf16_normal(rng, (1, nh, hd))
    scale = 1.0 / np.sqrt(hd)
    want = exact(oracle, c, q, klen=T, scale=scale)
    parts = [fused(c, q, klen=T // 2, win_start=g * (T // 2), scale=scale, partial=True)[0] for g in range(2)]
    out = torch.full((nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    ops.attn_merge_partials(None, dev(np.stack(parts)), 2, nh, hd, out)
    torch.cuda.synchronize()
    ok, rel = within(host(out)[None], want, TOL)
    assert ok, f"{rel:.2e} x RMS"
