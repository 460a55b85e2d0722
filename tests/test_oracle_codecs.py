"""The two CPU restatements of the quantizers (C loops, NumPy vectors) must agree
bit-for-bit, including on the rounding edge cases (CPU only)."""
import numpy as np
import pytest

from oracle import np_codecs as npc
from tests._cases import KVCache, bf16_normal


def _edge_rows(hd: int) -> np.ndarray:
    rng = np.random.default_rng(3)
    rows = [np.zeros(hd, np.float32)]                                   # all-zero row -> scale 1.0
    r = np.zeros(hd, np.float32); r[0] = -0.0; r[5] = 127.0; rows.append(r)   # -0.0 and scale exactly 1
    r = np.full(hd, 0.49999997, np.float32); r[1] = 127.0; rows.append(r)     # 0.49999997f+0.5f == 1.0f
    r = np.full(hd, -0.49999997, np.float32); r[1] = -127.0; rows.append(r)
    r = rng.standard_normal(hd).astype(np.float32); r[3] = 4.0; r[9] = -4.0; rows.append(r)  # +-amax tie
    r = (np.arange(hd, dtype=np.float32) - hd / 2 + 0.5).astype(np.float32); rows.append(r)  # exact .5 codes
    r = np.full(hd, 1e-30, np.float32); rows.append(r)                  # tiny but non-zero
    r = rng.standard_normal(hd).astype(np.float32) * 8; rows.append(r)
    r = np.zeros(hd, np.float32); r[32:64] = rng.standard_normal(32).astype(np.float32); rows.append(r)  # zero blocks
    return np.stack(rows)


@pytest.mark.parametrize("hd", [128, 256])
def test_i8_rows_c_equals_numpy(oracle, hd):
    x = np.concatenate([_edge_rows(hd), bf16_normal(np.random.default_rng(1), (64, hd))])
    n = x.shape[0]
    c = KVCache("i8", 1, n, hd)
    c.append(x[:, None, :], -x[:, None, :], 0)
    codes, scale = npc.quant_rows_i8(x)
    assert np.array_equal(c.k[0], codes)
    assert np.array_equal(c.row_scales_f32("k")[0], scale)
    codes_v, scale_v = npc.quant_rows_i8(-x)
    assert np.array_equal(c.v[0], codes_v) and np.array_equal(c.row_scales_f32("v")[0], scale_v)
    assert np.abs(codes.astype(int)).max() <= 127


@pytest.mark.parametrize("hd", [128, 256])
def test_i4_rows_c_equals_numpy(oracle, hd):
    x = np.concatenate([_edge_rows(hd), bf16_normal(np.random.default_rng(2), (64, hd))])
    n = x.shape[0]
    c = KVCache("i4", 1, n, hd)
    c.append(x[:, None, :], x[:, None, :] * np.float32(0.73), 0)
    codes, scale = npc.quant_rows_i4(x)
    assert np.array_equal(c.k[0], npc.pack_nibbles(codes))
    assert np.array_equal(c.row_scales_f32("k")[0], scale)
    assert np.abs(codes.astype(int)).max() <= 7


@pytest.mark.parametrize("hd", [128, 256, 512])
def test_i4_block32_rows_c_equals_numpy(oracle, hd):
    rows = _edge_rows(hd)
    rows = rows[[0, 1, 4, 5, 7, 8]]       # block-32 needs amax/7 inside the fp16 normal range
    x = np.concatenate([rows, bf16_normal(np.random.default_rng(4), (64, hd)) * np.float32(3.0)])
    n = x.shape[0]
    nb = hd // 32
    c = KVCache("i4b32", 1, n, hd)
    c.append(x[:, None, :], x[:, None, :], 0)
    codes, s16, q8s = npc.quant_rows_i4_block32(x)
    assert np.array_equal(c.k[0], npc.pack_nibbles(codes))
    got16 = c.ks[: n * nb * 2].view(np.float16).reshape(n, nb)
    assert np.array_equal(got16.view(np.uint16), s16.view(np.uint16))
    gotq8 = c.ks[n * nb * 2:].view(np.float32)
    assert np.array_equal(gotq8, q8s)


def test_block32_division_differs_from_reciprocal():
    """The block-32 codec divides by the fp16-rounded scale; a reciprocal multiply
    gives different codes on some inputs, so the distinction is observable."""
    rng = np.random.default_rng(9)
    F = np.float32
    sf = rng.uniform(0.01, 4, size=4096).astype(np.float16).astype(F)
    x = np.zeros((4096, 32), F)
    x[:, 0] = (sf * F(7)).astype(F)                       # pins the block scale to sf
    k = rng.integers(0, 6, size=(4096, 31)).astype(F) + F(0.5)
    x[:, 1:] = (k * sf[:, None]).astype(F)                # sits on a rounding boundary ...
    step = np.where(rng.random((4096, 31)) < 0.5, -np.inf, np.inf).astype(F)
    x[:, 1:] = np.nextafter(x[:, 1:], step)               # ... one ulp to either side
    codes, s16, _ = npc.quant_rows_i4_block32(x)
    assert np.array_equal(s16[:, 0].astype(F), sf)
    alt = npc.round_away_clamp((x * (F(1.0) / sf)[:, None]).astype(F), 7)
    assert (alt != codes).any()


def test_ring_wrap_slots(oracle):
    """Positions 0..8191 through a 1024-slot ring: slot = pos % 1024, last writer wins."""
    nkv, hd, cap = 2, 128, 1024
    rng = np.random.default_rng(13)
    c = KVCache("i4b32", nkv, cap, hd)
    last = {}
    for base in range(0, 8192, 512):
        k = bf16_normal(rng, (512, nkv, hd)); v = bf16_normal(rng, (512, nkv, hd))
        c.append(k, v, base)
        if base >= 8192 - 1024:
            last[base] = (k, v)
    # window [7168, 8192) occupies slots 0..1023 in order
    ref = KVCache("i4b32", nkv, cap, hd)
    for base, (k, v) in last.items():
        ref.append(k, v, base - 7168)
    assert np.array_equal(c.k, ref.k) and np.array_equal(c.ks, ref.ks)
    assert (8191 % cap) == 1023 and (7168 % cap) == 0


def test_readers_follow_ring(oracle):
    nkv, hd, cap = 2, 128, 8
    rng = np.random.default_rng(17)
    k = bf16_normal(rng, (20, nkv, hd)); v = bf16_normal(rng, (20, nkv, hd))
    for fmt in ("i8", "i4", "i4b32"):
        c = KVCache(fmt, nkv, cap, hd)
        c.append(k, v, 0)
        win_start, klen, pitch = 20 - 8, 8, 12
        out = np.zeros((nkv, pitch, hd), np.uint16)
        lin = KVCache(fmt, nkv, 32, hd)           # linear cache holding the same positions
        lin.append(k, v, 0)
        out_lin = np.zeros((nkv, pitch, hd), np.uint16)
        if fmt == "i8":
            oracle.dequant_kv_i8_layer(c.k, c.ks.view(np.float32), out, nkv, klen, hd, pitch, cap, win_start)
            oracle.dequant_kv_i8_layer(lin.k[:, win_start:].copy(), lin.ks.view(np.float32).reshape(nkv, 32)[:, win_start:].copy(),
                                       out_lin, nkv, klen, hd, pitch, 32 - win_start, 0)
        else:
            oracle.dequant_kv_i4_layer(c.k, c.ks, out, nkv, klen, hd, pitch, cap, win_start, c.scale_blocks)
            oracle.dequant_kv_i4_layer(lin.k, lin.ks, out_lin, nkv, klen, hd, pitch, 32, win_start, c.scale_blocks)
        assert np.array_equal(out, out_lin), fmt
