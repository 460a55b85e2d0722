"""Pins the CPU oracle against every known-answer property the reference's own
tests and probes hold for this path (CPU only).

  * nibble identities            tools/parity_attn_int4.mojo:15-78
  * int8 codec tolerance         tools/kv_quant_test.mojo:26-64
  * append->reader layout trip   tools/kv_quant_test.mojo:66-116
  * P1 batched == single append  nomos_ffi.mojo:979-1179
  * P2 overwrite insensitivity   nomos_ffi.mojo:1182-1414
  * P3 q8 view == reader view    nomos_ffi.mojo:840-976
"""
import numpy as np
import pytest

from oracle import np_codecs as npc
from tests._cases import KVCache, ref_probe_rows, ref_q8_probe_row


def test_nibble_sign_extend_all_values():
    for n in range(16):
        expected = n - 16 if n >= 8 else n
        assert (n ^ 8) - 8 == expected
        got = npc.unpack_nibbles(np.array([n], dtype=np.uint8))[0]
        assert int(got) == expected


def test_nibble_pack_unpack_all_225_pairs():
    q = np.array([(a, b) for a in range(-7, 8) for b in range(-7, 8)], dtype=np.int8)
    packed = npc.pack_nibbles(q)
    assert packed.shape == (225, 1)
    assert np.array_equal(npc.unpack_nibbles(packed), q)
    # low nibble is the even element
    assert np.array_equal(packed[:, 0] & 0xF, q[:, 0].astype(np.int32) & 0xF)


def test_int8_codec_tolerance_uniform(oracle):
    """U[-3,3) bf16 [256,512]: RMSE/||X|| < 0.01 after quant->dequant."""
    rng = np.random.default_rng(7)
    x = (rng.integers(0, 2000, size=(256, 512)).astype(np.float32) / np.float32(333.0) - np.float32(3.0))
    xb = oracle.f32_to_bf16(x)
    q = np.zeros((256, 512), np.int8)
    s = np.zeros(256, np.float32)
    oracle.quant_kv_i8(xb, q, s, 256, 512)
    back = np.zeros((256, 512), np.uint16)
    oracle.dequant_kv_i8(q, s, back, 256, 512)
    a = oracle.bf16_to_f32(xb).astype(np.float64)
    d = oracle.bf16_to_f32(back).astype(np.float64) - a
    assert np.sqrt((d * d).sum() / (a * a).sum()) < 0.01


def test_append_reader_layout_round_trip(oracle):
    """n_s=4, nkv=2, l_hd=256, cache_hd=512, max_seq=16 as in the reference test."""
    n_s, nkv, l_hd, cache_hd, max_seq = 4, 2, 256, 512, 16
    rng = np.random.default_rng(11)
    k = (rng.integers(0, 2000, size=(n_s, nkv, l_hd)).astype(np.float32) / np.float32(333.0) - np.float32(3.0))
    v = (rng.integers(0, 2000, size=(n_s, nkv, l_hd)).astype(np.float32) / np.float32(333.0) - np.float32(3.0))
    c = KVCache("i8", nkv, max_seq, l_hd, cache_hd)
    c.append(k, v, 0)
    dk = np.zeros((nkv, max_seq, cache_hd), np.uint16)
    oracle.dequant_kv_i8_layer(c.k, c.ks.view(np.float32), dk, nkv, n_s, cache_hd, max_seq, max_seq, 0)
    deq = oracle.bf16_to_f32(dk)[:, :n_s, :l_hd].transpose(1, 0, 2).astype(np.float64)
    d = deq - k
    assert np.sqrt((d * d).sum() / (k.astype(np.float64) ** 2).sum()) < 0.01
    assert not c.k[:, :n_s, l_hd:].any(), "pad [l_hd, cache_hd) must be zero"


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
@pytest.mark.parametrize("base_pos,n_rows,cap", [(0, 9, 64), (60, 9, 64), (8191 - 4, 9, 1024)])
def test_p1_batched_append_equals_single_row(oracle, fmt, base_pos, n_rows, cap):
    nkv, hd, layer = 4, 128, 3
    k, v = ref_probe_rows(n_rows, nkv * hd, layer, base_pos)
    k = k.reshape(n_rows, nkv, hd); v = v.reshape(n_rows, nkv, hd)
    batched = KVCache(fmt, nkv, cap, hd)
    batched.append(k, v, base_pos)
    single = KVCache(fmt, nkv, cap, hd)
    for r in range(n_rows):
        single.append(k[r:r + 1], v[r:r + 1], base_pos + r)
    for name in ("k", "v", "ks", "vs"):
        assert np.array_equal(getattr(batched, name), getattr(single, name)), name


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
def test_p2_append_over_garbage(oracle, fmt):
    nkv, hd, cap, n_rows, base_pos = 4, 128, 32, 5, 30   # wraps the ring
    k, v = ref_probe_rows(n_rows, nkv * hd, 1, base_pos)
    k = k.reshape(n_rows, nkv, hd); v = v.reshape(n_rows, nkv, hd)
    clean = KVCache(fmt, nkv, cap, hd)
    clean.append(k, v, base_pos)
    dirty = KVCache(fmt, nkv, cap, hd)
    rng = np.random.default_rng(5)
    for name in ("k", "v", "ks", "vs"):
        a = getattr(dirty, name)
        a[...] = rng.integers(0, 255, size=a.shape).astype(a.dtype)
    dirty.append(k, v, base_pos)
    slots = [(base_pos + r) % cap for r in range(n_rows)]
    assert np.array_equal(clean.k[:, slots], dirty.k[:, slots])
    assert np.array_equal(clean.v[:, slots], dirty.v[:, slots])


@pytest.mark.parametrize("hd,nkv", [(256, 16), (512, 4), (128, 16)])
def test_p3_q8_view_equals_reader_view_block32(oracle, hd, nkv):
    """append-with-q8 publishes the same bytes the block-32 -> q8 reader rebuilds."""
    kvd = nkv * hd
    nb = hd // 32
    k, v = ref_q8_probe_row(kvd, layer=7)
    c = KVCache("i4b32", nkv, 1, hd)
    kq8 = np.zeros((nkv, 1, hd), np.int8); vq8 = np.zeros((nkv, 1, hd), np.int8)
    kqs = np.zeros((nkv, 1), np.float32); vqs = np.zeros((nkv, 1), np.float32)
    oracle.append_quant_kv_i4_with_q8(k, v, c.k, c.v, c.ks, c.vs, kq8, vq8, kqs, vqs,
                                      1, nkv, hd, kvd, 1, hd, 0, 1, nb)
    rk = np.zeros_like(kq8); rv = np.zeros_like(vq8)
    rks = np.zeros_like(kqs); rvs = np.zeros_like(vqs)
    oracle.dequant_kv_i4_to_q8_layer(c.k, c.ks, rk, rks, nkv, 1, hd, 1, 1, 0, nb)
    oracle.dequant_kv_i4_to_q8_layer(c.v, c.vs, rv, rvs, nkv, 1, hd, 1, 1, 0, nb)
    assert np.array_equal(kq8, rk) and np.array_equal(vq8, rv)
    assert np.array_equal(kqs, rks) and np.array_equal(vqs, rvs)
    # and the plain block-32 append writes the same packed bytes/scales as the q8 twin
    c2 = KVCache("i4b32", nkv, 1, hd)
    c2.append(k.reshape(1, nkv, hd), v.reshape(1, nkv, hd), 0)
    assert np.array_equal(c.k, c2.k) and np.array_equal(c.ks, c2.ks)


def test_p3_row_scale_q8_view_is_the_code(oracle):
    nkv, hd, cap, n_s, base = 2, 128, 16, 3, 5
    k, v = ref_probe_rows(n_s, nkv * hd, 2, base)
    c = KVCache("i4", nkv, cap, hd)
    pitch = 32
    kq8 = np.zeros((nkv, pitch, hd), np.int8); vq8 = np.zeros((nkv, pitch, hd), np.int8)
    kqs = np.zeros((nkv, pitch), np.float32); vqs = np.zeros((nkv, pitch), np.float32)
    oracle.append_quant_kv_i4_with_q8(k, v, c.k, c.v, c.ks, c.vs, kq8, vq8, kqs, vqs,
                                      n_s, nkv, hd, nkv * hd, cap, hd, base, pitch, 1)
    codes = npc.unpack_nibbles(c.k)
    for s in range(n_s):
        assert np.array_equal(kq8[:, base + s], codes[:, (base + s) % cap])
        assert np.array_equal(kqs[:, base + s], c.row_scales_f32("k")[:, (base + s) % cap])
