"""GPU parity of the KV-cache codecs: bytes and scales must equal the CPU oracle
bit-for-bit.  Every call goes through the C ABI (nomos_nvfp4_b200.ops)."""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import KVCache, bf16_normal, ref_probe_rows, ref_q8_probe_row
from tests._gpu import DEV, dev, host
from tests.test_oracle_codecs import _edge_rows

pytestmark = pytest.mark.gpu


class DevCache:
    """Device twin of tests._cases.KVCache, poisoned so unwritten bytes show up."""

    def __init__(self, ref: KVCache, poison: int = 0):
        self.ref = ref
        self.k = torch.full(ref.k.shape, poison, dtype=torch.uint8, device=DEV)
        self.v = torch.full_like(self.k, poison)
        if ref.fmt == "i8":
            self.k, self.v = self.k.view(torch.int8), self.v.view(torch.int8)
        self.ks = torch.full((ref.ks.size,), poison, dtype=torch.uint8, device=DEV)
        self.vs = torch.full_like(self.ks, poison)

    def append(self, k_rows, v_rows, base_pos):
        r = self.ref
        n_s = k_rows.shape[0]
        dk, dv = dev(np.ascontiguousarray(k_rows, np.float32)), dev(np.ascontiguousarray(v_rows, np.float32))
        if r.fmt == "i8":
            ops.gpu_append_quant_kv_i8(None, dk, dv, self.k, self.v, self.ks, self.vs, n_s, r.nkv, r.l_hd,
                                       r.nkv * r.l_hd, r.cache_cap, r.cache_hd, base_pos)
        else:
            ops.gpu_append_quant_kv_i4(None, dk, dv, self.k, self.v, self.ks, self.vs, n_s, r.nkv, r.l_hd,
                                       r.nkv * r.l_hd, r.cache_cap, r.cache_hd, base_pos, r.scale_blocks)
        torch.cuda.synchronize()


def _same(dc: DevCache, ref: KVCache, rows=None):
    for name in ("k", "v"):
        a, b = host(getattr(dc, name)), getattr(ref, name)
        if rows is not None:
            a, b = a[:, rows], b[:, rows]
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), f"{name} bytes differ"
    if rows is None:
        assert np.array_equal(host(dc.ks), ref.ks) and np.array_equal(host(dc.vs), ref.vs), "scales differ"


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
@pytest.mark.parametrize("hd", [128, 256, 512])
def test_append_bit_exact_random_and_edges(oracle, fmt, hd):
    rng = np.random.default_rng(100 + hd)
    nkv, n = 4, 48
    x = bf16_normal(rng, (n, nkv, hd)) * np.float32(2.5)
    edges = _edge_rows(hd)
    if fmt == "i4b32":
        edges = edges[[0, 1, 4, 5, 7, 8]]
    x[: len(edges), 0] = edges
    x[: len(edges), 1] = -edges
    v = bf16_normal(rng, (n, nkv, hd))
    ref = KVCache(fmt, nkv, n, hd)
    ref.append(x, v, 0)
    dc = DevCache(ref)
    dc.append(x, v, 0)
    _same(dc, ref)


def test_block32_true_division_on_boundaries(oracle):
    """Inputs one ulp either side of a rounding boundary: a reciprocal multiply would differ."""
    rng = np.random.default_rng(9)
    F = np.float32
    nkv, hd, n = 2, 128, 256
    sf = rng.uniform(0.01, 4, size=(n, nkv, 4)).astype(np.float16).astype(F)
    x = np.zeros((n, nkv, 4, 32), F)
    x[..., 0] = sf * F(7)
    k = rng.integers(0, 6, size=(n, nkv, 4, 31)).astype(F) + F(0.5)
    x[..., 1:] = (k * sf[..., None]).astype(F)
    step = np.where(rng.random(x[..., 1:].shape) < 0.5, -np.inf, np.inf).astype(F)
    x[..., 1:] = np.nextafter(x[..., 1:], step)
    x = x.reshape(n, nkv, hd)
    ref = KVCache("i4b32", nkv, n, hd)
    ref.append(x, -x, 0)
    dc = DevCache(ref)
    dc.append(x, -x, 0)
    _same(dc, ref)


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
def test_cache_hd_wider_than_head(oracle, fmt):
    """cache_hd > l_hd: int8 / row-scale int4 zero the pad, block-32 leaves it untouched."""
    nkv, hd, chd, n = 2, 128, 256, 8
    rng = np.random.default_rng(5)
    k, v = bf16_normal(rng, (n, nkv, hd)), bf16_normal(rng, (n, nkv, hd))
    ref = KVCache(fmt, nkv, n, hd, chd)
    ref.k[...] = 0x5A
    ref.v[...] = 0x5A
    ref.append(k, v, 0)
    dc = DevCache(ref, poison=0x5A)
    dc.append(k, v, 0)
    _same(dc, ref)


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
def test_p1_p2_batched_vs_single_over_garbage_ring(oracle, fmt):
    """Reference probe inputs (row gains (s+1)^2): S-row append == S single-row appends,
    also over a poisoned ring that wraps (nomos_ffi.mojo:979-1414)."""
    nkv, hd, cap, n_rows, base_pos = 4, 128, 32, 9, 28
    k, v = ref_probe_rows(n_rows, nkv * hd, 3, base_pos)
    k, v = k.reshape(n_rows, nkv, hd), v.reshape(n_rows, nkv, hd)
    ref = KVCache(fmt, nkv, cap, hd)
    ref.append(k, v, base_pos)
    batched = DevCache(ref, poison=0xA5)
    batched.append(k, v, base_pos)
    single = DevCache(ref, poison=0x3C)
    for r in range(n_rows):
        single.append(k[r:r + 1], v[r:r + 1], base_pos + r)
    slots = [(base_pos + r) % cap for r in range(n_rows)]
    _same(batched, ref, rows=slots)
    _same(single, ref, rows=slots)
    untouched = [s for s in range(cap) if s not in slots]
    assert (host(batched.k)[:, untouched].view(np.uint8) == 0xA5).all(), "append wrote outside its slots"


def test_ring_7x_wrap_block32(oracle):
    """Positions 0..8191 through a 1024-slot ring in chunks (configuration 3's state)."""
    nkv, hd, cap = 2, 128, 1024
    rng = np.random.default_rng(1003)
    ref = KVCache("i4b32", nkv, cap, hd)
    dc = DevCache(ref)
    for base in range(0, 8192, 1024):
        k, v = bf16_normal(rng, (1024, nkv, hd)), bf16_normal(rng, (1024, nkv, hd))
        ref.append(k, v, base)
        dc.append(k, v, base)
    _same(dc, ref)


@pytest.mark.parametrize("scale_blocks_fmt", ["i4", "i4b32"])
def test_append_with_q8_view_and_p3(oracle, scale_blocks_fmt):
    nkv, hd, cap, n_s, base, pitch = 4, 128, 16, 5, 9, 32
    k, v = ref_probe_rows(n_s, nkv * hd, 2, base)
    ref = KVCache(scale_blocks_fmt, nkv, cap, hd)
    sb = ref.scale_blocks
    kq8 = np.zeros((nkv, pitch, hd), np.int8); vq8 = np.zeros_like(kq8)
    kqs = np.zeros((nkv, pitch), np.float32); vqs = np.zeros_like(kqs)
    oracle.append_quant_kv_i4_with_q8(k, v, ref.k, ref.v, ref.ks, ref.vs, kq8, vq8, kqs, vqs,
                                      n_s, nkv, hd, nkv * hd, cap, hd, base, pitch, sb)
    dc = DevCache(ref)
    d_kq8 = torch.zeros((nkv, pitch, hd), dtype=torch.int8, device=DEV); d_vq8 = torch.zeros_like(d_kq8)
    d_kqs = torch.zeros((nkv, pitch), dtype=torch.float32, device=DEV); d_vqs = torch.zeros_like(d_kqs)
    ops.gpu_append_quant_kv_i4_with_q8(None, dev(k), dev(v), dc.k, dc.v, dc.ks, dc.vs, d_kq8, d_vq8, d_kqs, d_vqs,
                                       n_s, nkv, hd, nkv * hd, cap, hd, base, pitch, sb)
    torch.cuda.synchronize()
    slots = [(base + s) % cap for s in range(n_s)]
    _same(dc, ref, rows=slots)
    assert np.array_equal(host(d_kq8), kq8) and np.array_equal(host(d_vq8), vq8)
    assert np.array_equal(host(d_kqs), kqs) and np.array_equal(host(d_vqs), vqs)
    # P3: the reader rebuilds the same int8 view from the packed cache
    klen, win_start = n_s, base
    r_k = torch.zeros((nkv, pitch, hd), dtype=torch.int8, device=DEV)
    r_s = torch.zeros((nkv, pitch), dtype=torch.float32, device=DEV)
    ops.gpu_dequant_kv_i4_to_q8_layer(None, dc.k, dc.ks, r_k, r_s, nkv, klen, hd, pitch, cap, win_start, sb)
    torch.cuda.synchronize()
    assert np.array_equal(host(r_k)[:, :klen], kq8[:, base:base + n_s])
    assert np.array_equal(host(r_s)[:, :klen], kqs[:, base:base + n_s])


def test_p3_block32_probe_row(oracle):
    """The reference's own q8-view probe input (nomos_ffi.mojo:875-879), hd 256 / nkv 16."""
    nkv, hd = 16, 256
    nb = hd // 32
    k, v = ref_q8_probe_row(nkv * hd, layer=7)
    ref = KVCache("i4b32", nkv, 1, hd)
    dc = DevCache(ref)
    d_kq8 = torch.zeros((nkv, 1, hd), dtype=torch.int8, device=DEV); d_vq8 = torch.zeros_like(d_kq8)
    d_kqs = torch.zeros((nkv, 1), dtype=torch.float32, device=DEV); d_vqs = torch.zeros_like(d_kqs)
    ops.gpu_append_quant_kv_i4_with_q8(None, dev(k), dev(v), dc.k, dc.v, dc.ks, dc.vs, d_kq8, d_vq8, d_kqs, d_vqs,
                                       1, nkv, hd, nkv * hd, 1, hd, 0, 1, nb)
    r_k = torch.zeros_like(d_kq8); r_s = torch.zeros_like(d_kqs)
    ops.gpu_dequant_kv_i4_to_q8_layer(None, dc.k, dc.ks, r_k, r_s, nkv, 1, hd, 1, 1, 0, nb)
    torch.cuda.synchronize()
    assert torch.equal(r_k, d_kq8) and torch.equal(r_s, d_kqs)


@pytest.mark.parametrize("fmt", ["i8", "i4", "i4b32"])
def test_window_readers_to_bf16(oracle, fmt):
    nkv, hd, cap = 2, 128, 8
    rng = np.random.default_rng(17)
    k, v = bf16_normal(rng, (20, nkv, hd)), bf16_normal(rng, (20, nkv, hd))
    ref = KVCache(fmt, nkv, cap, hd)
    ref.append(k, v, 0)
    win_start, klen, pitch = 12, 8, 12
    want = np.zeros((nkv, pitch, hd), np.uint16)
    got = torch.zeros((nkv, pitch, hd), dtype=torch.bfloat16, device=DEV)
    dk, dks = dev(ref.k), dev(ref.ks)
    if fmt == "i8":
        oracle.dequant_kv_i8_layer(ref.k, ref.ks.view(np.float32), want, nkv, klen, hd, pitch, cap, win_start)
        ops.gpu_dequant_kv_i8_layer(None, dk, dks, got, nkv, klen, hd, pitch, cap, win_start)
    else:
        oracle.dequant_kv_i4_layer(ref.k, ref.ks, want, nkv, klen, hd, pitch, cap, win_start, ref.scale_blocks)
        ops.gpu_dequant_kv_i4_layer(None, dk, dks, got, nkv, klen, hd, pitch, cap, win_start, ref.scale_blocks)
    torch.cuda.synchronize()
    assert np.array_equal(host(got, np.uint16), want)


def test_standalone_i8_codec(oracle):
    rng = np.random.default_rng(21)
    x = (rng.integers(0, 2000, size=(256, 512)).astype(np.float32) / np.float32(333.0) - np.float32(3.0))
    xb = oracle.f32_to_bf16(x)
    q = np.zeros((256, 512), np.int8); s = np.zeros(256, np.float32)
    oracle.quant_kv_i8(xb, q, s, 256, 512)
    back = np.zeros((256, 512), np.uint16)
    oracle.dequant_kv_i8(q, s, back, 256, 512)
    d_in = dev(xb).view(torch.bfloat16)
    d_q = torch.zeros((256, 512), dtype=torch.int8, device=DEV)
    d_s = torch.zeros(256, dtype=torch.float32, device=DEV)
    d_back = torch.zeros((256, 512), dtype=torch.bfloat16, device=DEV)
    ops.gpu_quant_kv_i8(None, d_in, d_q, d_s, 256, 512)
    ops.gpu_dequant_kv_i8(None, d_q, d_s, d_back, 256, 512)
    torch.cuda.synchronize()
    assert np.array_equal(host(d_q), q) and np.array_equal(host(d_s), s)
    assert np.array_equal(host(d_back, np.uint16), back)


def test_dense_appends(oracle):
    nkv, hd, chd, max_seq = 4, 128, 256, 16
    rng = np.random.default_rng(23)
    k = rng.standard_normal((3, nkv, hd)).astype(np.float32); v = rng.standard_normal((3, nkv, hd)).astype(np.float32)
    want_k = np.zeros((nkv, max_seq, chd), np.uint16); want_v = np.zeros_like(want_k)
    oracle.append_kv_batched_bf16(k, v, want_k, want_v, 3, nkv, hd, nkv * hd, max_seq, chd, 5)
    d_k = torch.zeros((nkv, max_seq, chd), dtype=torch.bfloat16, device=DEV); d_v = torch.zeros_like(d_k)
    ops.gpu_append_kv_batched_bf16(None, dev(k), dev(v), d_k, d_v, 3, nkv, hd, nkv * hd, max_seq, chd, 5)
    f_k = torch.zeros((nkv, max_seq, chd), dtype=torch.float32, device=DEV); f_v = torch.zeros_like(f_k)
    ops.append_kv_gpu_dev_async(None, f_k, f_v, dev(k[0]), dev(v[0]), nkv, hd, chd, max_seq, 7)
    b_k = torch.zeros_like(d_k); b_v = torch.zeros_like(d_k)
    ops.append_kv_gpu_bf16_dev(None, b_k, b_v, dev(k[1]), dev(v[1]), None, None, nkv, hd, chd, max_seq, 6)
    torch.cuda.synchronize()
    assert np.array_equal(host(d_k, np.uint16), want_k) and np.array_equal(host(d_v, np.uint16), want_v)
    wf_k = np.zeros((nkv, max_seq, chd), np.float32); wf_v = np.zeros_like(wf_k)
    oracle.append_kv_fp32(wf_k, wf_v, k[0].copy(), v[0].copy(), nkv, hd, chd, max_seq, 7)
    assert np.array_equal(host(f_k), wf_k) and np.array_equal(host(f_v), wf_v)
    assert np.array_equal(host(b_k, np.uint16)[:, 6, :hd], want_k[:, 6, :hd])
