"""Paged int8 caches (pages of 128 keys, one block table row per sequence): decode attention of a
batch of sequences with different lengths against exact attention over each sequence's own
linear cache, and the paged append against the oracle's row codec, through the C ABI."""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import KVCache, bf16_normal
from tests._gpu import DEV, dev, host, within

pytestmark = pytest.mark.gpu
PAGE = 128


def build_pools(rng, lens, nkv, hd, n_pages, max_pages):
    """Per-sequence linear caches (oracle codec) scattered into shuffled pages."""
    table = np.full((len(lens), max_pages), -1, np.int32)
    free = list(rng.permutation(n_pages))
    k_pool = np.zeros((n_pages, nkv, PAGE, hd), np.int8); v_pool = np.zeros_like(k_pool)
    ks_pool = np.ones((n_pages, nkv, PAGE), np.float32); vs_pool = np.ones_like(ks_pool)
    lin = []
    for b, T in enumerate(lens):
        c = KVCache("i8", nkv, T, hd)
        c.append(bf16_normal(rng, (T, nkv, hd)), bf16_normal(rng, (T, nkv, hd)), 0)
        lin.append(c)
        ks, vs = c.row_scales_f32("k"), c.row_scales_f32("v")
        for j in range((T + PAGE - 1) // PAGE):
            pg = int(free.pop())
            table[b, j] = pg
            n = min(PAGE, T - j * PAGE)
            k_pool[pg, :, :n] = c.k[:, j * PAGE:j * PAGE + n]; v_pool[pg, :, :n] = c.v[:, j * PAGE:j * PAGE + n]
            ks_pool[pg, :, :n] = ks[:, j * PAGE:j * PAGE + n]; vs_pool[pg, :, :n] = vs[:, j * PAGE:j * PAGE + n]
    table[table < 0] = 0                   # unused entries: any valid page, never read
    return table, k_pool, v_pool, ks_pool, vs_pool, lin


@pytest.mark.parametrize("kvg,lens", [(2, [1, 127, 128, 129, 300, 2000]), (8, [5, 1000]), (2, [40000, 17, 12345])])
def test_paged_decode_matches_linear_attention(oracle, kvg, lens):
    rng = np.random.default_rng(sum(lens) + kvg)
    nkv, hd = 4, 128
    nh = nkv * kvg
    max_len = max(lens)
    max_pages = (max_len + PAGE - 1) // PAGE + 2
    n_pages = sum((T + PAGE - 1) // PAGE for T in lens) + 5
    table, k_pool, v_pool, ks_pool, vs_pool, lin = build_pools(rng, lens, nkv, hd, n_pages, max_pages)
    q = bf16_normal(rng, (len(lens), nh, hd))
    out = torch.full((len(lens), nh, hd), -1e30, dtype=torch.float32, device=DEV)
    wsb = ops.attn_paged_workspace_bytes(len(lens), nh, nkv, kvg, hd, max_len)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=DEV)
    keep = [dev(np.ascontiguousarray(q, np.float32)), dev(k_pool), dev(v_pool), dev(ks_pool), dev(vs_pool), dev(table),
            dev(np.asarray(lens, np.int32))]
    for _ in range(2):                      # twice in a row: the workspace and its counters are reused
        ops.attn_paged_decode_i8(None, *keep, out, ws, wsb, batch=len(lens), nh=nh, nkv=nkv, kvg=kvg, l_hd=hd, n_pages=n_pages,
                                 max_pages=max_pages, max_len=max_len, softmax_scale=0.1)
    torch.cuda.synchronize()
    got = host(out)
    assert not np.any(got == -1e30), "output not fully written"
    for b, T in enumerate(lens):
        c = lin[b]
        want = oracle.attn_exact(q[b:b + 1], c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, hd, T, S=1, window=0,
                                 query_base_pos=T - 1, win_lo=0, softmax_scale=0.1)
        ok, rel = within(got[b:b + 1], want, 2e-3)
        assert ok, f"sequence {b} (T={T}): {rel:.2e} x RMS"
    assert ops.device_faults() == 0


def test_paged_append_is_the_row_codec():
    rng = np.random.default_rng(5)
    nkv, hd, batch, n_pages, max_pages = 4, 128, 3, 9, 3
    table = np.array([[4, 1, 0], [7, 2, 0], [3, 8, 5]], np.int32)
    positions = np.array([0, 130, 383], np.int32)
    k = bf16_normal(rng, (batch, nkv, hd)); v = bf16_normal(rng, (batch, nkv, hd))
    pools = [torch.zeros((n_pages, nkv, PAGE, hd), dtype=torch.int8, device=DEV) for _ in range(2)]
    spools = [torch.zeros((n_pages, nkv, PAGE), dtype=torch.float32, device=DEV) for _ in range(2)]
    ops.kv_paged_append_quant_i8(None, dev(k), dev(v), pools[0], pools[1], spools[0], spools[1], dev(table), dev(positions),
                                 batch=batch, nkv=nkv, l_hd=hd, l_kvd=nkv * hd, max_pages=max_pages)
    torch.cuda.synchronize()
    kp, vp, ksp, vsp = host(pools[0]), host(pools[1]), host(spools[0]), host(spools[1])
    written = np.zeros((n_pages, nkv, PAGE), bool)
    for b in range(batch):
        c = KVCache("i8", nkv, 1, hd)
        c.append(k[b:b + 1], v[b:b + 1], 0)
        pg, r = table[b, positions[b] // PAGE], positions[b] % PAGE
        assert np.array_equal(kp[pg, :, r], c.k[:, 0]) and np.array_equal(vp[pg, :, r], c.v[:, 0])
        assert np.array_equal(ksp[pg, :, r], c.row_scales_f32("k")[:, 0]) and np.array_equal(vsp[pg, :, r], c.row_scales_f32("v")[:, 0])
        written[pg, :, r] = True
    assert not kp[~written].any() and not ksp[~written].any(), "rows outside the three positions were touched"
