"""GPU parity at the benchmark configurations' FULL sizes, through the C ABI, against the CPU oracle.

The other GPU tests use contexts of a few thousand keys; these run the shapes the benchmark times:
configuration 2 (32768 keys), configuration 4 (9 verify rows over 16384 cached keys), a call large
enough for the library's cost model to switch kernels, configuration 5b's sequence shards merged
from exported partials, and configurations 5a / 5b at their single-GPU sizes (batch 8 x 131072 and
524288 keys: byte offsets beyond 2^31, more than a thousand tiles per CTA).  Gate as everywhere:
max|out - exact| <= 2e-3 x RMS(exact) on the fp32 output, `exact` = the oracle's fp64 attention over
the same cache bytes.

The caches of the two largest cases are drawn directly as int8 codes and fp32 scales with the
statistics of a quantised N(0,1) tensor (on the device, seeded): pushing 4 GB of fp32 rows through
the quantiser on the host would take minutes and adds nothing to what these cases check.
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import KVCache, bf16_normal
from tests._gpu import DEV, bf16_dev, dev, host, within
from tests.test_gpu_attn import build_cache, exact

pytestmark = pytest.mark.gpu
TOL = 2e-3
SENTINEL = -1.0e30
PATHS = {"auto": 0, "mma_sync": ops.NO_TCGEN05, "tcgen05": ops.TCGEN05_ALWAYS}

_memo = {}


def _case(oracle, key, make):
    """Build a configuration's cache, query and exact answer once for all kernel paths."""
    if key not in _memo:
        _memo.clear()                                  # one large case resident at a time
        _memo[key] = make()
    return _memo[key]


def _run(c: KVCache, q, *, S, klen, scale, flags, q_type=ops.BF16, win_start=0, partial=False, batch=1, force_splits=0):
    nh = q.shape[-2]
    dq = bf16_dev(q) if q_type == ops.BF16 else dev(np.ascontiguousarray(q, np.float32))
    out = torch.full((batch, S, nh, c.l_hd), SENTINEL, dtype=torch.float32, device=DEV)
    part = torch.full((batch * S * nh, c.l_hd + 2), SENTINEL, dtype=torch.float32, device=DEV) if partial else None
    keep = [dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)]
    a = ops.make_args(q=dq, k_cache=keep[0], v_cache=keep[1], k_scales=keep[2], v_scales=keep[3], out=out, partial_out=part,
                      kv_fmt=c.kv_fmt, q_type=q_type, out_type=ops.F32, batch=batch, S=S, nh=nh, nkv=c.nkv, kvg=nh // c.nkv,
                      l_hd=c.l_hd, cache_hd=c.cache_hd, cache_cap=c.cache_cap, win_start=win_start, klen=klen,
                      softmax_scale=scale, flags=flags, force_splits=force_splits)
    choice = ops.attn_kernel_choice(a)
    need = ops.attn_workspace_bytes(a)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = ws.data_ptr(), need
    ops.attn_fused(None, a)
    torch.cuda.synchronize()
    return (host(part) if partial else host(out)), choice


@pytest.mark.parametrize("path", list(PATHS))
def test_config2_decode_i8_32768_keys(oracle, path):
    """Configuration 2 as the benchmark runs it: 32 q / 16 kv heads x 128, 32768 keys, K with 4 outlier
    channels per head, bf16 query, softmax scale 1/sqrt(128)."""
    def make():
        rng = np.random.default_rng(1002)
        nh, nkv, hd, T = 32, 16, 128, 32768
        c = build_cache("i8", rng, T, nkv, hd, outliers=True)
        q = bf16_normal(rng, (1, nh, hd))
        return c, q, exact(oracle, c, q, klen=T, scale=1.0 / np.sqrt(128.0))
    c, q, want = _case(oracle, "c2", make)
    got, choice = _run(c, q, S=1, klen=32768, scale=1.0 / np.sqrt(128.0), flags=PATHS[path])
    assert choice == (1 if path == "tcgen05" else 0)
    ok, rel = within(got[0], want, TOL)
    assert ok, f"{path}: {rel:.2e} x RMS"
    assert not np.any(got == SENTINEL)


@pytest.mark.parametrize("path", list(PATHS))
def test_config4_verify_9_rows_over_16384_keys(oracle, path):
    """Configuration 4: 9 draft rows (causal among themselves) against 16384 cached keys, every row gated
    against its own RMS."""
    def make():
        rng = np.random.default_rng(1004)
        nh, nkv, hd, S, T0 = 32, 16, 128, 9, 16384
        c = build_cache("i8", rng, T0 + S, nkv, hd)
        q = bf16_normal(rng, (S, nh, hd))
        return c, q, exact(oracle, c, q, S=S, klen=T0 + S, scale=1.0 / np.sqrt(128.0))
    c, q, want = _case(oracle, "c4", make)
    got, choice = _run(c, q, S=9, klen=16384 + 9, scale=1.0 / np.sqrt(128.0), flags=PATHS[path])
    assert choice == (0 if path == "mma_sync" else 1)
    for r in range(9):
        ok, rel = within(got[0][r], want[r], TOL)
        assert ok, f"{path} row {r}: {rel:.2e} x RMS"


def _device_cache(batch, nkv, T, hd, seed):
    """int8 codes ~ round(N(0,1) * 127 / 4) clipped, scales ~ 4/127 * U(0.8, 1.2): a quantised N(0,1) tensor."""
    g = torch.Generator(device=DEV); g.manual_seed(seed)
    def codes():
        x = torch.empty((batch, nkv, T, hd), dtype=torch.int8, device=DEV)
        for b in range(batch):
            for h in range(nkv):
                x[b, h] = torch.randn((T, hd), generator=g, device=DEV).mul_(127.0 / 4.0).round_().clamp_(-127, 127).to(torch.int8)
        return x
    k, v = codes(), codes()
    ks = (torch.rand((batch, nkv, T), generator=g, device=DEV) * 0.4 + 0.8) * (4.0 / 127.0)
    vs = (torch.rand((batch, nkv, T), generator=g, device=DEV) * 0.4 + 0.8) * (4.0 / 127.0)
    return k, v, ks.contiguous(), vs.contiguous()


def _exact_of_device_cache(oracle, cache, q, b, T, scale, lo=0, klen=None, want_partial=False):
    k, v, ks, vs = cache
    nkv, hd = k.shape[1], k.shape[3]
    nh = q.shape[-2]
    klen = klen or T
    return oracle.attn_exact(q[b], host(k[b]), host(v[b]), host(ks[b]), host(vs[b]), oracle.KV_I8, nh, nkv, hd, hd, T, S=1, window=0, query_base_pos=lo + klen - 1, win_lo=lo,
                             softmax_scale=scale, want_partial=want_partial)


def _call(cache, q, *, batch, T, scale, flags=0, win_start=0, klen=None, partial=False):
    k, v, ks, vs = cache
    nkv, hd = k.shape[1], k.shape[3]
    nh = q.shape[-2]
    dq = bf16_dev(q)
    out = torch.full((batch, 1, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    part = torch.full((batch * nh, hd + 2), SENTINEL, dtype=torch.float32, device=DEV) if partial else None
    a = ops.make_args(q=dq, k_cache=k, v_cache=v, k_scales=ks, v_scales=vs, out=out, partial_out=part, kv_fmt=ops.KV_I8,
                      q_type=ops.BF16, out_type=ops.F32, batch=batch, S=1, nh=nh, nkv=nkv, kvg=nh // nkv, l_hd=hd, cache_hd=hd,
                      cache_cap=T, win_start=win_start, klen=klen or T, softmax_scale=scale, flags=flags)
    choice = ops.attn_kernel_choice(a)
    need = ops.attn_workspace_bytes(a)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = ws.data_ptr(), need
    ops.attn_fused(None, a)
    torch.cuda.synchronize()
    return (part if partial else out), choice


def test_library_switches_kernel_for_large_caches(oracle):
    """Batch 2 x 65536 keys x 16 KV heads = 537 MB of cache: the cost model's own pick must be the tcgen05
    kernel, and the same call pinned to the mma.sync kernel must agree with the oracle too."""
    nh, nkv, hd, T, B = 32, 16, 128, 65536, 2
    cache = _device_cache(B, nkv, T, hd, 2401)
    rng = np.random.default_rng(2401)
    q = bf16_normal(rng, (B, 1, nh, hd))
    scale = 1.0 / np.sqrt(128.0)
    wants = [_exact_of_device_cache(oracle, cache, q, b, T, scale) for b in range(B)]
    for flags, expect in ((0, 1), (ops.NO_TCGEN05, 0)):
        out, choice = _call(cache, q, batch=B, T=T, scale=scale, flags=flags)
        assert choice == expect
        got = host(out)
        for b in range(B):
            ok, rel = within(got[b], wants[b], TOL)
            assert ok, f"flags={flags} sequence {b}: {rel:.2e} x RMS"


def test_config5b_shards_of_65536_keys_merge_to_the_full_answer(oracle):
    """Sequence-sharded decode as configuration 5b runs it on 8 GPUs: shards of 65536 keys export (o, m, l)
    through partial_out, nomos_attn_merge_partials merges them.  Two shards of one 131072-key cache here."""
    nh, nkv, hd, T, G = 32, 16, 128, 131072, 2
    cache = _device_cache(1, nkv, T, hd, 2502)
    rng = np.random.default_rng(2502)
    q = bf16_normal(rng, (1, 1, nh, hd))
    scale = 1.0 / np.sqrt(128.0)
    want = _exact_of_device_cache(oracle, cache, q, 0, T, scale)
    chunk = T // G
    gathered = torch.empty((G, nh, hd + 2), dtype=torch.float32, device=DEV)
    for g in range(G):
        part, choice = _call(cache, q, batch=1, T=T, scale=scale, win_start=g * chunk, klen=chunk, partial=True)
        assert choice == 0                              # 277 MB per shard: still the mma.sync kernel (it switches at 330 MB)
        gathered[g].copy_(part)
        # the shard's exported triple against the oracle's for the same keys
        _, wp = _exact_of_device_cache(oracle, cache, q, 0, T, scale, lo=g * chunk, klen=chunk, want_partial=True)
        gp = host(part).astype(np.float64)
        w = np.exp(gp[:, hd] - wp[:, hd])               # references may differ: compare in a common one
        assert np.allclose(gp[:, hd + 1] * w, wp[:, hd + 1], rtol=2e-3)
    out = torch.full((nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    ops.attn_merge_partials(None, gathered, G, nh, hd, out)
    torch.cuda.synchronize()
    ok, rel = within(host(out)[None], want, TOL)
    assert ok, f"{rel:.2e} x RMS"


def test_config5a_batch8_131072_keys_single_gpu(oracle):
    """Configuration 5a on one GPU: 8 sequences x 131072 keys (4.4 GB of cache; K and V planes of 2.1 GB each,
    so row offsets exceed 2^31).  Three of the eight sequences are checked against the oracle."""
    nh, nkv, hd, T, B = 32, 16, 128, 131072, 8
    cache = _device_cache(B, nkv, T, hd, 2503)
    rng = np.random.default_rng(2503)
    q = bf16_normal(rng, (B, 1, nh, hd))
    scale = 1.0 / np.sqrt(128.0)
    out, choice = _call(cache, q, batch=B, T=T, scale=scale)
    assert choice == 1
    got = host(out)
    assert not np.any(got == SENTINEL)
    for b in (0, 5, 7):
        want = _exact_of_device_cache(oracle, cache, q, b, T, scale)
        ok, rel = within(got[b], want, TOL)
        assert ok, f"sequence {b}: {rel:.2e} x RMS"


def test_config5b_524288_keys_single_gpu(oracle):
    """Configuration 5b on one GPU: one sequence of 524288 keys (2.2 GB), both kernels."""
    nh, nkv, hd, T = 32, 16, 128, 524288
    cache = _device_cache(1, nkv, T, hd, 2504)
    rng = np.random.default_rng(2504)
    q = bf16_normal(rng, (1, 1, nh, hd))
    scale = 1.0 / np.sqrt(128.0)
    want = _exact_of_device_cache(oracle, cache, q, 0, T, scale)
    for flags in (0, ops.NO_TCGEN05):
        out, _ = _call(cache, q, batch=1, T=T, scale=scale, flags=flags)
        ok, rel = within(host(out)[0], want, TOL)
        assert ok, f"flags={flags}: {rel:.2e} x RMS"
