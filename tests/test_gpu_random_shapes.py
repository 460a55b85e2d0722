"""Seeded random call shapes through nomos_attn_fused against the oracle's exact attention.

Every case draws a cache format, head geometry, number of query rows, window length, ring position, sliding
window, split count and kernel flags, builds the cache with the oracle's quantize-on-write (optionally leaving the
last rows to the call's own fused append) and checks every output row at the 2e-3 x RMS bar.  The point is the
combinations: ring wrap x forced splits x merge route (last CTA, cooperative, cluster) x verify rows x fused append,
which the per-feature tests cover one at a time.
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import bf16_normal
from tests._gpu import DEV, dev, within
from tests.test_gpu_attn import SENTINEL, TOL, build_cache, exact

pytestmark = pytest.mark.gpu


def _draw(seed):
    rng = np.random.default_rng(9000 + seed)
    fmt = ["i8", "i8", "i4", "i4b32"][rng.integers(4)]
    hd = [128, 128, 128, 256, 512][rng.integers(5)]
    nkv = int([1, 2, 4, 8][rng.integers(4)])
    kvg = int([1, 2, 4, 8][rng.integers(4)])
    S = int([1, 1, 1, 2, 3, 9][rng.integers(6)])
    klen = int(rng.integers(1, 3000))
    cap = int(klen + rng.integers(0, 40)) if rng.integers(3) else int(max(klen, S) + rng.integers(0, 8))
    start = int(rng.integers(0, 4 * cap)) if rng.integers(2) else 0       # ring position of the window's first key
    window = int(rng.integers(1, klen + 1)) if rng.integers(3) == 0 else 0
    splits = int([0, 0, 1, 2, 3, 4, 5, 9, 16][rng.integers(9)])
    flags = int([0, 0, ops.NO_TCGEN05, ops.TCGEN05_ALWAYS, ops.NO_CLUSTER, ops.NO_TMA, ops.SETTLED_CACHE][rng.integers(7)])
    n_new = int(min(S, klen)) if (rng.integers(3) == 0 and S <= 8) else 0     # rows left to the call's own fused append
    return rng, fmt, hd, nkv, kvg, S, klen, cap, start, window, splits, flags, n_new


@pytest.mark.parametrize("seed", range(128))
def test_random_call_shape_matches_the_oracle(oracle, seed):
    rng, fmt, hd, nkv, kvg, S, klen, cap, start, window, splits, flags, n_new = _draw(seed)
    S = min(S, klen)
    nh = nkv * kvg
    total = start + klen                                  # positions start .. start + klen - 1 are the window
    k_rows = bf16_normal(rng, (klen, nkv, hd))
    v_rows = bf16_normal(rng, (klen, nkv, hd))
    from tests._cases import KVCache
    full = KVCache(fmt, nkv, cap, hd)                     # the oracle's cache with every row appended
    part = KVCache(fmt, nkv, cap, hd)                     # the cache handed to the call: without its own new rows
    for c, n in ((full, klen), (part, klen - n_new)):
        for b in range(0, n, 1024):
            c.append(k_rows[b:min(n, b + 1024)], v_rows[b:min(n, b + 1024)], start + b)
    q = bf16_normal(rng, (S, nh, hd)) * np.float32(0.5)
    scale = float(1.0 / np.sqrt(hd))
    want = exact(oracle, full, q, S=S, klen=klen, win_start=start, window=window, scale=scale)
    keep = [dev(np.ascontiguousarray(q, np.float32)), dev(part.k), dev(part.v), dev(part.ks), dev(part.vs)]
    out = torch.full((S, nh, hd), SENTINEL, dtype=torch.float32, device=DEV)
    a = ops.make_args(q=keep[0], k_cache=keep[1], v_cache=keep[2], k_scales=keep[3], v_scales=keep[4], out=out,
                      kv_fmt=full.kv_fmt, S=S, nh=nh, nkv=nkv, kvg=kvg, l_hd=hd, cache_hd=hd, cache_cap=cap,
                      win_start=start, klen=klen, window=window, softmax_scale=scale, force_splits=splits, flags=flags)
    if n_new:
        nk = dev(np.ascontiguousarray(k_rows[klen - n_new:], np.float32)); nv = dev(np.ascontiguousarray(v_rows[klen - n_new:], np.float32))
        keep += [nk, nv]
        a.new_k, a.new_v, a.n_new, a.new_base_pos = nk.data_ptr(), nv.data_ptr(), n_new, total - n_new
    need = ops.attn_workspace_bytes(a)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = ws.data_ptr(), need
    what = f"seed {seed}: {fmt} hd={hd} nkv={nkv} kvg={kvg} S={S} klen={klen} cap={cap} start={start} window={window} splits={splits} flags={flags} n_new={n_new}"
    for call in range(2):                                 # twice on one workspace (the second call re-appends the same rows)
        ops.attn_fused(None, a)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert not np.any(got == SENTINEL), f"{what}: output not fully written"
        for r in range(S):
            ok, rel = within(got[r], want[r], TOL)
            assert ok, f"{what}: call {call} row {r}: {rel:.2e} x RMS (launch {ops.attn_last_launch()})"
    if n_new:                                             # the call's own append left the oracle's bytes in the ring
        assert np.array_equal(keep[1].cpu().numpy(), full.k) and np.array_equal(keep[2].cpu().numpy(), full.v), f"{what}: appended bytes"
        assert np.array_equal(keep[3].cpu().numpy(), full.ks) and np.array_equal(keep[4].cpu().numpy(), full.vs), f"{what}: appended scales"
    assert ops.device_faults() == 0
