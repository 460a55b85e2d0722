"""GPU parity of the cluster route of the mma.sync kernel, through the C ABI.

When the splits of every KV head fit one thread-block cluster (2..16 CTAs) and all clusters of the launch are
resident at once, the kernel merges the splits through distributed shared memory instead of the workspace and an
arrival counter.  Every case runs with the route allowed and with NOMOS_ATTN_NO_CLUSTER, several calls in a row,
and both are held to the oracle's exact attention (2e-3 x RMS); the two routes merge the same per-CTA rows, so
they also have to agree with each other to rounding.
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import bf16_normal
from tests._gpu import DEV, dev, within
from tests.test_gpu_attn import SENTINEL, TOL, build_cache, exact

pytestmark = pytest.mark.gpu

CASES = [
    # fmt, hd, nkv, kvg, S, T, splits
    ("i8", 128, 16, 2, 1, 32768, 0),        # configuration 2: two rows per unit, the counter merge either way
    ("i8", 128, 4, 4, 1, 5000, 2),
    ("i8", 128, 16, 2, 1, 1024, 3),         # a sliding-window ring: two rows per unit, small clusters
    ("i4b32", 128, 16, 2, 1, 1024, 4),
    ("i8", 128, 4, 4, 1, 5000, 3),
    ("i8", 128, 4, 8, 1, 9001, 16),         # the largest cluster
    ("i8", 128, 2, 8, 1, 3000, 7),
    ("i4", 128, 4, 4, 1, 4097, 5),
    ("i4b32", 128, 4, 8, 1, 4097, 9),
    ("i4b32", 256, 4, 4, 1, 2048, 8),       # quads of two warps
    ("i4b32", 512, 2, 8, 1, 4096, 12),      # quads of four warps
    ("i8", 128, 4, 2, 9, 6000, 6),          # verify rows: three 8-row groups per KV head
    ("i8", 128, 2, 2, 3, 2000, 4),
]


def _call(c, q, S, T, scale, splits, flags, keep):
    nh = q.shape[-2]
    out = torch.full((S, nh, c.l_hd), SENTINEL, dtype=torch.float32, device=DEV)
    a = ops.make_args(q=keep["q"], k_cache=keep["k"], v_cache=keep["v"], k_scales=keep["ks"], v_scales=keep["vs"], out=out,
                      kv_fmt=c.kv_fmt, S=S, nh=nh, nkv=c.nkv, kvg=nh // c.nkv, l_hd=c.l_hd, cache_hd=c.cache_hd,
                      cache_cap=c.cache_cap, klen=T, softmax_scale=scale, force_splits=splits, flags=flags | ops.NO_TCGEN05)
    need = ops.attn_workspace_bytes(a)
    if keep.get("ws") is None or keep["ws"].numel() < max(need, 16):
        keep["ws"] = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = keep["ws"].data_ptr(), need
    ops.attn_fused(None, a)
    kernel, nsplit, route = ops.attn_last_launch()
    assert kernel == 0 and (splits == 0 or nsplit == splits)
    assert route in ((1, 2, 3) if not flags & ops.NO_CLUSTER else (1, 2)), "NOMOS_ATTN_NO_CLUSTER must keep the counter merge"
    keep.setdefault("routes", set()).add(route)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("fmt,hd,nkv,kvg,S,T,splits", CASES)
def test_cluster_and_counter_merges_match_the_oracle(oracle, fmt, hd, nkv, kvg, S, T, splits):
    rng = np.random.default_rng(hd + T + splits)
    nh = nkv * kvg
    c = build_cache(fmt, rng, T, nkv, hd, outliers=(hd == 128 and fmt == "i8"))
    keep = {"k": dev(c.k), "v": dev(c.v), "ks": dev(c.ks), "vs": dev(c.vs), "ws": None}
    scale = 1.0 / np.sqrt(hd)
    for call in range(3):
        q = bf16_normal(rng, (S, nh, hd))
        keep["q"] = dev(np.ascontiguousarray(q, np.float32))
        want = exact(oracle, c, q, S=S, klen=T, scale=scale)
        got = {name: _call(c, q, S, T, scale, splits, flags, keep) for name, flags in (("cluster", 0), ("counter", ops.NO_CLUSTER))}
        for name, g in got.items():
            assert not np.any(g == SENTINEL), f"{name}: output not fully written"
            for r in range(S):
                ok, rel = within(g[r], want[r], TOL)
                assert ok, f"call {call} {name} row {r}: {rel:.2e} x RMS"
        ok, rel = within(got["cluster"], got["counter"], 1e-5)
        assert ok, f"call {call}: the two merges differ by {rel:.2e} x RMS"
    assert ops.device_faults() == 0
    print(f"merge routes taken: {sorted(keep['routes'])}")
