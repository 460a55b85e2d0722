"""The workspace-free entry point (nomos_attn_fused_static_ws) against the regular one.

Some callers of the library have no buffer to pass as split workspace: an engine that hands its
whole device-memory budget out at start-up, or a decode loop that must never call the allocator.
For them the library carries a fixed 4 MiB scratch array.  This file checks, through the C ABI,
that the workspace-free call gives the same attention output as the regular call and as the CPU
oracle's exact attention over the same cache (the 2e-3 x RMS bar of the other GPU tests, both
times), twice in a row so that the second call runs over the scratch contents the first one left
behind, and that an oversized request is refused instead of overrunning the array.  It is named
to be collected last.
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import bf16_normal
from tests._gpu import DEV, dev, host, within
from tests.test_gpu_attn import build_cache, exact

pytestmark = pytest.mark.gpu


def _args(c, q, out, T, scale):
    nh = q.shape[-2]
    keep = [dev(np.ascontiguousarray(q, np.float32)), dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)]
    a = ops.make_args(q=keep[0], k_cache=keep[1], v_cache=keep[2], k_scales=keep[3], v_scales=keep[4], out=out,
                      kv_fmt=c.kv_fmt, nh=nh, nkv=c.nkv, kvg=nh // c.nkv, l_hd=c.l_hd, cache_hd=c.cache_hd,
                      cache_cap=c.cache_cap, klen=T, softmax_scale=scale)
    return a, keep


def test_static_workspace_matches_regular_entry_point_twice(oracle):
    rng = np.random.default_rng(4242)
    nh, nkv, hd = 32, 16, 128
    for call, T in enumerate((6000, 3500)):               # two calls in a row; both split the sequence
        c = build_cache("i8", rng, T, nkv, hd, outliers=True)
        q = bf16_normal(rng, (1, nh, hd))
        scale = 1.0 / np.sqrt(128.0)
        want = torch.full((1, nh, hd), -1e30, dtype=torch.float32, device=DEV)
        a, keep = _args(c, q, want, T, scale)
        need = ops.attn_workspace_bytes(a)
        assert need > 0, "the case must use split scratch, otherwise the test checks nothing"
        ws = torch.empty(need, dtype=torch.uint8, device=DEV)
        a.workspace, a.ws_bytes = ws.data_ptr(), need
        ops.attn_fused(None, a)
        got = torch.full((1, nh, hd), -1e30, dtype=torch.float32, device=DEV)
        b, keep2 = _args(c, q, got, T, scale)              # no workspace fields set at all
        ops.attn_fused_static_ws(None, b)
        torch.cuda.synchronize()
        ok, rel = within(host(got), host(want), 2e-3)
        assert ok, f"call {call}: static-workspace output differs by {rel:.2e} x RMS"
        ok, rel = within(host(got), exact(oracle, c, q, klen=T, scale=scale), 2e-3)
        assert ok, f"call {call}: static-workspace output is {rel:.2e} x RMS from the oracle"
        assert not np.any(host(got) == -1e30), "output not fully written"


def test_static_workspace_refuses_oversized_request():
    rng = np.random.default_rng(7)
    nh, nkv, hd, S, T = 32, 16, 128, 17, 4096            # 17 verify rows x 32 heads: split scratch above 4 MiB
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (S, nh, hd))
    out = torch.zeros((S, nh, hd), dtype=torch.float32, device=DEV)
    keep = [dev(q), dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)]
    a = ops.make_args(q=keep[0], k_cache=keep[1], v_cache=keep[2], k_scales=keep[3], v_scales=keep[4], out=out,
                      kv_fmt=c.kv_fmt, S=S, nh=nh, nkv=nkv, kvg=2, l_hd=hd, cache_hd=hd, cache_cap=T, klen=T,
                      force_splits=32)
    if ops.attn_workspace_bytes(a) <= (4 << 20):
        pytest.skip("plan fits the built-in scratch on this device")
    with pytest.raises(ops.NomosError) as e:
        ops.attn_fused_static_ws(None, a)
    assert e.value.status == -3
    torch.cuda.synchronize()


def test_no_device_fault_bits_after_the_suite():
    """Every wait in the kernels is bounded and reports through a sticky device word; after
    all the GPU tests above it must still read zero."""
    assert ops.device_faults() == 0
