"""GPU parity of the cooperative split merge, through the C ABI.

When the partials of one unit of work (a KV head's query rows) are large and the whole grid is resident at once,
the library lets every CTA of the unit merge a share of the output rows once all of them have arrived, instead of
leaving the merge to the CTA that arrives last.  The launcher takes that route when
    2 <= splits <= 64,  splits x rows per unit x (head_dim + 2) x 4 bytes >= 48 KiB,
    the CTAs of the launch fit the SMs at once,  the outputs are 8-byte aligned;
with at most 12 splits the shares are merged by the no-staging merge of verify calls, with more by the
lane-per-split merge.
The cases below are sized to meet those conditions on both kernels; each runs several calls in a row on one
workspace (the arrival and departure words must come back to their idle state) and checks every output, and the
exported partials, against the oracle's exact attention.
"""
import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import bf16_normal
from tests._gpu import DEV, dev, host, within
from tests.test_gpu_attn import SENTINEL, TOL, build_cache, exact

pytestmark = pytest.mark.gpu

CASES = [
    # fmt, hd, nkv, kvg, S, T, splits, flags                  bytes of partials per unit
    ("i4b32", 512, 2, 8, 1, 8192, 32, 0),                   # 32 x 8 x 514 x 4 = 526 KB
    ("i8", 512, 2, 8, 1, 6000, 40, 0),                      # ragged last tile, 658 KB
    ("i8", 256, 2, 8, 1, 8192, 64, 0),                      # 64 x 8 x 258 x 4 = 528 KB
    ("i8", 128, 4, 2, 9, 16384, 32, ops.TCGEN05_ALWAYS),    # 32 x 18 x 130 x 4 = 300 KB, tcgen05 kernel (verify rows)
    ("i8", 128, 4, 2, 9, 16384, 32, ops.NO_TCGEN05),        # the same rows on the mma.sync kernel
    ("i8", 128, 16, 2, 9, 16393, 9, ops.TCGEN05_ALWAYS),    # the verify configuration: 9 x 18 x 130 x 4 = 84 KB, few splits
    ("i8", 128, 16, 2, 9, 16393, 9, ops.NO_TCGEN05),
    ("i4b32", 256, 4, 8, 1, 4000, 12, 0),                   # 12 x 8 x 258 x 4 = 99 KB, few splits, wide head, ragged
]


@pytest.mark.parametrize("fmt,hd,nkv,kvg,S,T,splits,flags", CASES)
@pytest.mark.parametrize("out_type", [ops.F32, ops.BF16])
def test_cooperative_merge_matches_oracle_on_repeated_calls(oracle, fmt, hd, nkv, kvg, S, T, splits, flags, out_type):
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    if flags != ops.NO_TCGEN05 or S == 1:     # (verify rows on the mma.sync kernel run as 8-row groups: whichever merge they get)
        assert splits * nkv <= sm, "the case must keep its whole grid resident"
        assert splits * min(S * kvg, 32) * (hd + 2) * 4 >= 48 * 1024
    rng = np.random.default_rng(hd * 7 + T + splits)
    nh = nkv * kvg
    c = build_cache(fmt, rng, T, nkv, hd, outliers=(hd == 128))
    dk, dv, dks, dvs = dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)
    scale = 1.0 / np.sqrt(hd)
    ws = None
    for call in range(3):
        q = bf16_normal(rng, (S, nh, hd))
        dq = dev(np.ascontiguousarray(q, np.float32))
        out = torch.full((S, nh, hd), SENTINEL, dtype=torch.bfloat16 if out_type == ops.BF16 else torch.float32, device=DEV)
        part = torch.full((S * nh, hd + 2), SENTINEL, dtype=torch.float32, device=DEV) if call == 2 else None
        a = ops.make_args(q=dq, k_cache=dk, v_cache=dv, k_scales=dks, v_scales=dvs, out=out, partial_out=part,
                          kv_fmt=c.kv_fmt, out_type=out_type, S=S, nh=nh, nkv=nkv, kvg=kvg, l_hd=hd, cache_hd=c.cache_hd,
                          cache_cap=c.cache_cap, klen=T, softmax_scale=scale, force_splits=splits, flags=flags)
        if flags:
            assert ops.attn_kernel_choice(a) == (1 if flags == ops.TCGEN05_ALWAYS else 0)
        need = ops.attn_workspace_bytes(a)
        if ws is None:
            ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
        a.workspace, a.ws_bytes = ws.data_ptr(), need
        ops.attn_fused(None, a)
        torch.cuda.synchronize()
        got = out.float().cpu().numpy()
        want = exact(oracle, c, q, S=S, klen=T, scale=scale)
        for r in range(S if part is None else 0):           # (a call that exports partials leaves `out` alone)
            # a bf16 output adds half an ulp (2^-9 relative) of the largest element to the bar
            bar = TOL if out_type == ops.F32 else TOL + 2.0 ** -8 * float(np.abs(want[r]).max() / np.sqrt(np.mean(want[r] ** 2)))
            ok, rel = within(got[r], want[r], bar)
            assert ok, f"call {call} row {r}: {rel:.2e} x RMS"
        assert part is not None or not np.any(got == SENTINEL), "output not fully written"
        if part is not None:
            p = host(part).reshape(S, nh, hd + 2)
            assert not np.any(p == SENTINEL), "exported partials not fully written"
            o = p[..., :hd] / p[..., hd + 1:hd + 2]
            for r in range(S):
                ok, rel = within(o[r], want[r], TOL)
                assert ok, f"exported partial row {r}: {rel:.2e} x RMS"
    assert ops.device_faults() == 0
