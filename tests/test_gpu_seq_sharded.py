"""The sequence-sharded decode (nomos_attn_seq_sharded): every rank's attention kernel pushes its chunk's (o, m, l)
rows into the peers' mailboxes, waits for theirs with a time limit and writes the merged output -- one launch.

On ONE GPU two ranks cannot run as two kernels that wait on each other, so the exchange is checked in three parts:
  * rank 0 of a two-rank group with rank 1's rows and stamps already sitting in its mailbox (written by the test
    from an exported partial): the output must equal full attention, and the rows rank 0 pushed into the "peer"
    mailbox (a second buffer on the same GPU) must be its own chunk's partial with the step's stamp;
  * a peer that never shows up (stamps nothing sets): the wait runs out, the launch returns without an output,
    the status call answers -4, and the context stays usable;
  * with two or more GPUs visible: real ranks as child processes, mailboxes opened across processes, several
    steps in a row (both mailbox slots reused), each step's output against the oracle.
"""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from nomos_nvfp4_b200 import ops
from tests._cases import bf16_normal
from tests._gpu import DEV, dev, host, within
from tests.test_gpu_attn import build_cache, exact

pytestmark = pytest.mark.gpu
TOL = 2e-3
ROOT = Path(__file__).resolve().parent.parent


def shard_args(c, dq, out, *, win_start, klen, scale, flags=0, partial=None):
    nh = dq.shape[-2]
    keep = [dev(c.k), dev(c.v), dev(c.ks), dev(c.vs)]
    a = ops.make_args(q=dq, k_cache=keep[0], v_cache=keep[1], k_scales=keep[2], v_scales=keep[3], out=out, partial_out=partial,
                      kv_fmt=c.kv_fmt, nh=nh, nkv=c.nkv, kvg=nh // c.nkv, l_hd=c.l_hd, cache_hd=c.cache_hd,
                      cache_cap=c.cache_cap, win_start=win_start, klen=klen, softmax_scale=scale, flags=flags)
    need = ops.attn_workspace_bytes(a)
    ws = torch.empty(max(need, 4096) + 4096, dtype=torch.uint8, device=DEV)
    a.workspace, a.ws_bytes = ws.data_ptr(), ws.numel()
    return a, keep + [ws]


@pytest.mark.parametrize("flags", [ops.NO_TCGEN05, ops.TCGEN05_ALWAYS])
@pytest.mark.parametrize("fmt,hd,T", [("i8", 128, 6000), ("i8", 128, 200), ("i4b32", 256, 3000)])
def test_rank0_merges_a_peer_row_that_is_already_there(oracle, flags, fmt, hd, T):
    if fmt != "i8" and flags == ops.TCGEN05_ALWAYS:
        pytest.skip("the tcgen05 kernel serves int8 / head_dim 128")
    rng = np.random.default_rng(T + hd)
    nh, nkv, world, step = 8, 4, 2, 5
    c = build_cache(fmt, rng, T, nkv, hd)
    q = bf16_normal(rng, (1, nh, hd))
    scale = 1.0 / np.sqrt(hd)
    want = exact(oracle, c, q, klen=T, scale=scale)
    dq = dev(np.ascontiguousarray(q, np.float32))
    half = (T // 2) // 32 * 32
    # rank 1's chunk through the ordinary partial export
    part1 = torch.zeros((nh, hd + 2), dtype=torch.float32, device=DEV)
    a1, keep1 = shard_args(c, dq, None, win_start=half, klen=T - half, scale=scale, flags=flags, partial=part1)
    ops.attn_fused(None, a1)
    torch.cuda.synchronize()
    # mailboxes of the two "ranks" (both on this GPU): rows [2][world][nh][hd+2] fp32, then stamps [2][world][nh] u64
    nbytes = ops.attn_peer_mailbox_bytes(world, nh, hd)
    rows_bytes = (2 * world * nh * (hd + 2) * 4 + 15) // 16 * 16
    box0 = torch.zeros(nbytes, dtype=torch.uint8, device=DEV); box1 = torch.zeros_like(box0)
    slot = step & 1
    rows0 = box0[:2 * world * nh * (hd + 2) * 4].view(torch.float32).view(2, world, nh, hd + 2)
    flags0 = box0[rows_bytes:rows_bytes + 2 * world * nh * 8].view(torch.int64).view(2, world, nh)
    rows0[slot, 1].copy_(part1)
    flags0[slot, 1].fill_(step)
    out = torch.full((1, nh, hd), -1e30, dtype=torch.float32, device=DEV)
    a0, keep0 = shard_args(c, dq, out, win_start=0, klen=half, scale=scale, flags=flags)
    peer = ops.make_peer(0, world, [box0, box1], nbytes, step, timeout_us=200000)
    ops.attn_seq_sharded(None, a0, peer)
    assert ops.attn_seq_sharded_status(None) == 0
    ok, rel = within(host(out), want, TOL)
    assert ok, f"{rel:.2e} x RMS"
    # what rank 0 pushed to its peer: its own chunk's partial, stamped with the step
    rows1 = box1[:2 * world * nh * (hd + 2) * 4].view(torch.float32).view(2, world, nh, hd + 2)
    flags1 = box1[rows_bytes:rows_bytes + 2 * world * nh * 8].view(torch.int64).view(2, world, nh)
    assert torch.all(flags1[slot, 0] == step) and torch.all(flags1[1 - slot] == 0)
    _, wp = oracle.attn_exact(q, c.k, c.v, c.ks, c.vs, c.kv_fmt, nh, nkv, hd, c.cache_hd, c.cache_cap, query_base_pos=half - 1,
                              win_lo=0, softmax_scale=scale, want_partial=True)
    merged = oracle.merge_partials(np.stack([host(rows1[slot, 0]).astype(np.float64), host(part1).astype(np.float64)]), hd)
    assert within(merged[None], want, TOL)[0]
    assert np.allclose(host(rows1[slot, 0])[:, hd + 1] * np.exp(host(rows1[slot, 0])[:, hd].astype(np.float64) - wp[:, hd]), wp[:, hd + 1], rtol=2e-3)


def test_a_peer_that_never_arrives_is_given_up_on():
    rng = np.random.default_rng(3)
    nh, nkv, hd, T, world = 8, 4, 128, 2000, 2
    c = build_cache("i8", rng, T, nkv, hd)
    q = bf16_normal(rng, (1, nh, hd))
    dq = dev(np.ascontiguousarray(q, np.float32))
    nbytes = ops.attn_peer_mailbox_bytes(world, nh, hd)
    box0 = torch.zeros(nbytes, dtype=torch.uint8, device=DEV); box1 = torch.zeros_like(box0)
    out = torch.full((1, nh, hd), -1e30, dtype=torch.float32, device=DEV)
    a0, keep0 = shard_args(c, dq, out, win_start=0, klen=T, scale=0.1)
    assert ops.device_faults(clear=True) == 0
    peer = ops.make_peer(0, world, [box0, box1], nbytes, 1, timeout_us=20000)       # 20 ms
    ops.attn_seq_sharded(None, a0, peer)
    assert ops.attn_seq_sharded_status(None, clear=True) == -4
    assert torch.all(out == -1e30), "no output may be written when the exchange failed"
    assert ops.device_faults() == 0                                               # the status call cleared its bit
    # the context is intact: the same call with the peer's rows present succeeds
    rows_bytes = (2 * world * nh * (hd + 2) * 4 + 15) // 16 * 16
    flags0 = box0[rows_bytes:rows_bytes + 2 * world * nh * 8].view(torch.int64).view(2, world, nh)
    flags0[0, 1].fill_(2)                     # step 2, slot 0: an empty partial (l = 0) from the "peer"
    peer = ops.make_peer(0, world, [box0, box1], nbytes, 2, timeout_us=20000)
    ops.attn_seq_sharded(None, a0, peer)
    assert ops.attn_seq_sharded_status(None) == 0
    assert not torch.any(out == -1e30)


def test_bad_peer_arguments():
    t = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    a = ops.make_args(q=t, k_cache=t, v_cache=t, k_scales=t, v_scales=t, out=t, nh=8, nkv=4, kvg=2, l_hd=128, cache_hd=128,
                      cache_cap=64, klen=64)
    for kw, status in ((dict(step=0), -1), (dict(world=9), -1), (dict(rank=2), -1), (dict(nbytes=64), -3)):
        world = kw.get("world", 2)
        peer = ops.make_peer(kw.get("rank", 0), world, [t] * min(world, 8), kw.get("nbytes", 1 << 16), kw.get("step", 1))
        with pytest.raises(ops.NomosError) as e:
            ops.attn_seq_sharded(None, a, peer)
        assert e.value.status == status
    torch.cuda.synchronize()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_real_ranks_exchange_through_peer_memory(world):
    """One process per GPU; skipped when the box shows fewer GPUs than ranks."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", env["MASTER_PORT"], str(ROOT / "tests" / "seq_sharded_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "SEQ_SHARDED_OK" in r.stdout
