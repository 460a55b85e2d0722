"""Child process of tests/test_gpu_seq_sharded.py: one rank of a real sequence-sharded decode group.

Launched by torchrun (one process per GPU).  Every rank builds the same seeded cache on the host, keeps its own
chunk on its GPU, and runs several decode steps through SeqShardGroup; every step's output is checked against
the oracle's exact attention over the whole context on every rank.  The process group (gloo: nothing here needs a
collective library on the GPUs) only passes the mailbox handles round and lines the ranks up.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from nomos_nvfp4_b200 import ops                                    # noqa: E402
from nomos_nvfp4_b200.sharding import SeqShardGroup, sequence_shard   # noqa: E402
from oracle import oracle as orc                                    # noqa: E402
from tests._cases import KVCache, bf16_normal                        # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("gloo")

    def all_gather_bytes(b):
        out = [None] * world
        dist.all_gather_object(out, b)
        return out

    rng = np.random.default_rng(4321)                               # the same inputs on every rank
    nh, nkv, hd, T, steps = 32, 16, 128, 40000, 5
    k, v = bf16_normal(rng, (T, nkv, hd)), bf16_normal(rng, (T, nkv, hd))
    qs = bf16_normal(rng, (steps, 1, nh, hd))
    c = KVCache("i8", nkv, T, hd)
    c.append(k, v, 0)
    scale = 1.0 / np.sqrt(hd)
    begin, n = sequence_shard(T, world, rank)
    dk, dv = torch.from_numpy(c.k).to(dev), torch.from_numpy(c.v).to(dev)
    dks, dvs = torch.from_numpy(c.ks).to(dev), torch.from_numpy(c.vs).to(dev)
    group = SeqShardGroup(rank, world, nh, hd, all_gather_bytes, timeout_us=5_000_000)
    outs = torch.full((steps, 1, nh, hd), -1e30, dtype=torch.float32, device=dev)
    dq = torch.from_numpy(np.ascontiguousarray(qs)).to(dev)
    args = []
    for i in range(steps):
        flags = (0, ops.NO_TCGEN05, ops.TCGEN05_ALWAYS)[(i + rank) % 3]      # ranks need not run the same kernel
        a = ops.make_args(q=dq[i], k_cache=dk, v_cache=dv, k_scales=dks, v_scales=dvs, out=outs[i], kv_fmt=ops.KV_I8, nh=nh, nkv=nkv,
                          kvg=nh // nkv, l_hd=hd, cache_hd=hd, cache_cap=T, win_start=begin, klen=n, softmax_scale=scale, flags=flags)
        args.append(a)
    need = max(ops.attn_workspace_bytes(a) for a in args)
    ws = torch.empty(max(need, 4096) + 65536, dtype=torch.uint8, device=dev)
    for a in args:
        a.workspace, a.ws_bytes = ws.data_ptr(), ws.numel()
    dist.barrier()
    for a in args:                                                  # back to back: both mailbox slots are reused
        group.decode(None, a)
    rc = group.status(None)
    assert rc == 0, f"rank {rank}: exchange status {rc}"
    got = outs.cpu().numpy()
    worst = 0.0
    for i in range(steps):
        want = orc.attn_exact(qs[i], c.k, c.v, c.ks, c.vs, orc.KV_I8, nh, nkv, hd, hd, T, query_base_pos=T - 1, softmax_scale=scale)
        err = float(np.max(np.abs(got[i] - want)) / np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        worst = max(worst, err)
        assert err <= 2e-3, f"rank {rank} step {i}: {err:.2e} x RMS"
    dist.barrier()
    group.close()
    dist.destroy_process_group()
    if rank == 0:
        print(f"SEQ_SHARDED_OK world={world} worst={worst:.2e}")


if __name__ == "__main__":
    main()
