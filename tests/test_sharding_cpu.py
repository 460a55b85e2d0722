"""Multi-GPU host logic on CPU: the two work partitions, exercised by two gloo ranks.

Each rank computes its shard with the CPU oracle (standing in for the kernel), the partials cross
the process group exactly as they cross NCCL on GPUs, and the merged result must equal full
attention.  No GPU is involved."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nomos_nvfp4_b200.sharding import head_group_shard, sequence_shard


def test_head_group_shard_covers_all_heads():
    for world in (1, 2, 4, 8, 16):
        seen_kv, seen_q = [], []
        for r in range(world):
            s = head_group_shard(16, 2, world, r)
            seen_kv += list(range(s.kv_begin, s.kv_end)); seen_q += list(range(s.q_begin, s.q_end))
            assert s.nh == s.nkv * 2
        assert seen_kv == list(range(16)) and seen_q == list(range(32))
    with pytest.raises(ValueError):
        head_group_shard(16, 2, 3, 0)
    with pytest.raises(ValueError):
        head_group_shard(16, 2, 4, 4)


@pytest.mark.parametrize("klen", [1, 31, 32, 33, 1000, 4096, 524288])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_sequence_shard_partitions_window(klen, world):
    pos = 0
    for r in range(world):
        b, n = sequence_shard(klen, world, r)
        assert b == pos and n >= 0 and (b % 32 == 0 or n == 0)
        pos += n
    assert pos == klen


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as orc
        from tests._cases import KVCache, bf16_normal
        rng = np.random.default_rng(99)                      # same inputs on every rank
        nh, nkv, hd, T = 8, 4, 128, 777
        k, v = bf16_normal(rng, (T, nkv, hd)), bf16_normal(rng, (T, nkv, hd))
        q = bf16_normal(rng, (1, nh, hd))
        c = KVCache("i8", nkv, T, hd)
        c.append(k, v, 0)
        full = orc.attn_exact(q, c.k, c.v, c.ks, c.vs, orc.KV_I8, nh, nkv, hd, hd, T, query_base_pos=T - 1, softmax_scale=0.2)
        if mode == "seq":
            b, n = sequence_shard(T, world, rank)
            part = np.zeros((nh, hd + 2), np.float64)
            if n > 0:
                _, part = orc.attn_exact(q, c.k, c.v, c.ks, c.vs, orc.KV_I8, nh, nkv, hd, hd, T, query_base_pos=b + n - 1,
                                         win_lo=b, softmax_scale=0.2, want_partial=True)
            mine = torch.from_numpy(part.astype(np.float32))  # the wire format is fp32 [nh, hd+2]
            gathered = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine)
            merged = orc.merge_partials(torch.stack(gathered).numpy().astype(np.float64), hd)
            err = float(np.abs(merged - full[0]).max() / np.sqrt(np.mean(full.astype(np.float64) ** 2)))
        else:
            s = head_group_shard(nkv, nh // nkv, world, rank)
            sub = KVCache("i8", s.nkv, T, hd)
            sub.append(k[:, s.kv_begin:s.kv_end], v[:, s.kv_begin:s.kv_end], 0)
            mine = orc.attn_exact(q[:, s.q_begin:s.q_end], sub.k, sub.v, sub.ks, sub.vs, orc.KV_I8, s.nh, s.nkv, hd, hd, T,
                                  query_base_pos=T - 1, softmax_scale=0.2)
            err = float(np.abs(mine[0] - full[0, s.q_begin:s.q_end]).max())    # disjoint slices, no collective
        out_q.put((rank, err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["seq", "heads"])
def test_two_rank_shards_reproduce_full_attention(mode, oracle):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err in results:
        assert err < 1e-5, f"rank {rank}: {err}"
