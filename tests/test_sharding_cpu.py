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


class _FakeMailboxOps:
    """Stand-in for the mailbox calls of the library: records what a SeqShardGroup does with them."""

    def __init__(self, fail_create=False, fail_open_of=None):
        self.fail_create, self.fail_open_of = fail_create, fail_open_of
        self.closed, self.opened = [], []

    def attn_peer_mailbox_bytes(self, world, rows, l_hd):
        return world * (rows * (l_hd + 2) * 4 + 256)

    def attn_peer_mailbox_create(self, nbytes):
        if self.fail_create:
            raise RuntimeError("no memory for the mailbox")
        return 0x1000, b"handle-of-this-rank"

    def attn_peer_mailbox_open(self, handle):
        if handle == self.fail_open_of:
            raise RuntimeError("no peer access")
        self.opened.append(handle)
        return 0x2000 + len(self.opened)

    def attn_peer_mailbox_close(self, ptr, own):
        self.closed.append((ptr, own))


def _group_with(monkeypatch, fake, rank, world, gathered):
    import nomos_nvfp4_b200.ops as ops
    from nomos_nvfp4_b200.sharding import SeqShardGroup
    for name in ("attn_peer_mailbox_bytes", "attn_peer_mailbox_create", "attn_peer_mailbox_open", "attn_peer_mailbox_close"):
        monkeypatch.setattr(ops, name, getattr(fake, name))
    calls = []

    def all_gather_bytes(b):
        calls.append(b)
        return [b if g == rank else h for g, h in enumerate(gathered)]

    return SeqShardGroup, all_gather_bytes, calls


def test_seq_shard_group_opens_every_peer_and_closes_them(monkeypatch):
    fake = _FakeMailboxOps()
    cls, agb, calls = _group_with(monkeypatch, fake, 1, 3, [b"h0", None, b"h2"])
    g = cls(1, 3, 32, 128, agb)
    assert calls == [b"handle-of-this-rank"]
    assert g.mailboxes[1] == 0x1000 and fake.opened == [b"h0", b"h2"]
    g.close()
    assert sorted(fake.closed) == sorted([(0x2001, False), (0x2002, False), (0x1000, True)])
    g.close()                                               # idempotent
    assert len(fake.closed) == 3


def test_seq_shard_group_takes_part_in_the_handle_exchange_when_its_own_mailbox_fails(monkeypatch):
    """A rank whose mailbox cannot be created must still enter the host exchange (its peers are blocked in it)
    and every rank must then see the missing handle and give up, instead of one of them waiting for ever."""
    fake = _FakeMailboxOps(fail_create=True)
    cls, agb, calls = _group_with(monkeypatch, fake, 0, 2, [None, b"h1"])
    with pytest.raises(RuntimeError, match="no memory"):
        cls(0, 2, 32, 128, agb)
    assert calls == [b""]
    # the peer of that rank: it receives an empty handle
    fake2 = _FakeMailboxOps()
    cls, agb, calls = _group_with(monkeypatch, fake2, 1, 2, [b"", None])
    with pytest.raises(ValueError, match="mailbox handles"):
        cls(1, 2, 32, 128, agb)
    assert fake2.closed == [(0x1000, True)]


def test_seq_shard_group_releases_what_it_opened_when_a_peer_cannot_be_mapped(monkeypatch):
    fake = _FakeMailboxOps(fail_open_of=b"h2")
    cls, agb, _ = _group_with(monkeypatch, fake, 0, 3, [None, b"h1", b"h2"])
    with pytest.raises(RuntimeError, match="no peer access"):
        cls(0, 3, 32, 128, agb)
    assert sorted(fake.closed) == sorted([(0x2001, False), (0x1000, True)])
