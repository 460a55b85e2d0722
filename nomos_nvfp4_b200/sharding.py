"""Work partition of the attention path across the GPUs of one box (host-side arithmetic only).

The reference is single-GPU; these two partitions are the multi-GPU surface of this library.

* KV-head groups: rank g owns ``nkv/G`` KV heads (and their ``kvg`` query heads) of every
  sequence.  Outputs are disjoint slices of ``[nh, l_hd]``; no collective is needed.
* Sequence chunks (batch 1, long context): rank g owns a contiguous run of cached positions and
  produces un-normalised partials ``(o, m, l)`` per query head.  Either the partials are all-gathered
  by a collective library and merged by ``nomos_attn_merge_partials``, or -- ``SeqShardGroup`` -- every
  rank's attention kernel stores them into the peers' mailboxes itself and merges what arrives
  (``nomos_attn_seq_sharded``: one launch per rank and step).  Chunk boundaries fall on multiples of
  32 positions so every rank's kernel streams whole tiles.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class HeadShard:
    kv_begin: int
    kv_end: int
    q_begin: int
    q_end: int

    @property
    def nkv(self) -> int:
        return self.kv_end - self.kv_begin

    @property
    def nh(self) -> int:
        return self.q_end - self.q_begin


def head_group_shard(nkv: int, kvg: int, world: int, rank: int) -> HeadShard:
    """KV heads [kv_begin, kv_end) and query heads [q_begin, q_end) of `rank`."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if nkv % world:
        raise ValueError(f"{world} ranks do not divide {nkv} KV heads")
    per = nkv // world
    return HeadShard(rank * per, (rank + 1) * per, rank * per * kvg, (rank + 1) * per * kvg)


def sequence_shard(klen: int, world: int, rank: int, align: int = 32) -> tuple[int, int]:
    """(first position, number of positions) of `rank`'s chunk of a `klen`-key window.
    Chunks are aligned to `align` positions; trailing ranks may own nothing (length 0)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    tiles = -(-klen // align)
    per = -(-tiles // world)
    begin = min(klen, rank * per * align)
    end = min(klen, (rank + 1) * per * align)
    return begin, end - begin


class SeqShardGroup:
    """Mailboxes and step counter of one sequence-sharded decode group (one process per GPU).

    ``all_gather_bytes(b: bytes) -> list[bytes]`` exchanges a byte string between the ranks on the host, in rank
    order (e.g. ``torch.distributed.all_gather_object``); it is used once, to pass the mailbox handles round.
    Every rank must make every ``decode`` call: the step counter advances in lockstep."""

    def __init__(self, rank: int, world: int, rows: int, l_hd: int, all_gather_bytes, timeout_us: int = 0):
        from . import ops
        self._ops, self.rank, self.world, self.timeout_us = ops, rank, world, timeout_us
        self.step = 0
        self.mailbox_bytes = ops.attn_peer_mailbox_bytes(world, rows, l_hd)
        self.own, self.mailboxes = 0, []
        try:
            self.own, handle = ops.attn_peer_mailbox_create(self.mailbox_bytes)
            failure = None
        except Exception as e:                      # still take part in the exchange below: the peers are waiting in it
            handle, failure = b"", e
        handles = all_gather_bytes(handle)
        if failure is not None:
            raise failure
        if len(handles) != world or not all(handles):
            self.close()
            raise ValueError(f"expected {world} mailbox handles, got {sum(1 for h in handles if h)}")
        self.mailboxes = [0] * world
        self.mailboxes[rank] = self.own
        try:
            for g in range(world):
                if g != rank:
                    self.mailboxes[g] = ops.attn_peer_mailbox_open(handles[g])
        except Exception:
            self.close()
            raise

    def decode(self, stream, args) -> None:
        """Attention over this rank's chunk + exchange + merge; the final output lands in ``args.out`` on every rank."""
        self.step += 1
        peer = self._ops.make_peer(self.rank, self.world, self.mailboxes, self.mailbox_bytes, self.step, self.timeout_us)
        self._ops.attn_seq_sharded(stream, args, peer)

    def status(self, stream, clear: bool = False) -> int:
        return self._ops.attn_seq_sharded_status(stream, clear)

    def close(self) -> None:
        for g, m in enumerate(self.mailboxes):
            if m and g != self.rank:
                self._ops.attn_peer_mailbox_close(m, False)
        if self.own:
            self._ops.attn_peer_mailbox_close(self.own, True)
        self.own, self.mailboxes = 0, []
