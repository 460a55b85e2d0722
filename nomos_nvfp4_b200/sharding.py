"""Work partition of the attention path across the GPUs of one box (host-side arithmetic only).

The reference is single-GPU; these two partitions are the multi-GPU surface of this library.

* KV-head groups: rank g owns ``nkv/G`` KV heads (and their ``kvg`` query heads) of every
  sequence.  Outputs are disjoint slices of ``[nh, l_hd]``; no collective is needed.
* Sequence chunks (batch 1, long context): rank g owns a contiguous run of cached positions and
  produces un-normalised partials ``(o, m, l)`` per query head; the partials are all-gathered and
  merged (``nomos_attn_merge_partials``).  Chunk boundaries fall on multiples of 32 positions so
  every rank's kernel streams whole tiles.
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
