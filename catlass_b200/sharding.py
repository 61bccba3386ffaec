"""Placement of a grouped (MoE) matmul over several GPUs.

Groups (experts) and rows inside a group are independent, so the problem shards with no exchange step:
each rank receives whole experts, or row slices of a hot expert together with a replica of that expert's
weights, and computes its own rows.  Nothing here runs on the GPU; it only decides who computes what.

Two placements are offered:
  "whole"  every expert lives on exactly one rank (speed-up limited by the largest expert),
  "split"  experts larger than a chunk are cut into row chunks (multiples of the 128-row tile) that are
           placed independently; weights of a cut expert are replicated on the ranks that hold a chunk.
Both use longest-processing-time-first bin packing on the row counts.
"""
from dataclasses import dataclass
from typing import List

ROW_TILE = 128


@dataclass(frozen=True)
class Piece:
    expert: int      # index into the global expert list
    row_begin: int   # first row inside the expert's row block
    rows: int


@dataclass
class RankShard:
    rank: int
    pieces: List[Piece]          # sorted by (expert, row_begin)

    @property
    def rows(self):
        return sum(p.rows for p in self.pieces)

    def group_list(self):
        """Local prefix sums, one entry per piece (the group list of the rank's own grouped matmul)."""
        out, total = [], 0
        for p in self.pieces:
            total += p.rows
            out.append(total)
        return out

    def experts(self):
        """Expert index of each piece."""
        return [p.expert for p in self.pieces]

    def local_groups(self):
        """[(expert, rows)]: one local group per distinct expert on this rank.  Rows are independent, so
        all pieces of one expert are computed as a single group against one copy of its weights."""
        out = []
        for p in self.pieces:
            if out and out[-1][0] == p.expert:
                out[-1] = (p.expert, out[-1][1] + p.rows)
            else:
                out.append((p.expert, p.rows))
        return out


def plan(group_sizes, world_size, mode="split", chunk_rows=None):
    """Returns one RankShard per rank. group_sizes: rows per expert. Every row is placed exactly once."""
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    if mode not in ("whole", "split"):
        raise ValueError("mode must be 'whole' or 'split'")
    sizes = [int(s) for s in group_sizes]
    if any(s < 0 for s in sizes):
        raise ValueError("negative group size")
    total = sum(sizes)
    units: List[Piece] = []
    if mode == "whole" or world_size == 1:
        units = [Piece(e, 0, s) for e, s in enumerate(sizes) if s > 0]
    else:
        if chunk_rows is None:
            # small enough that the packing error is a few percent of a rank's load
            target = max(total // (world_size * 16), ROW_TILE)
            chunk_rows = max(ROW_TILE, (target // ROW_TILE) * ROW_TILE)
        if chunk_rows % ROW_TILE:
            raise ValueError("chunk_rows must be a multiple of the 128-row tile")
        for e, s in enumerate(sizes):
            r = 0
            while r < s:
                take = min(chunk_rows, s - r)
                units.append(Piece(e, r, take))
                r += take
    loads = [0] * world_size
    bins: List[List[Piece]] = [[] for _ in range(world_size)]
    for u in sorted(units, key=lambda p: (-p.rows, p.expert, p.row_begin)):
        r = min(range(world_size), key=lambda i: (loads[i], i))
        bins[r].append(u)
        loads[r] += u.rows
    shards = []
    for r in range(world_size):
        pieces = sorted(bins[r], key=lambda p: (p.expert, p.row_begin))
        # adjacent chunks of one expert on one rank form a single local group again
        merged: List[Piece] = []
        for p in pieces:
            if merged and merged[-1].expert == p.expert and merged[-1].row_begin + merged[-1].rows == p.row_begin:
                last = merged.pop()
                merged.append(Piece(last.expert, last.row_begin, last.rows + p.rows))
            else:
                merged.append(p)
        shards.append(RankShard(r, merged))
    return shards


def global_row_ranges(group_sizes, shard):
    """(global_row_begin, rows) of each piece of `shard` in the expert-contiguous global row order."""
    starts, total = [], 0
    for s in group_sizes:
        starts.append(total)
        total += int(s)
    return [(starts[p.expert] + p.row_begin, p.rows) for p in shard.pieces]
