"""Placement of a grouped (MoE) matmul over several GPUs.

Groups (experts) and rows inside a group are independent, so the problem shards with no exchange step:
each rank receives whole experts, or row slices of a hot expert together with a replica of that expert's
weights, and computes its own rows.  Nothing here runs on the GPU; it only decides who computes what.

Two placements are offered:
  "whole"  every expert lives on exactly one rank (speed-up limited by the largest expert); longest-processing-
           time-first bin packing on the tile cost,
  "split"  the experts' row tiles are laid on a line, expert after expert, and the line is cut into world_size
           contiguous stretches of equal cost: a rank holds whole experts plus at most two partial ones, cuts fall
           on multiples of the kernel's 256-row tile, and an expert's weights are replicated only on the ranks
           its rows span (a hot expert with a quarter of all rows spans three of eight ranks).
What is balanced is the kernel's cost, not the row count: the grouped kernel works in 256-row tiles per expert,
so an expert costs its full tiles plus one for a partial tile, plus a constant per expert present on the rank
(every expert brings 29 MB of weights of its own through HBM and L2; a rank that holds thirty small experts
is slower than one that holds two large ones with the same number of tiles).
"""
from dataclasses import dataclass
from typing import List

# Mirror of the grouped kernel's row tile (kPairTileM in catlass_b200/csrc/w8a8_gemm_pair.cuh; a test compares them):
# shard cuts fall on its multiples.
ROW_TILE = 256


# Cost of one more expert on a rank, in row tiles.  Measured on one B200 with 64 row tiles of K = 7168, N = 4096 cut
# into 1, 16, 32 and 64 experts (306, 336, 359, 395 us per launch): 4.76 us per row tile + 1.4 us per expert.
GROUP_COST = 0.3


def tile_cost(rows):
    """Cost of `rows` rows of one expert on one rank, in 256-row tiles: a partial tile costs a full one (a
    narrower tensor-core shape for it was measured and did not pay: the MMA issue rate, not the math, bounds it)."""
    return float((int(rows) + ROW_TILE - 1) // ROW_TILE)


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

    @property
    def cost(self):
        """Kernel cost of this rank's launch in full tiles (pieces of one expert form one group)."""
        return sum(tile_cost(r) + GROUP_COST for _, r in self.local_groups())

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
    """Returns one RankShard per rank. group_sizes: rows per expert. Every row is placed exactly once.
    chunk_rows (split mode): granularity of the cuts, a multiple of ROW_TILE (default: ROW_TILE)."""
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    if mode not in ("whole", "split"):
        raise ValueError("mode must be 'whole' or 'split'")
    sizes = [int(s) for s in group_sizes]
    if any(s < 0 for s in sizes):
        raise ValueError("negative group size")
    if chunk_rows is None:
        chunk_rows = ROW_TILE
    if chunk_rows <= 0 or chunk_rows % ROW_TILE:
        raise ValueError(f"chunk_rows must be a multiple of the {ROW_TILE}-row tile")
    bins: List[List[Piece]] = [[] for _ in range(world_size)]
    if mode == "whole" or world_size == 1:
        loads = [0.0] * world_size
        units = [Piece(e, 0, s) for e, s in enumerate(sizes) if s > 0]
        for u in sorted(units, key=lambda p: (-p.rows, p.expert)):
            r = min(range(world_size), key=lambda i: (loads[i], i))
            bins[r].append(u)
            loads[r] += tile_cost(u.rows) + GROUP_COST
    else:
        # units of chunk_rows rows in expert order, each with the cost it adds to its expert
        units = []
        for e, s in enumerate(sizes):
            r = 0
            while r < s:
                take = min(chunk_rows, s - r)
                units.append((Piece(e, r, take), tile_cost(take) + (GROUP_COST if r == 0 else 0.0)))
                r += take
        total = sum(c for _, c in units)
        done = 0.0
        for piece, c in units:
            # the unit goes to the rank whose equal share of the line holds the unit's midpoint
            r = min(world_size - 1, int((done + 0.5 * c) * world_size / total)) if total > 0 else 0
            bins[r].append(piece)
            done += c
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
