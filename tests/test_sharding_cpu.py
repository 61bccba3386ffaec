"""Expert / row placement for the multi-GPU grouped matmul: pure host logic, plus a two-process gloo run in
which every rank computes its shard (with the CPU oracle standing in for the kernel) and one all-gather
reassembles the full output."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from catlass_b200 import sharding  # noqa: E402
import problems as P  # noqa: E402


def _check_partition(sizes, shards):
    covered = [np.zeros(int(s), np.int32) for s in sizes]
    for sh in shards:
        for p in sh.pieces:
            assert p.rows > 0
            covered[p.expert][p.row_begin:p.row_begin + p.rows] += 1
    assert all((c == 1).all() for c in covered), "every row must be placed exactly once"


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("mode", ["whole", "split"])
def test_plan_partitions_all_rows(world, mode):
    sizes = P.zipf_group_sizes(131072, 64, seed=20240)
    shards = sharding.plan(sizes, world, mode=mode)
    assert len(shards) == world
    _check_partition(sizes, shards)
    loads = [s.rows for s in shards]
    assert sum(loads) == 131072
    if mode == "split":
        # what is balanced is the kernel's cost (256-row tiles per expert): every rank within one tile of the mean
        costs = [s.cost for s in shards]
        assert max(costs) <= sum(costs) / world + 1.0, costs
        for sh in shards:
            assert len(sh.pieces) == len(sh.local_groups())  # contiguous cuts: one piece per expert and rank
            for p in sh.pieces:
                assert p.row_begin % sharding.ROW_TILE == 0
        # an expert is replicated only where its rows are: whole experts plus at most two partial ones per rank
        for sh in shards:
            partial = [p for p in sh.pieces if p.rows != int(sizes[p.expert])]
            assert len(partial) <= 2
    else:
        assert max(loads) >= int(max(sizes))   # bounded by the hottest expert


def test_whole_expert_placement_is_capped_by_the_hot_expert():
    sizes = P.zipf_group_sizes(131072, 64, seed=20240)
    whole = max(s.cost for s in sharding.plan(sizes, 8, mode="whole"))
    split = max(s.cost for s in sharding.plan(sizes, 8, mode="split"))
    assert whole >= sharding.tile_cost(int(max(sizes))) and split < whole / 1.8
    # the top expert holds about a quarter of all rows: whole-expert speed-up cannot exceed ~4x
    assert 131072 / max(s.rows for s in sharding.plan(sizes, 8, mode="whole")) < 4.2


@pytest.mark.parametrize("world", [2, 4, 8])
def test_split_placement_balances_tiles_plus_a_cost_per_expert(world):
    """What is balanced is row tiles plus GROUP_COST per expert on the rank (an expert brings its own weights through
    HBM): the costs of the ranks stay within a tile and a half of each other, and the rank that gets the tail of small
    experts holds fewer rows than the rank that gets the hot expert."""
    sizes = P.zipf_group_sizes(131072, 64, seed=20240)
    shards = sharding.plan(sizes, world, mode="split")
    costs = [sh.cost for sh in shards]
    assert max(costs) - min(costs) <= 1.5 + sharding.GROUP_COST
    for sh in shards:
        want = sum(sharding.tile_cost(r) + sharding.GROUP_COST for _, r in sh.local_groups())
        assert abs(sh.cost - want) < 1e-9
    experts = [len(sh.local_groups()) for sh in shards]
    assert experts[-1] > experts[0] and shards[-1].rows < shards[0].rows


def test_local_groups_merge_pieces_of_one_expert():
    shards = sharding.plan([1000, 10, 0, 300], 2, mode="split", chunk_rows=256)
    _check_partition([1000, 10, 0, 300], shards)
    for sh in shards:
        experts = [e for e, _ in sh.local_groups()]
        assert experts == sorted(set(experts))
        assert sum(r for _, r in sh.local_groups()) == sh.rows


def test_tile_constants_mirror_the_kernel():
    import re
    text = open(os.path.join(ROOT, "catlass_b200", "csrc", "w8a8_gemm_pair.cuh")).read()
    val = lambda name: int(re.search(r"constexpr int " + name + r" = (\d+);", text).group(1))  # noqa: E731
    assert val("kPairTileM") == sharding.ROW_TILE
    assert sharding.tile_cost(512) == 2.0 and sharding.tile_cost(513) == 3.0 and sharding.tile_cost(0) == 0.0


def test_edge_cases():
    assert [s.rows for s in sharding.plan([0, 0], 2)] == [0, 0]
    with pytest.raises(ValueError):
        sharding.plan([1], 0)
    with pytest.raises(ValueError):
        sharding.plan([-1], 1)
    with pytest.raises(ValueError):
        sharding.plan([10], 2, mode="split", chunk_rows=100)


def _worker(rank, world, port, tmpdir):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sizes = [300, 0, 40, 700, 5, 129]
        n, k = 48, 64
        a, b, scale, pt, gl = P.w8a8_grouped(sizes, n, k, seed=17)   # every rank generates the same problem
        m = a.shape[0]
        shards = sharding.plan(sizes, world, mode="split")
        mine = shards[rank]
        ranges = sharding.global_row_ranges(sizes, mine)
        rows = np.concatenate([np.arange(s, s + c) for s, c in ranges]) if ranges else np.zeros(0, np.int64)
        groups = mine.local_groups()
        local_gl = np.cumsum([r for _, r in groups]).astype(np.int64)
        experts = [e for e, _ in groups]
        out_local = np.zeros((len(rows), n), np.float32)
        if len(rows):
            out_local = O.grouped_quant_matmul(a[rows], b[experts], local_gl, scale[experts], pt[rows], len(rows),
                                               n, k, O.ROW_MAJOR)
        # one all-gather assembles the output (padded to the largest shard)
        cap = max(s.rows for s in shards)
        buf = torch.zeros((cap, n))
        buf[:len(rows)] = torch.from_numpy(out_local)
        idx = torch.full((cap,), -1, dtype=torch.int64)
        idx[:len(rows)] = torch.from_numpy(rows)
        outs = [torch.zeros_like(buf) for _ in range(world)]
        idxs = [torch.zeros_like(idx) for _ in range(world)]
        dist.all_gather(outs, buf)
        dist.all_gather(idxs, idx)
        full = np.zeros((m, n), np.float32)
        for o, i in zip(outs, idxs):
            sel = i >= 0
            full[i[sel].numpy()] = o[sel].numpy()
        want = O.grouped_quant_matmul(a, b, gl, scale, pt, m, n, k, O.ROW_MAJOR)
        ok = np.array_equal(full.view(np.uint32), want.view(np.uint32))
        open(os.path.join(tmpdir, f"rank{rank}.txt"), "w").write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo_shards_reassemble_to_the_full_result(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [open(tmp_path / f"rank{r}.txt").read() for r in range(2)] == ["ok", "ok"]
