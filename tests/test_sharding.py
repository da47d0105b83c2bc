"""Host-side unit partitioning, including a two-process gloo run on CPU (the N > 1 path has no
data-path collective; the processes only agree on who owns which units)."""
import os
import socket
import sys

import pytest
import torch.multiprocessing as mp

from conftest import ROOT, load_package


def test_partition_covers_and_balances():
    sh = load_package().sharding
    for units in (0, 1, 7, 8, 256, 1000):
        for world in (1, 2, 3, 4, 8):
            ranges = [sh.partition(units, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == units
            for (a, b), (c, d) in zip(ranges, ranges[1:]):
                assert b == c
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sh.partition(4, 2, 2)


def test_partition_alive_skips_unavailable_ranks():
    sh = load_package().sharding
    assert sh.partition_alive(8, [0, 1, 3], 2) == (0, 0)
    got = [sh.partition_alive(8, [0, 1, 3], r) for r in (0, 1, 3)]
    assert got[0][0] == 0 and got[-1][1] == 8 and sum(b - a for a, b in got) == 8
    with pytest.raises(ValueError):
        sh.partition_alive(8, [], 0)


def test_groupnorm_pieces_split_by_image_then_by_group():
    sh = load_package().sharding
    # batch 8 over 8/4/2 ranks: whole images
    for world in (1, 2, 4, 8):
        seen = []
        for r in range(world):
            calls = sh.merge_whole_images(sh.groupnorm_pieces(8, 32, world, r), 32)
            assert len(calls) == 1 and calls[0][2:] == (0, 32) and calls[0][1] == 8 // world
            seen += list(range(calls[0][0], calls[0][0] + calls[0][1]))
        assert seen == list(range(8))
    # batch 2 over 8 ranks: quarter images (8 groups each)
    pieces = [sh.groupnorm_pieces(2, 32, 8, r) for r in range(8)]
    assert all(len(p) == 1 and p[0].ng == 8 for p in pieces)
    assert [(p[0].image, p[0].g0) for p in pieces] == [(i // 4, 8 * (i % 4)) for i in range(8)]
    # ragged: 3 images x 5 groups over 4 ranks straddles images
    slabs = []
    for r in range(4):
        for p in sh.groupnorm_pieces(3, 5, 4, r):
            slabs += [(p.image, g) for g in range(p.g0, p.g0 + p.ng)]
    assert slabs == [(i, g) for i in range(3) for g in range(5)]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, root: str, out):
    import torch.distributed as dist
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    from conftest import load_package as lp
    sh = lp().sharding
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    mine = [(p.image, p.g0, p.ng) for p in sh.groupnorm_pieces(8, 32, world, rank)]
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    # the timing reduction bench.py performs: max over ranks
    import torch
    t = torch.tensor([1.0 + rank])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    if rank == 0:
        out.put((gathered, float(t.item())))
    dist.destroy_process_group()


def test_two_gloo_ranks_agree_on_a_disjoint_cover():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ROOT, out)) for r in range(2)]
    for p in procs:
        p.start()
    gathered, tmax = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    slabs = [(img, g) for rank_pieces in gathered for (img, g0, ng) in rank_pieces
             for g in range(g0, g0 + ng)]
    assert slabs == [(i, g) for i in range(8) for g in range(32)]
    assert tmax == 2.0
