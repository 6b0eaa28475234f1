"""Host logic of the multi-GPU paths, run as world_size-2 gloo ranks on CPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import GOLDEN, load_case


def test_partition_by_tiles_is_balanced_and_complete():
    from graph_rws_b200.parallel import partition_windows_by_tiles
    rng = np.random.default_rng(0)
    tiles = np.concatenate([rng.integers(0, 40, 500), [4000, 0, 0, 3000], rng.integers(0, 40, 300)])
    wo = torch.from_numpy(np.concatenate([[0], np.cumsum(tiles)]).astype(np.int64))
    for world in (1, 2, 3, 4, 8):
        part = partition_windows_by_tiles(wo, world)
        assert part.window_bounds[0] == 0 and part.window_bounds[-1] == tiles.size
        assert all(a <= b for a, b in zip(part.window_bounds, part.window_bounds[1:]))
        loads = [int(wo[hi] - wo[lo]) for lo, hi in (part.windows(r) for r in range(world))]
        assert sum(loads) == int(wo[-1])
        assert max(loads) <= int(wo[-1]) / world + tiles.max()      # within one window of the ideal share


def test_sharded_graph_reproduces_the_full_product(oracle):
    from graph_rws_b200.parallel import partition_windows_by_tiles, shard_bcsr
    c = load_case(os.path.join(GOLDEN, "bcsr_chunglu_600.npz"))
    wo, cols, vals = (torch.from_numpy(c[k]) for k in ("window_offset", "cols", "vals"))
    B = np.random.default_rng(1).standard_normal((600, 16)).astype(np.float32)
    full = oracle.spmm_fwd(c["window_offset"], c["cols"], c["vals"], B)
    part = partition_windows_by_tiles(wo, 3, num_rows=600)
    pieces = []
    for r in range(3):
        w, cc, vv = shard_bcsr(wo, cols, vals, part, r)
        assert int(w[0]) == 0 and int(w[-1]) * 8 == cc.numel()
        pieces.append(oracle.spmm_fwd(w.numpy(), cc.numpy(), vv.numpy(), B))
    assert np.array_equal(np.concatenate(pieces), full)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from graph_rws_b200.parallel import (all_gather_rows, exchange_rows, partition_windows_by_tiles, shard_seeds)
        # uneven row shards are gathered into the full matrix
        wo = torch.tensor([0, 5, 5, 9, 30, 31, 40, 41], dtype=torch.int64)
        part = partition_windows_by_tiles(wo, world, num_rows=7 * 16 - 3)
        full = torch.arange(part.num_rows * 3, dtype=torch.float32).view(-1, 3)
        lo, hi = part.rows(rank)
        got = all_gather_rows(full[lo:hi].clone(), part)
        assert torch.equal(got, full)
        # sharded feature rows are fetched by global id
        n = 101
        per = (n + world - 1) // world
        x = torch.arange(n * 4, dtype=torch.float32).view(n, 4)
        x_local = x[rank * per:(rank + 1) * per].clone()
        ids = torch.tensor([100, 3, 50, 51, 0, 99, 3], dtype=torch.int32) if rank == 0 else torch.tensor([7, 60], dtype=torch.int32)
        rows = exchange_rows(x_local, ids, n)
        assert torch.equal(rows, x[ids.long()])
        # seeds split without loss
        seeds = torch.arange(11)
        mine = shard_seeds(seeds, rank, world)
        sizes = [torch.zeros(1, dtype=torch.long) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([mine.numel()]))
        assert sum(int(s) for s in sizes) == 11
        out[rank] = 1
    finally:
        dist.destroy_process_group()


def test_collectives_with_two_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Array("i", world)
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(out) == [1] * world
