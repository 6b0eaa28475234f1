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


def _layers_worker(rank, world, port, out):
    """Row-sharded two-layer forward / backward on `world` gloo ranks against the single-process
    result.  The product kernel is CUDA-only, so this test (and only this test) puts the CPU checker
    in its place; everything around it is the shipped code: RowShardedGraph, the all-gather of H
    and of dY, BCSRSPMMFunction / BCSRGraphConv, the summed weight gradients."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import scipy.sparse as sps
        import oracle
        from graph_rws_b200 import BCSRGraph, core
        from graph_rws_b200.helper.engine import _allreduce_grads
        from graph_rws_b200.layers import BCSRGraphConv
        from graph_rws_b200.parallel import RowShardedGraph, partition_windows_by_tiles, shard_bcsr

        def cpu_spmm(wo, cols, vals, dense, **kw):
            return torch.from_numpy(oracle.spmm_fwd(wo.numpy(), cols.numpy(), vals.float().numpy(),
                                                    dense.detach().float().numpy())).to(dense.dtype)
        core.spmm_raw = cpu_spmm

        n = 333                                        # last window is partial
        rng = np.random.default_rng(5)
        A = sps.random(n, n, density=0.03, random_state=7, format="csr", dtype=np.float32) + sps.eye(n, dtype=np.float32, format="csr")
        A = A.tocsr()
        A.sort_indices()

        def graph_of(m):
            wo, cols, vals = oracle.csr_to_bcsr(n, m.indptr.astype(np.int64), m.indices.astype(np.int32), m.data.astype(np.float32))
            return BCSRGraph(num_nodes=n, num_edges=None, tile_rows=16, tile_cols=8, window_offset=torch.from_numpy(wo),
                             original_col_indices=torch.from_numpy(cols), values_condensed=torch.from_numpy(vals),
                             device=torch.device("cpu"))
        At = A.T.tocsr()
        At.sort_indices()
        g, gt = graph_of(A), graph_of(At)
        g._shared[("T", n, torch.float32)] = (g._versions(), gt)            # the cached transposed graph

        torch.manual_seed(3)
        l1, l2 = BCSRGraphConv(24, 16), BCSRGraphConv(16, 5)
        for p in list(l1.parameters()) + list(l2.parameters()):
            dist.broadcast(p.data, 0)
        params = list(l1.parameters()) + list(l2.parameters())
        X = torch.from_numpy(rng.standard_normal((n, 24)).astype(np.float32))
        y = torch.from_numpy(rng.integers(0, 5, n))

        def forward(graph, x):
            h = torch.relu(l1(graph, x)[:x.shape[0]])
            return l2(graph, h)[:x.shape[0]]

        ref = forward(g, X)
        torch.nn.functional.cross_entropy(ref, y, reduction="sum").backward()
        ref_grads = [p.grad.clone() for p in params]
        for p in params:
            p.grad = None

        part = partition_windows_by_tiles(g.window_offset, world, num_rows=n)
        lo, hi = part.rows(rank)

        def shard(graph):
            wo, cols, vals = shard_bcsr(graph.window_offset, graph.original_col_indices, graph.values_condensed, part, rank)
            return BCSRGraph(num_nodes=hi - lo, num_edges=None, tile_rows=16, tile_cols=8, window_offset=wo,
                             original_col_indices=cols, values_condensed=vals, device=torch.device("cpu"),
                             num_rows=hi - lo, num_cols=n)
        sharded = RowShardedGraph(shard(g), part, rank, local_t=RowShardedGraph(shard(gt), part, rank))
        logits = forward(sharded, X[lo:hi].contiguous())
        assert logits.shape[0] == hi - lo
        assert torch.allclose(logits, ref[lo:hi], rtol=1e-4, atol=1e-5)
        torch.nn.functional.cross_entropy(logits, y[lo:hi], reduction="sum").backward()

        class _M:                                      # what _allreduce_grads needs of a module
            @staticmethod
            def parameters():
                return params
        _allreduce_grads(_M, average=False)
        for p, r in zip(params, ref_grads):
            assert torch.allclose(p.grad, r, rtol=1e-3, atol=1e-4), float((p.grad - r).abs().max())
        out[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_sharded_layers_match_the_single_process_result(world):
    ctx = mp.get_context("spawn")
    out = ctx.Array("i", world)
    port = _free_port()
    procs = [ctx.Process(target=_layers_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.kill()
            p.join()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(out) == [1] * world
