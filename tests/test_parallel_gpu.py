"""Row-partitioned SpMM and sharded-feature exchange on two GPUs over NCCL (skipped with fewer)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from graph_rws_b200 import BCSRGraph, core
        from graph_rws_b200.data import synthetic
        from graph_rws_b200.parallel import DistributedSpMM, exchange_rows, partition_windows_by_tiles
        g = synthetic.sym_normalized_csr(9000, *synthetic.chung_lu_edges(9000, 120000, 2.2, 13))
        graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev, values_dtype=torch.float16)
        H = torch.randn(g.num_nodes, 128, generator=torch.Generator().manual_seed(4)).half().to(dev)
        full = core.spmm_raw(graph.window_offset, graph.original_col_indices, graph.values_condensed, H)[:g.num_nodes]
        part = partition_windows_by_tiles(graph.window_offset, world, num_rows=g.num_nodes)
        lo, hi = part.rows(rank)
        local = DistributedSpMM(graph, part, rank)(H[lo:hi].contiguous())
        # the shard cuts its tile array at other places than the full graph does, so windows that
        # are split between CTAs are summed in other groupings: equal up to fp32 rounding and the
        # final fp16 rounding
        err = (local.float() - full[lo:hi].float()).norm() / full[lo:hi].float().norm()
        assert err < 1e-3, float(err)
        # feature rows sharded in contiguous blocks, fetched by global id with all_to_all_single
        per = (g.num_nodes + world - 1) // world
        ids = torch.randint(0, g.num_nodes, (5000,), generator=torch.Generator().manual_seed(rank)).int().to(dev)
        rows = exchange_rows(H[rank * per:(rank + 1) * per].contiguous(), ids, g.num_nodes)
        assert torch.equal(rows, H[ids.long()])
        torch.cuda.synchronize()
        out[rank] = 1
    finally:
        dist.destroy_process_group()


def test_row_partitioned_spmm_and_row_exchange_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Array("i", world)
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(out) == [1] * world
