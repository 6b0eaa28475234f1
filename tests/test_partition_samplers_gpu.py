"""Partition-based batches (BCSRSampler.sample_partitions / repack_subgraph / sample_dps_online)
against dense algebra: the sub-BCSR a batch carries multiplies like the matching rows and columns
of the full adjacency."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup():
    from graph_rws_b200 import BCSRGraph
    from graph_rws_b200.data import synthetic
    g = synthetic.sym_normalized_csr(2000, *synthetic.chung_lu_edges(2000, 14000, 2.4, 41))
    dev = torch.device("cuda")
    graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev)
    A = torch.zeros(g.num_nodes, g.num_nodes, dtype=torch.float64)
    rows = np.repeat(np.arange(g.num_nodes), np.diff(g.row_ptr))
    A[torch.from_numpy(rows), torch.from_numpy(g.col_idx.astype(np.int64))] = torch.from_numpy(g.values).double()
    X = torch.randn(g.num_nodes, 24, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    return g, graph, A.to(dev), X.to(dev)


def _spmm(sub, dense):
    from graph_rws_b200 import core
    return core.spmm_raw(sub.window_offset, sub.original_col_indices, sub.values_condensed, dense.float().contiguous()).double()


def test_sample_partitions_is_the_induced_subgraph(setup):
    from graph_rws_b200.sampler import BCSRSampler
    g, graph, A, X = setup
    book = [dict(start_idx=s, end_idx=min(s + 400, 2000)) for s in range(0, 2000, 400)]      # window-aligned ranges
    sampler = BCSRSampler([5, 5], partition_book=book, verbose=False)
    pids = torch.tensor([3, 1], device="cuda")
    sub = sampler.sample_partitions(graph, pids)
    nodes = torch.cat([torch.arange(1200, 1600), torch.arange(400, 800)]).cuda()
    assert sub.num_rows == sub.num_cols == 800 and sub.is_local_input
    assert torch.equal(sub.active_windows, torch.arange(50, dtype=torch.int32, device="cuda"))
    got = _spmm(sub, X[nodes])[:800]
    want = A[nodes][:, nodes] @ X[nodes]
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-3)
    # edges that leave the selection keep no column
    c = sub.original_col_indices
    assert int(c.max()) < 800 and bool((c >= -1).all())


def test_repack_subgraph_with_and_without_the_halo_budget(setup):
    from graph_rws_b200.sampler import BCSRSampler
    g, graph, A, X = setup
    sampler = BCSRSampler([5, 5], verbose=False)
    wins = torch.tensor([70, 3, 19, 44, 3 + 100], device="cuda")
    sub = sampler.repack_subgraph(graph, wins, max_external_ratio=1e9)
    ws = torch.sort(wins).values
    internal = (ws[:, None] * 16 + torch.arange(16, device="cuda")[None, :]).reshape(-1)
    assert sub.num_internal_nodes == internal.numel() and torch.equal(sub.original_node_ids[:internal.numel()], internal)
    assert torch.equal(sub.original_window_ids, ws) and sub.is_local_input
    halo = sub.original_node_ids[internal.numel():]
    assert bool((halo[1:] > halo[:-1]).all()) and not bool(torch.isin(halo, internal).any())
    got = _spmm(sub, X[sub.original_node_ids])[:internal.numel()]
    assert torch.allclose(got, (A @ X)[internal], rtol=2e-2, atol=2e-3)            # every neighbour kept: the full rows
    # the inner graph keeps only the edges among the internal nodes
    got_in = _spmm(sub.inner_graph, X[internal])[:internal.numel()]
    assert torch.allclose(got_in, A[internal][:, internal] @ X[internal], rtol=2e-2, atol=2e-3)
    # a tight budget drops halo nodes, never internal ones, and the product matches the kept columns
    small = sampler.repack_subgraph(graph, wins, max_external_ratio=0.5)
    assert small.original_node_ids.numel() == internal.numel() + int(internal.numel() * 0.5)
    kept = small.original_node_ids
    got_small = _spmm(small, X[kept])[:internal.numel()]
    assert torch.allclose(got_small, A[internal][:, kept] @ X[kept], rtol=2e-2, atol=2e-3)
    stub = sampler.repack_subgraph(graph, wins, dry_run=True)
    assert stub.total_tiles == int(sub.window_offset[-1]) and stub.num_internal_nodes == 80


def test_sample_dps_online_covers_the_sampled_hops(setup):
    from graph_rws_b200.sampler import BCSRSampler
    g, graph, A, X = setup
    sampler = BCSRSampler([5, 5], verbose=False, seed=3)
    seed_windows = torch.tensor([5, 60], device="cuda")
    sub = sampler.sample_dps_online(graph, seed_windows, fanouts=[4, 3])
    assert bool(torch.isin(seed_windows, sub.original_window_ids).all())
    blocks = BCSRSampler([4, 3], verbose=False, seed=3).sample_layers(
        graph, (seed_windows[:, None] * 16 + torch.arange(16, device="cuda")[None, :]).reshape(-1))
    reached = blocks[0].input_nodes
    assert bool(torch.isin(torch.div(reached[reached >= 0], 16, rounding_mode="floor"), sub.original_window_ids).all())
    got = _spmm(sub, X[sub.original_node_ids])[:sub.num_internal_nodes]
    rows = sub.original_node_ids[:sub.num_internal_nodes]
    assert torch.allclose(got, A[rows][:, sub.original_node_ids] @ X[sub.original_node_ids], rtol=2e-2, atol=2e-3)
