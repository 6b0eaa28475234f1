"""The reference's on-disk BCSR cache (four files per graph) read and written by this package."""
import os

import numpy as np
import pytest
import torch

from conftest import golden_cases, load_case


def _write_like_reference(c, cache_path):
    """What data/data_loader.py:323-352 leaves on disk for a converted graph."""
    from graph_rws_b200.data import bcsr_bin_paths
    meta_path, off_path, col_path, val_path = bcsr_bin_paths(cache_path)
    c["window_offset"].astype(np.int64).tofile(off_path)
    c["cols"].astype(np.int32).tofile(col_path)
    c["vals"].astype(np.float32).tofile(val_path)
    n = int(c["num_rows"]) if "num_rows" in c else (len(c["window_offset"]) - 1) * 16
    torch.save({'num_nodes': n, 'num_edges': int(np.count_nonzero(c["vals"])), 'num_rows': n, 'num_cols': n,
                'tile_rows': 16, 'tile_cols': 8, 'num_windows': len(c["window_offset"]) - 1,
                'window_offset_len': len(c["window_offset"]), 'col_indices_len': len(c["cols"]),
                'values_len': len(c["vals"])}, meta_path)
    return n


@pytest.mark.parametrize("path", golden_cases()[:3], ids=lambda p: os.path.basename(p)[5:-4])
def test_reads_a_cache_written_in_the_reference_layout(tmp_path, path):
    from graph_rws_b200.data import load_bcsr_bins
    c = load_case(path)
    if len(c["cols"]) == 0:
        pytest.skip("the reference treats an empty array as a missing cache")
    cache = str(tmp_path / "graph.pt")
    n = _write_like_reference(c, cache)
    g = load_bcsr_bins(cache, device='cpu')
    assert g is not None and g.num_nodes == n and g.tile_rows == 16 and g.tile_cols == 8
    assert np.array_equal(g.window_offset.numpy(), c["window_offset"])
    assert np.array_equal(g.original_col_indices.numpy(), c["cols"])
    assert np.array_equal(g.values_condensed.numpy(), c["vals"].astype(np.float32))


def test_round_trip_and_rejected_caches(tmp_path):
    from graph_rws_b200.data import BCSRGraph, bcsr_bin_paths, load_bcsr_bins, save_bcsr_bins
    c = load_case(golden_cases()[-1])
    W = len(c["window_offset"]) - 1
    g = BCSRGraph(num_nodes=W * 16, num_edges=None, tile_rows=16, tile_cols=8,
                  window_offset=torch.from_numpy(c["window_offset"]), original_col_indices=torch.from_numpy(c["cols"]),
                  values_condensed=torch.from_numpy(c["vals"]).half(), device=torch.device('cpu'),
                  values_dtype=torch.float16)
    cache = str(tmp_path / "g.pt")
    assert save_bcsr_bins(g, cache)
    meta = torch.load(bcsr_bin_paths(cache)[0], weights_only=False)
    assert set(meta) == {'num_nodes', 'num_edges', 'num_rows', 'num_cols', 'tile_rows', 'tile_cols', 'num_windows',
                         'window_offset_len', 'col_indices_len', 'values_len'}
    assert os.path.getsize(bcsr_bin_paths(cache)[3]) == 4 * g.values_condensed.numel()      # fp32 on disk
    back = load_bcsr_bins(cache, device='cpu', values_dtype=torch.float16)
    assert torch.equal(back.window_offset, g.window_offset)
    assert torch.equal(back.original_col_indices, g.original_col_indices)
    assert torch.equal(back.values_condensed, g.values_condensed)
    assert back.num_edges == g.num_edges
    # a truncated value file or a missing file is not a cache
    with open(bcsr_bin_paths(cache)[3], 'r+b') as f:
        f.truncate(8)
    assert load_bcsr_bins(cache, device='cpu') is None
    os.remove(bcsr_bin_paths(cache)[1])
    assert load_bcsr_bins(cache, device='cpu') is None


@pytest.mark.gpu
def test_loads_to_the_gpu_in_half_precision_and_multiplies(tmp_path, oracle):
    from graph_rws_b200 import BCSRGraph, core
    from graph_rws_b200.data import load_bcsr_bins, save_bcsr_bins, synthetic
    from gpu_util import check_spmm_tolerance
    g = synthetic.sym_normalized_csr(5000, *synthetic.chung_lu_edges(5000, 60000, 2.3, 31))
    dev = torch.device("cuda")
    graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev)
    cache = str(tmp_path / "g.pt")
    save_bcsr_bins(graph, cache)
    back = load_bcsr_bins(cache, device=dev, values_dtype=torch.float16)
    assert back.values_condensed.dtype == torch.float16 and back.values_condensed.is_cuda
    assert torch.equal(back.original_col_indices, graph.original_col_indices)
    assert torch.equal(back.values_condensed, graph.values_condensed.half())
    H = torch.randn(g.num_nodes, 128, generator=torch.Generator().manual_seed(2)).half()
    C = core.spmm_raw(back.window_offset, back.original_col_indices, back.values_condensed, H.to(dev), check=True)
    ref = oracle.spmm_fwd(back.window_offset.cpu().numpy(), back.original_col_indices.cpu().numpy(),
                          back.values_condensed.float().cpu().numpy(), H.float().numpy())
    check_spmm_tolerance(C.float().cpu().numpy(), ref, None, "loaded cache")
