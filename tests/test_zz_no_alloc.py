"""The allocation-free SpMM entry point (grws_spmm_fwd_static) against the regular one.

Some callers of the library cannot hand it device scratch or allocate any: they run inside another
framework's memory pool, or their device memory was frozen at start-up.  For them the kernel's
scratch lives in a fixed array inside the library.  This test calls the entry point through the
C ABI twice in a row (the array keeps the first call's contents, so the second call shows that
nothing stale leaks into a result) and compares with grws_spmm_fwd on the same inputs.  The file
name makes pytest collect it last.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

F16, BF16 = 1, 2


def _graph(seed, nodes, edges):
    from graph_rws_b200 import BCSRGraph
    from graph_rws_b200.data import synthetic
    g = synthetic.sym_normalized_csr(nodes, *synthetic.chung_lu_edges(nodes, edges, 2.2, seed))
    return BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=torch.device("cuda"),
                              values_dtype=torch.float16)


def _call_static(lib, graph, B, C):
    W, (K, N) = graph.num_windows, B.shape
    T = graph.original_col_indices.numel() // 8
    return lib.grws_spmm_fwd_static(graph.window_offset.data_ptr(), graph.original_col_indices.data_ptr(),
                                    graph.values_condensed.data_ptr(), F16, B.data_ptr(), F16, B.stride(0),
                                    C.data_ptr(), F16, N, W, T, K, N, torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_point_matches_regular_one(oracle):
    from graph_rws_b200 import core
    from graph_rws_b200.core import _native
    lib = _native.lib()
    # two different graphs and widths, back to back on one stream: the second call reuses the
    # array the first one left dirty (hub windows make both calls write partial tiles)
    cases = [(_graph(41, 30000, 400000), 128), (_graph(42, 9000, 150000), 256)]
    for graph, N in cases:
        B = torch.randn(graph.num_rows, N, generator=torch.Generator().manual_seed(N)).half().cuda()
        want = core.spmm_raw(graph.window_offset, graph.original_col_indices, graph.values_condensed, B,
                             algo=core.ALGO_TCGEN05, check=True)
        for _ in range(2):
            got = torch.full_like(want, float("nan"))
            st = _call_static(lib, graph, B, got)
            assert st == 0, lib.grws_last_error()
            torch.cuda.synchronize()
            # same kernel, same summation order: the results are identical, not merely close
            assert torch.equal(got, want)
    # its status word is out of the caller's reach (it lives in the library's array): a wait that ran
    # out would show in the per-device word instead
    core.check_device_status()
    # and against the CPU checker, under the tolerance of the other SpMM tests, on the last case
    ref = oracle.spmm_fwd(graph.window_offset.cpu().numpy(), graph.original_col_indices.cpu().numpy(),
                          graph.values_condensed.float().cpu().numpy(), B.float().cpu().numpy()).astype(np.float64)
    err = np.linalg.norm(got.float().cpu().numpy() - ref) / np.linalg.norm(ref)
    assert err <= 1e-3
    rown = np.maximum(np.linalg.norm(ref, axis=1, keepdims=True), 1e-30)
    assert (np.abs(got.float().cpu().numpy() - ref) <= 2e-2 * rown + 1e-7).all()


def test_static_scratch_entry_point_rejects_what_it_cannot_hold():
    from graph_rws_b200.core import _native
    lib = _native.lib()
    graph = _graph(43, 2000, 12000)
    B32 = torch.randn(graph.num_rows, 128, device="cuda")
    C32 = torch.empty(graph.num_windows * 16, 128, device="cuda")
    T = graph.original_col_indices.numel() // 8
    st = lib.grws_spmm_fwd_static(graph.window_offset.data_ptr(), graph.original_col_indices.data_ptr(),
                                  graph.values_condensed.data_ptr(), 0, B32.data_ptr(), 0, 128, C32.data_ptr(), 0, 128,
                                  graph.num_windows, T, graph.num_rows, 128, None)
    assert st == -2 and b"allocation-free" in lib.grws_last_error()          # fp32: no static-scratch path
    B = torch.randn(graph.num_rows, 512, device="cuda").half()
    C = torch.empty(graph.num_windows * 16, 512, device="cuda", dtype=torch.float16)
    st = lib.grws_spmm_fwd_static(graph.window_offset.data_ptr(), graph.original_col_indices.data_ptr(),
                                  graph.values_condensed.data_ptr(), F16, B.data_ptr(), F16, 512, C.data_ptr(), F16, 512,
                                  graph.num_windows, T, graph.num_rows, 512, None)
    assert st == -2                                                            # width beyond the built-in scratch
