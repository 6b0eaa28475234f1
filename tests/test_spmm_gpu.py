"""GPU parity of the forward / transposed SpMM against the CPU checker, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, golden_cases, load_case
from gpu_util import DT, check_spmm_tolerance

pytestmark = pytest.mark.gpu


def _run(oracle, wo, cols, vals_np, num_cols, N, dt, algo, seed=0, out_dtype=None):
    """bf16 operands are checked with an fp32 output: the stated tolerance (relative Frobenius
    1e-3) is for fp16/bf16 inputs with fp32 accumulation, and rounding the *output* to bf16 alone
    costs 2^-9/sqrt(3) = 1.1e-3.  bf16 outputs get their own test with that floor added."""
    from graph_rws_b200 import core
    dev = torch.device("cuda")
    dtype = DT[dt]
    if out_dtype is None:
        out_dtype = torch.float32 if dt == "bf16" else dtype
    g = torch.Generator().manual_seed(seed)
    B = torch.randn(num_cols, N, generator=g).to(dtype)
    vals = torch.from_numpy(vals_np).to(dtype)
    C = core.spmm_raw(torch.from_numpy(wo).to(dev), torch.from_numpy(cols).to(dev), vals.to(dev), B.to(dev),
                      out_dtype=out_dtype, algo=algo, check=True)
    torch.cuda.synchronize()
    C_ref = oracle.spmm_fwd(wo, cols, vals.float().numpy(), B.float().numpy())
    return C.float().cpu().numpy(), C_ref


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: os.path.basename(p)[5:-4])
def test_warp_mma_matches_oracle_on_golden_graphs(oracle, path, dt):
    from graph_rws_b200 import core
    c = load_case(path)
    num_cols = int(c["col_idx"].max()) + 1 if c["col_idx"].size else 8
    for N in (8, 72, 128):
        C, C_ref = _run(oracle, c["window_offset"], c["cols"], c["vals"], num_cols, N, dt, core.ALGO_WARP_MMA)
        assert C.shape == C_ref.shape
        check_spmm_tolerance(C, C_ref, None, f"{os.path.basename(path)} N={N} {dt}")


@pytest.mark.parametrize("dt,N", [("f16", 128), ("bf16", 256), ("f32", 16), ("f32", 136), ("f16", 64)])
def test_warp_mma_power_law_graph_with_split_windows(oracle, dt, N):
    """A hub-heavy graph: windows longer than the split threshold exercise the partial-sum path."""
    from graph_rws_b200 import core
    from graph_rws_b200.data import synthetic
    g = synthetic.sym_normalized_csr(6000, *synthetic.chung_lu_edges(6000, 90000, 2.1, 21))
    wo, cols, vals = oracle.csr_to_bcsr(g.num_nodes, g.row_ptr, g.col_idx, g.values)
    assert (np.diff(wo) > 128).any(), "test graph must contain windows that get split"
    C, C_ref = _run(oracle, wo, cols, vals, g.num_nodes, N, dt, core.ALGO_WARP_MMA, seed=5)
    check_spmm_tolerance(C, C_ref, None, f"power-law N={N} {dt}")


@pytest.mark.parametrize("dt,N", [("f16", 128), ("bf16", 128), ("f16", 256), ("bf16", 256)])
@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: os.path.basename(p)[5:-4])
def test_tcgen05_matches_oracle_on_golden_graphs(oracle, path, dt, N):
    from graph_rws_b200 import core
    c = load_case(path)
    num_cols = int(c["col_idx"].max()) + 1 if c["col_idx"].size else 8
    C, C_ref = _run(oracle, c["window_offset"], c["cols"], c["vals"], num_cols, N, dt, core.ALGO_TCGEN05)
    check_spmm_tolerance(C, C_ref, None, f"tcgen05 {os.path.basename(path)} N={N} {dt}")


@pytest.mark.parametrize("dt,N,out", [("f16", 128, "f16"), ("bf16", 256, "f32"), ("f16", 256, "f32")])
def test_tcgen05_power_law_graph(oracle, dt, N, out):
    """Hub windows span several CTAs' tile ranges: exercises the partial tiles and the fix-up.
    With 20,000 rows the width-256 cases also take the two-pass route (128 columns per pass,
    strided operand and output); the small golden graphs take the single two-slab pass."""
    from graph_rws_b200 import core
    from graph_rws_b200.data import synthetic
    g = synthetic.sym_normalized_csr(20000, *synthetic.chung_lu_edges(20000, 300000, 2.1, 23))
    wo, cols, vals = oracle.csr_to_bcsr(g.num_nodes, g.row_ptr, g.col_idx, g.values)
    assert np.diff(wo).max() > wo[-1] // 148 + 2, "a window must be longer than one CTA's share"
    C, C_ref = _run(oracle, wo, cols, vals, g.num_nodes, N, dt, core.ALGO_TCGEN05, seed=5, out_dtype=DT[out])
    check_spmm_tolerance(C, C_ref, None, f"tcgen05 power-law N={N} {dt}")


@pytest.mark.parametrize("dt,N,out", [("f16", 48, "f16"), ("bf16", 64, "f32"), ("f16", 96, "f16"), ("f16", 8, "f32"), ("bf16", 120, "bf16")])
def test_tcgen05_narrow_operands(oracle, dt, N, out):
    """Widths below 128: the operand is multiplied as 128 features of which the missing ones are
    zeros (the TMA unit fills them in), and only the existing features are written.  Output rows are
    placed in a wider buffer whose other columns must stay untouched."""
    from graph_rws_b200 import core
    from graph_rws_b200.core import _native
    from graph_rws_b200.data import synthetic
    dev = torch.device("cuda")
    g = synthetic.sym_normalized_csr(20000, *synthetic.chung_lu_edges(20000, 300000, 2.1, 23))
    wo, cols, vals = oracle.csr_to_bcsr(g.num_nodes, g.row_ptr, g.col_idx, g.values)
    C, C_ref = _run(oracle, wo, cols, vals, g.num_nodes, N, dt, core.ALGO_TCGEN05, seed=7, out_dtype=DT[out])
    if out == "bf16":
        C_ref = torch.from_numpy(C_ref).bfloat16().float().numpy()
        assert np.abs(C - C_ref).max() <= 2 ** -7 * np.abs(C_ref).max() + 1e-6
    else:
        check_spmm_tolerance(C, C_ref, None, f"tcgen05 narrow N={N} {dt}")
    # strided output: columns N .. ldc-1 of the buffer belong to somebody else
    lib = _native.lib()
    dtype = DT[dt]
    W, T, ldc = len(wo) - 1, int(wo[-1]), 136
    B = torch.randn(g.num_nodes, N, generator=torch.Generator().manual_seed(7)).to(dtype).to(dev)
    vals_d = torch.from_numpy(vals).to(dtype).to(dev)
    wo_d, cols_d = torch.from_numpy(wo).to(dev), torch.from_numpy(cols).to(dev)
    buf = torch.full((W * 16, ldc), 7.0, dtype=dtype, device=dev)
    nbytes = lib.grws_spmm_scratch_bytes(W, T, N, core.ALGO_TCGEN05)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    code = {"f16": 1, "bf16": 2}[dt]
    _native.check(lib.grws_spmm_fwd(wo_d.data_ptr(), cols_d.data_ptr(), vals_d.data_ptr(), code, B.data_ptr(), code, N,
                                    buf.data_ptr(), code, ldc, W, T, g.num_nodes, N, scratch.data_ptr(), nbytes,
                                    core.ALGO_TCGEN05, torch.cuda.current_stream().cuda_stream))
    core.check_device_status()
    assert bool((buf[:, N:] == 7.0).all()), "columns beyond N were written"
    ref16 = oracle.spmm_fwd(wo, cols, vals_d.float().cpu().numpy(), B.float().cpu().numpy())
    if dt == "f16":
        check_spmm_tolerance(buf[:, :N].float().cpu().numpy(), ref16, None, f"strided narrow N={N}")


def test_tcgen05_and_warp_paths_agree(oracle):
    from graph_rws_b200 import core
    c = load_case(os.path.join(GOLDEN, "bcsr_chunglu_600.npz"))
    a, _ = _run(oracle, c["window_offset"], c["cols"], c["vals"], 600, 128, "f16", core.ALGO_TCGEN05, out_dtype=torch.float32)
    b, _ = _run(oracle, c["window_offset"], c["cols"], c["vals"], 600, 128, "f16", core.ALGO_WARP_MMA, out_dtype=torch.float32)
    np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-5)


def test_bf16_output_rounding_floor(oracle):
    """bf16 in, bf16 out: error = accumulation error (<= 1e-3) + one bf16 rounding of the result."""
    from graph_rws_b200 import core
    c = load_case(os.path.join(GOLDEN, "bcsr_chunglu_600.npz"))
    C, C_ref = _run(oracle, c["window_offset"], c["cols"], c["vals"], 600, 128, "bf16", core.ALGO_WARP_MMA,
                    out_dtype=torch.bfloat16)
    fro = np.linalg.norm(C - C_ref) / np.linalg.norm(C_ref)
    assert fro <= 1e-3 + 2.0 ** -9, fro
    C16 = torch.from_numpy(C_ref).bfloat16().float().numpy()          # the checker's result rounded the same way
    assert np.linalg.norm(C - C16) / np.linalg.norm(C16) <= 1e-3


def test_padding_columns_contribute_nothing(oracle):
    """-1 column ids are masked even when their value slots hold non-zero data."""
    from graph_rws_b200 import core
    c = load_case(os.path.join(GOLDEN, "bcsr_ragged_37x50.npz"))
    vals = c["vals"].copy().reshape(-1, 16, 8)
    pad = (c["cols"].reshape(-1, 8) == -1)
    assert pad.any()
    vals[np.broadcast_to(pad[:, None, :], vals.shape)] = 123.0
    C, _ = _run(oracle, c["window_offset"], c["cols"], vals.reshape(-1), 50, 64, "f16", core.ALGO_WARP_MMA)
    _, C_ref = _run(oracle, c["window_offset"], c["cols"], c["vals"], 50, 64, "f16", core.ALGO_WARP_MMA)
    check_spmm_tolerance(C, C_ref, None, "padding")


def test_reference_named_entry_points(oracle):
    """spmm_tc / spmm_transpose keep the reference's signatures (core/wrapper/bind.cpp:124-140)."""
    from graph_rws_b200 import core
    c = load_case(os.path.join(GOLDEN, "bcsr_chunglu_600.npz"))
    dev = torch.device("cuda")
    wo, cols = torch.from_numpy(c["window_offset"]).to(dev), torch.from_numpy(c["cols"]).to(dev)
    vals = torch.from_numpy(c["vals"]).to(dev)
    B = torch.randn(600, 7, device=dev)                       # N = 7: padded inside
    C, ms = core.spmm_tc(wo, cols, vals, B, 8)
    assert C.shape == (38 * 16, 7) and C.dtype == torch.float32 and ms == 0.0
    C_ref = oracle.spmm_fwd(c["window_offset"], c["cols"], c["vals"], B.cpu().numpy())
    check_spmm_tolerance(C.cpu().numpy(), C_ref, None, "spmm_tc")
    G = torch.randn(38 * 16, 24, device=dev)
    Gin = core.spmm_transpose(wo, cols, vals, G, 600)
    assert Gin.shape == (600, 24)
    Gin_ref = oracle.spmm_transpose(c["window_offset"], c["cols"], c["vals"], G.cpu().numpy(), 600)
    check_spmm_tolerance(Gin.cpu().numpy(), Gin_ref, None, "spmm_transpose")
    # second call hits the cached transposed graph and is bit-identical (no atomics)
    assert torch.equal(core.spmm_transpose(wo, cols, vals, G, 600), Gin)
    with pytest.raises(RuntimeError):
        core.spmm_tc(wo, cols, vals, B.cpu(), 8)
    with pytest.raises(RuntimeError):
        core.spmm_tc(wo, cols, vals, B.t(), 8)
    core.set_spmm_timing(True)
    try:
        _, ms = core.spmm_tc(wo, cols, vals, B, 8)
        assert ms > 0.0
    finally:
        core.set_spmm_timing(False)


def test_against_reference_kernels_when_built(oracle):
    """Same inputs through the reference's own CUDA kernels (compiled into oracle/_ref/):
    spmm_tc with warps_per_block = N/8 (it computes 8 columns per warp) and spmm_transpose."""
    from oracle import build_ref
    from graph_rws_b200 import core
    ref = build_ref.load()
    if ref is None:
        pytest.skip("oracle/_ref/core_lib.so not built")
    c = load_case(os.path.join(GOLDEN, "bcsr_chunglu_600.npz"))
    dev = torch.device("cuda")
    wo, cols = torch.from_numpy(c["window_offset"]).to(dev), torch.from_numpy(c["cols"]).to(dev)
    vals = torch.from_numpy(c["vals"]).to(dev)
    for N in (64, 128, 256):
        B = torch.randn(600, N, device=dev)
        C_theirs, _ = ref.spmm_tc(wo, cols, vals, B, N // 8)
        C_ours, _ = core.spmm_tc(wo, cols, vals, B, N // 8)
        check_spmm_tolerance(C_ours.cpu().numpy(), C_theirs.cpu().numpy(), None, f"vs reference spmm_tc N={N}")
    G = torch.randn(38 * 16, 64, device=dev)
    G_theirs = ref.spmm_transpose(wo, cols, vals, G, 600)
    G_ours = core.spmm_transpose(wo, cols, vals, G, 600)
    check_spmm_tolerance(G_ours.cpu().numpy(), G_theirs.cpu().numpy(), None, "vs reference spmm_transpose")
    # reindex_bcsr: the reference's own kernel (core/include/reindex.cuh:33-102) on the same ids,
    # hits, misses and -1 padding included; new ids and the pruned values are bit-identical
    active = torch.unique(torch.div(cols[cols >= 0], 16, rounding_mode="floor"))[::2].int().contiguous()
    v_theirs, v_ours = vals.clone(), vals.clone()
    new_theirs = ref.reindex_bcsr(cols, v_theirs, active, 16, 8)
    new_ours = core.reindex_bcsr(cols, v_ours, active, 16, 8)
    assert torch.equal(new_ours, new_theirs) and torch.equal(v_ours, v_theirs)


def test_full_size_spmm_mid_forward_and_transposed(oracle):
    """The workload the headline is quoted on, at its stated size (169,343 nodes, 313,640 tiles,
    fp16, N = 128): forward and transposed product against the CPU checker."""
    from graph_rws_b200 import BCSRGraph, core
    from graph_rws_b200.data import synthetic
    dev = torch.device("cuda")
    g = synthetic.graph_for_config("spmm_mid")
    graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev, values_dtype=torch.float16)
    wo, cols, vals = oracle.csr_to_bcsr(g.num_nodes, g.row_ptr, g.col_idx, g.values)
    assert np.array_equal(graph.window_offset.cpu().numpy(), wo) and np.array_equal(graph.original_col_indices.cpu().numpy(), cols)
    vals16 = torch.from_numpy(vals).half().float().numpy()
    H = torch.randn(g.num_nodes, 128, generator=torch.Generator().manual_seed(2002)).half()
    G = torch.randn(graph.num_windows * 16, 128, generator=torch.Generator().manual_seed(3002)).half()
    C = core.spmm_raw(graph.window_offset, graph.original_col_indices, graph.values_condensed, H.to(dev), check=True)
    check_spmm_tolerance(C.float().cpu().numpy(), oracle.spmm_fwd(wo, cols, vals16, H.float().numpy()), None, "spmm_mid forward")
    D = core.spmm_transpose(graph.window_offset, graph.original_col_indices, graph.values_condensed, G.to(dev), g.num_nodes)
    core.check_device_status()
    check_spmm_tolerance(D.float().cpu().numpy(), oracle.spmm_transpose(wo, cols, vals16, G.float().numpy(), g.num_nodes), None,
                         "spmm_mid transposed")


@pytest.mark.parametrize("N", [256, 48])
def test_dense_community_shape_bf16(oracle, N):
    """The full-graph GCN configuration's graph shape at a quarter of its node count (58,241 nodes,
    ~7.2 M non-zeros, ~120 tiles per window), bf16: width 256 takes the two-pass tcgen05 route
    (operand above 8 MB), width 48 the warp-MMA kernel.  fp32 output, as for every bf16 case."""
    from graph_rws_b200 import BCSRGraph, core
    from graph_rws_b200.data import synthetic
    dev = torch.device("cuda")
    n = int(232965 * 0.25)
    rp, ci, vv = synthetic.community_csr_torch(n, int((114_600_000 * 0.0625 - n) // 2), 50, 0.8, 1003, dev)
    graph = BCSRGraph.from_csr(n, rp, ci, vv, device=dev, values_dtype=torch.bfloat16)
    wo, cols, vals = oracle.csr_to_bcsr(n, rp.cpu().numpy(), ci.cpu().numpy(), vv.cpu().numpy())
    assert np.array_equal(graph.window_offset.cpu().numpy(), wo)
    assert n * N * 2 > (8 << 20) or N == 48
    B = torch.randn(n, N, generator=torch.Generator().manual_seed(N)).bfloat16()
    C = core.spmm_raw(graph.window_offset, graph.original_col_indices, graph.values_condensed, B.to(dev),
                      out_dtype=torch.float32, check=True)
    C_ref = oracle.spmm_fwd(wo, cols, torch.from_numpy(vals).bfloat16().float().numpy(), B.float().numpy())
    check_spmm_tolerance(C.cpu().numpy(), C_ref, None, f"dense-community bf16 N={N}")


def test_column_ids_beyond_the_operand_contribute_nothing(oracle):
    """Ids >= K (a global-id graph multiplied with fewer rows than it names) read zeros in both
    kernels, like the -1 padding; the warp-MMA path must not touch memory past the operand."""
    from graph_rws_b200 import core
    c = load_case(os.path.join(GOLDEN, "bcsr_chunglu_600.npz"))
    dev = torch.device("cuda")
    K = 400                                                  # the graph names columns up to 599
    cols_ref = np.where(c["cols"] >= K, -1, c["cols"])
    for dt, N, algo in (("f16", 128, core.ALGO_TCGEN05), ("f16", 128, core.ALGO_WARP_MMA), ("f32", 72, core.ALGO_WARP_MMA)):
        dtype = DT[dt]
        B = torch.randn(K, N, generator=torch.Generator().manual_seed(3)).to(dtype)
        vals = torch.from_numpy(c["vals"]).to(dtype)
        C = core.spmm_raw(torch.from_numpy(c["window_offset"]).to(dev), torch.from_numpy(c["cols"]).to(dev), vals.to(dev),
                          B.to(dev), algo=algo, check=True)
        C_ref = oracle.spmm_fwd(c["window_offset"], cols_ref, vals.float().numpy(), B.float().numpy())
        check_spmm_tolerance(C.float().cpu().numpy(), C_ref, None, f"ids >= K, {dt} algo {algo}")
    # an operand without rows: every id is out of range, the product is zero rows
    Z = core.spmm_raw(torch.from_numpy(c["window_offset"]).to(dev), torch.from_numpy(c["cols"]).to(dev),
                      torch.from_numpy(c["vals"]).half().to(dev), torch.empty(0, 128, dtype=torch.float16, device=dev))
    assert Z.shape == (38 * 16, 128) and not Z.any()
