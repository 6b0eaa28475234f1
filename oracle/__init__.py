"""CPU checker for the Graph_RWS hot path -- TEST INFRASTRUCTURE ONLY.

numpy-facing wrappers over ``libgrws_oracle.so`` (``grws_oracle.c``, plain C + OpenMP).  Only the
tests, the smoke check and the CPU-baseline leg of the benchmark may import this package; the
product package never does.  Each wrapper names the reference code it restates.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libgrws_oracle.so")
_lib = None

_i64p = ctypes.POINTER(ctypes.c_int64)
_i32p = ctypes.POINTER(ctypes.c_int32)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_f32p = ctypes.POINTER(ctypes.c_float)


def build(force: bool = False) -> str:
    """Compile the C restatement (``make -C oracle``)."""
    src = os.path.join(_HERE, "grws_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.grws_oracle_csr_to_bcsr_count.restype = ctypes.c_int64
        _lib.grws_oracle_windows_and_masks.restype = ctypes.c_int64
        _lib.grws_oracle_dedup_reindex.restype = ctypes.c_int64
        _lib.grws_oracle_num_threads.restype = ctypes.c_int
    return _lib


def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return int(lib().grws_oracle_num_threads())


def use_all_host_threads() -> int:
    """OpenMP thread count := the cores this process may run on (a launcher may have exported
    OMP_NUM_THREADS=1); returns the count."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().grws_oracle_set_num_threads(ctypes.c_int(n))
    return num_threads()


def csr_to_bcsr(num_rows, row_ptr, col_idx, values, tile_rows=16, tile_cols=8):
    """CSR -> (window_offset i64, original_col_indices i32, values_condensed f32).

    Restates ``csr_to_bcsr_cpu`` (core/wrapper/convert_wrapper.cpp:27-180)."""
    row_ptr = _c(row_ptr, np.int64)
    col_idx = _c(col_idx, np.int32)
    values = _c(values, np.float32)
    W = (num_rows + tile_rows - 1) // tile_rows
    wo = np.zeros(W + 1, dtype=np.int64)
    T = lib().grws_oracle_csr_to_bcsr_count(
        ctypes.c_int64(num_rows), _p(row_ptr, _i64p), _p(col_idx, _i32p),
        ctypes.c_int64(tile_rows), ctypes.c_int64(tile_cols), _p(wo, _i64p))
    cols = np.empty(T * tile_cols, dtype=np.int32)
    vals = np.empty(T * tile_rows * tile_cols, dtype=np.float32)
    lib().grws_oracle_csr_to_bcsr_fill(
        ctypes.c_int64(num_rows), _p(row_ptr, _i64p), _p(col_idx, _i32p), _p(values, _f32p),
        ctypes.c_int64(tile_rows), ctypes.c_int64(tile_cols), _p(wo, _i64p),
        _p(cols, _i32p), _p(vals, _f32p))
    return wo, cols, vals


def spmm_fwd(window_offset, cols, vals, B, tile_rows=16, tile_cols=8):
    """C[W*16, N] = A_bcsr @ B; restates core/include/spmm_tc.cuh:113-193 in float64 accumulate."""
    window_offset = _c(window_offset, np.int64)
    cols = _c(cols, np.int32)
    vals = _c(vals, np.float32)
    B = _c(B, np.float32)
    W = window_offset.shape[0] - 1
    N = B.shape[1]
    C = np.zeros((W * tile_rows, N), dtype=np.float32)
    lib().grws_oracle_spmm_fwd(
        ctypes.c_int64(W), ctypes.c_int64(N), ctypes.c_int64(tile_rows), ctypes.c_int64(tile_cols),
        _p(window_offset, _i64p), _p(cols, _i32p), _p(vals, _f32p), _p(B, _f32p),
        ctypes.c_int64(N), _p(C, _f32p), ctypes.c_int64(N))
    return C


def spmm_transpose(window_offset, cols, vals, grad_out, num_cols, tile_rows=16, tile_cols=8):
    """G_in[num_cols, F] = A^T @ grad_out; restates core/include/spmm_tc.cuh:238-269."""
    window_offset = _c(window_offset, np.int64)
    cols = _c(cols, np.int32)
    vals = _c(vals, np.float32)
    grad_out = _c(grad_out, np.float32)
    W = window_offset.shape[0] - 1
    F = grad_out.shape[1]
    assert grad_out.shape[0] >= W * tile_rows
    out = np.zeros((num_cols, F), dtype=np.float32)
    lib().grws_oracle_spmm_transpose(
        ctypes.c_int64(W), ctypes.c_int64(F), ctypes.c_int64(tile_rows), ctypes.c_int64(tile_cols),
        _p(window_offset, _i64p), _p(cols, _i32p), _p(vals, _f32p), _p(grad_out, _f32p),
        ctypes.c_int64(num_cols), _p(out, _f32p))
    return out


def reindex(in_cols, values, active_windows, tile_rows=16, tile_cols=8):
    """Returns (new_cols, pruned_values); restates core/include/reindex.cuh:33-102."""
    in_cols = _c(in_cols, np.int32)
    values = np.array(values, dtype=np.float32, copy=True)
    active_windows = _c(active_windows, np.int32)
    out = np.empty_like(in_cols)
    lib().grws_oracle_reindex(
        _p(in_cols, _i32p), _p(values, _f32p), _p(active_windows, _i32p),
        ctypes.c_int64(in_cols.shape[0]), ctypes.c_int64(active_windows.shape[0]),
        ctypes.c_int32(tile_rows), ctypes.c_int32(tile_cols), _p(out, _i32p))
    return out, values


def windows_and_masks(seeds, tile_rows=16):
    """Sorted unique (window, OR-mask); restates core/wrapper/sampling_wrapper.cu:307-346."""
    seeds = _c(seeds, np.int32)
    n = seeds.shape[0]
    w = np.empty(max(n, 1), dtype=np.int32)
    m = np.empty(max(n, 1), dtype=np.int32)
    u = lib().grws_oracle_windows_and_masks(_p(seeds, _i32p), ctypes.c_int64(n),
                                            ctypes.c_int32(tile_rows), _p(w, _i32p), _p(m, _i32p))
    return w[:u].copy(), m[:u].copy()


def philox4x32_10(ctr, key):
    ctr = _c(ctr, np.uint32)
    key = _c(key, np.uint32)
    out = np.empty(4, dtype=np.uint32)
    lib().grws_oracle_philox4x32_10(_p(ctr, _u32p), _p(key, _u32p), _p(out, _u32p))
    return out


def sample_hop(row_ptr, col_idx, values, nodes, fanout, seed, hop):
    """Uniform sampling without replacement keyed by (seed, node, hop).

    Returns (nbr i32 [n, fanout] with -1 padding, w f32 [n, fanout], cnt i32 [n])."""
    assert 0 < fanout <= 1024
    row_ptr = _c(row_ptr, np.int64)
    col_idx = _c(col_idx, np.int32)
    values = None if values is None else _c(values, np.float32)
    nodes = _c(nodes, np.int32)
    n = nodes.shape[0]
    nbr = np.empty((n, fanout), dtype=np.int32)
    w = np.empty((n, fanout), dtype=np.float32)
    cnt = np.empty(n, dtype=np.int32)
    lib().grws_oracle_sample_hop(
        _p(row_ptr, _i64p), _p(col_idx, _i32p),
        _p(values, _f32p) if values is not None else None, _p(nodes, _i32p),
        ctypes.c_int64(n), ctypes.c_int32(fanout), ctypes.c_uint64(seed), ctypes.c_uint32(hop),
        _p(nbr, _i32p), _p(w, _f32p), _p(cnt, _i32p))
    return nbr, w, cnt


def dedup_reindex(dst, nbr):
    """src list = dst ++ sorted(unique(nbr) - dst); returns (src i32 [n_src], local i32 like nbr)."""
    dst = _c(dst, np.int32)
    nbr = _c(nbr, np.int32)
    n_dst = dst.shape[0]
    fanout = nbr.shape[1] if nbr.ndim == 2 else 0
    src = np.empty(n_dst + n_dst * fanout, dtype=np.int32)
    local = np.empty_like(nbr)
    n_src = lib().grws_oracle_dedup_reindex(
        _p(dst, _i32p), ctypes.c_int64(n_dst), _p(nbr, _i32p), ctypes.c_int32(fanout),
        _p(src, _i32p), _p(local, _i32p))
    return src[:n_src].copy(), local


def build_block(dst, nbr, w, tile_rows=16, tile_cols=8):
    """Per-hop BCSR block: rows = dst nodes (local order), columns = local ids in the src list.

    The block is exactly ``csr_to_bcsr`` of the sampled edges written as a local CSR, i.e. the
    layout rules of core/wrapper/convert_wrapper.cpp:27-180 applied to the hop.
    Returns (src, window_offset, cols, vals)."""
    dst = _c(dst, np.int32)
    src, local = dedup_reindex(dst, nbr)
    n_dst = dst.shape[0]
    valid = local >= 0
    cnt = valid.sum(axis=1).astype(np.int64) if n_dst else np.zeros(0, np.int64)
    row_ptr = np.zeros(n_dst + 1, dtype=np.int64)
    np.cumsum(cnt, out=row_ptr[1:])
    ci = local[valid].astype(np.int32)
    vv = np.asarray(w, dtype=np.float32)[valid]
    wo, cols, vals = csr_to_bcsr(n_dst, row_ptr, ci, vv, tile_rows, tile_cols)
    return src, wo, cols, vals


def sample_layers(row_ptr, col_idx, values, seeds, fanouts, seed, tile_rows=16, tile_cols=8):
    """Multi-hop replay.  Fanouts are consumed reversed (output layer first), like
    sampler/sampler.py:202-204.  Returns blocks in input->output order; each block is a dict
    with dst, src, window_offset, cols, vals."""
    blocks = []
    dst = _c(seeds, np.int32)
    for hop, f in enumerate(reversed(list(fanouts))):
        nbr, w, _ = sample_hop(row_ptr, col_idx, values, dst, f, seed, hop)
        src, wo, cols, vals = build_block(dst, nbr, w, tile_rows, tile_cols)
        blocks.insert(0, dict(dst=dst, src=src, window_offset=wo, cols=cols, vals=vals,
                              nbr=nbr, w=w))
        dst = src
    return blocks
