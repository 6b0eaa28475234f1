"""Operator surface of the reference's ``core`` package (core/__init__.py:9-21), served by
libgrws_b200.so through its C ABI.

The five reference names keep their argument meaning and return shapes:

    spmm_tc, spmm_transpose, reindex_bcsr, sample_all_layers, csr_to_bcsr_cpu

Unlike the reference, a missing native library is an ImportError here, never ``None``: there is
no other implementation to fall back to.
"""
import torch

from . import _native
from ._native import ALGO_AUTO, ALGO_TCGEN05, ALGO_WARP_MMA  # noqa: F401

_DT = {torch.float32: _native.F32, torch.float16: _native.F16, torch.bfloat16: _native.BF16}

_native.lib()   # fail at import time when the library is absent

_timing_enabled = False
_default_algo = ALGO_AUTO


def set_spmm_timing(enabled: bool):
    """When on, ``spmm_tc`` brackets the kernel with CUDA events and synchronises to return the
    elapsed milliseconds, like the reference always does (core/helper/timer.h:22-52)."""
    global _timing_enabled
    _timing_enabled = bool(enabled)


def set_spmm_algo(algo: int):
    global _default_algo
    _default_algo = int(algo)


def _ptr(t):
    return 0 if t is None or t.numel() == 0 else t.data_ptr()


def _stream(device):
    return torch.cuda.current_stream(device).cuda_stream


def _device_visible(t: torch.Tensor, name: str):
    """Graph arrays may live on the GPU or in pinned host memory (the reference's UVA mode only
    checks contiguity, core/wrapper/spmm_wrapper.cu:46-50)."""
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if not t.is_cuda and not t.is_pinned():
        raise RuntimeError(f"{name} must be a CUDA tensor or pinned host memory")


def check_device_status(device=None):
    """Synchronises the current stream of ``device`` and raises RuntimeError (status -5) if any
    tcgen05 SpMM launch on that device gave up on a pipeline wait since the last check: its output
    is then incomplete.  The kernels' waits are bounded, so a broken pipeline ends with this status
    instead of hanging the GPU.  Call it where the host synchronises anyway (end of an epoch)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(device):
        _native.check(_native.lib().grws_spmm_check(_stream(device)))


def _scratch(nbytes: int, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def spmm_plan(window_offset, num_tiles, K, N):
    """Tile ranges of the tcgen05 kernel's CTAs for one graph, balanced by pipeline stages, as a
    uint8 CUDA tensor to pass to ``spmm_raw(plan=...)``.  Worth building for a graph that is
    multiplied many times; it has to be rebuilt when ``window_offset`` changes.  No host
    synchronisation."""
    lib = _native.lib()
    W = window_offset.shape[0] - 1
    nbytes = lib.grws_spmm_plan_bytes(W, int(num_tiles), int(K), int(N))
    plan = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=window_offset.device)
    _native.check(lib.grws_spmm_plan_build(_ptr(window_offset), W, int(num_tiles), int(K), int(N),
                                           plan.data_ptr(), plan.numel(), _stream(window_offset.device)))
    return plan


def spmm_raw(window_offset, cols, vals, B, out_dtype=None, algo=None, num_tiles_bound=None, check=False, plan=None,
             out=None):
    """C[W*16, N] = A_bcsr @ B with values already in B's dtype and N % 8 == 0.

    ``check=True`` synchronises and raises if a tcgen05 launch reported a timed-out wait;
    ``plan`` is the result of ``spmm_plan`` for this graph, K and N (optional); ``out`` is a
    [W*16, N] tensor to write into, possibly a column slice of a wider matrix (rows 16-byte
    aligned, unit column stride)."""
    lib = _native.lib()
    W = window_offset.shape[0] - 1
    K, N = B.shape
    if out is None:
        out_dtype = out_dtype or B.dtype
        C = torch.empty((W * 16, N), dtype=out_dtype, device=B.device)
    else:
        C, out_dtype = out, out.dtype
        if (tuple(C.shape) != (W * 16, N) or C.stride(1) != 1 or C.device != B.device
                or (C.stride(0) * C.element_size()) % 16 or C.data_ptr() % 16):
            raise RuntimeError("out must be a [W*16, N] matrix on B's device with 16-byte aligned rows")
    if W == 0:
        return C
    T = cols.numel() // 8 if num_tiles_bound is None else int(num_tiles_bound)
    algo = _default_algo if algo is None else algo
    nbytes = lib.grws_spmm_scratch_bytes(W, T, N, algo)
    scratch = _scratch(nbytes, B.device)
    if plan is not None:
        _native.check(lib.grws_spmm_fwd_planned(
            _ptr(window_offset), _ptr(cols), _ptr(vals), _DT[vals.dtype], _ptr(B), _DT[B.dtype], B.stride(0),
            C.data_ptr(), _DT[out_dtype], C.stride(0), W, T, K, N, scratch.data_ptr(), scratch.numel(), algo,
            plan.data_ptr(), plan.numel(), _stream(B.device)))
    else:
        _native.check(lib.grws_spmm_fwd(
            _ptr(window_offset), _ptr(cols), _ptr(vals), _DT[vals.dtype], _ptr(B), _DT[B.dtype], B.stride(0),
            C.data_ptr(), _DT[out_dtype], C.stride(0), W, T, K, N, scratch.data_ptr(), scratch.numel(), algo,
            _stream(B.device)))
    if check:
        check_device_status(B.device)
    return C


def _spmm_any(window_offset, cols, vals, B, algo=None):
    """Handles what the raw entry point does not: value dtype != B dtype, N % 8 != 0."""
    if B.dtype not in _DT:
        raise RuntimeError(f"unsupported dense dtype {B.dtype}")
    if vals.dtype != B.dtype:
        vals = vals.to(device=B.device, dtype=B.dtype)
    N = B.shape[1]
    pad = (-N) % 8
    if pad or B.stride(1) != 1 or (B.stride(0) * B.element_size()) % 16 or B.data_ptr() % 16:
        Bp = torch.zeros((B.shape[0], N + pad), dtype=B.dtype, device=B.device)
        Bp[:, :N] = B
        B = Bp
    C = spmm_raw(window_offset, cols, vals, B, algo=algo)
    return C[:, :N] if pad else C


def spmm_tc(window_offset, original_col_indices, values_condensed, input_B, warps_per_block=8):
    """(C[W*16, N], elapsed_ms) -- signature of core/wrapper/bind.cpp:124-130.

    ``warps_per_block`` is accepted and ignored: the reference uses it to decide how many of
    the N columns get computed (8 per warp, core/include/spmm_tc.cuh:70); here all N are."""
    _device_visible(window_offset, "window_offset")
    _device_visible(original_col_indices, "original_col_indices")
    _device_visible(values_condensed, "values_condensed")
    if not input_B.is_cuda:
        raise RuntimeError("input_B must be a CUDA tensor")
    if not input_B.is_contiguous():
        raise RuntimeError("input_B must be contiguous")
    if _timing_enabled:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        C = _spmm_any(window_offset, original_col_indices, values_condensed, input_B)
        e1.record()
        e1.synchronize()
        return C, float(e0.elapsed_time(e1))
    return _spmm_any(window_offset, original_col_indices, values_condensed, input_B), 0.0


# ---------------------------------------------------------------------------------------------
# CSR -> BCSR and the cached transposed BCSR
# ---------------------------------------------------------------------------------------------
def csr_to_bcsr(num_rows, row_ptr, col_idx, values, tile_rows=16, tile_cols=8, values_dtype=torch.float32,
                exact=True, nnz_is_bound=False, num_cols=0):
    """Device builder: CUDA tensors in, CUDA tensors out (window_offset, cols, vals).

    With ``exact`` the tile count is read back from the device to size ``cols`` / ``vals`` exactly
    (what the reference's builder returns).  ``exact=False`` skips that host synchronisation and
    sizes them by the bound ``entries / 8 + windows`` (every window wastes less than one tile): the
    arrays then end in unused tiles (column ids -1, values 0) which no kernel visits, since all of
    them walk ``window_offset``.  Per-step builders (sampled blocks, their transposes) use it.
    ``nnz_is_bound``: only the first ``row_ptr[num_rows]`` entries of ``col_idx`` / ``values`` exist,
    their length is a bound (the caller did not read the count back either); ``num_cols`` (with
    ``nnz_is_bound``): every column id is below it, which lets the builder sort narrower keys."""
    if tile_rows != 16 or tile_cols != 8:
        raise RuntimeError("Currently only supports tile 16x8")
    lib = _native.lib()
    dev = row_ptr.device
    row_ptr = row_ptr.to(torch.int64).contiguous()
    col_idx = col_idx.to(torch.int32).contiguous()
    values = values.to(torch.float32).contiguous()
    nnz = col_idx.numel()
    W = (num_rows + 15) // 16
    wo = torch.empty(W + 1, dtype=torch.int64, device=dev)
    scratch = _scratch(lib.grws_csr_to_bcsr_scratch_bytes(num_rows, nnz), dev)
    st = _stream(dev)
    if nnz_is_bound:
        _native.check(lib.grws_csr_to_bcsr_count_bounded(num_rows, _ptr(row_ptr), _ptr(col_idx), _ptr(values), nnz,
                                                         int(num_cols), wo.data_ptr(), scratch.data_ptr(),
                                                         scratch.numel(), st))
    else:
        _native.check(lib.grws_csr_to_bcsr_count(num_rows, _ptr(row_ptr), _ptr(col_idx), _ptr(values), nnz,
                                                 wo.data_ptr(), scratch.data_ptr(), scratch.numel(), st))
    T = int(wo[-1].item()) if exact else nnz // 8 + W
    cols = torch.empty(T * 8, dtype=torch.int32, device=dev)
    vals = torch.empty(T * 128, dtype=values_dtype, device=dev)
    _native.check(lib.grws_csr_to_bcsr_fill(num_rows, nnz, wo.data_ptr(), T, _ptr(cols), _ptr(vals),
                                            _DT[values_dtype], scratch.data_ptr(), scratch.numel(), st))
    return wo, cols, vals


def csr_to_bcsr_cpu(num_rows, row_ptr, col_idx, values, tile_rows, tile_cols):
    """Same contract as the reference's host builder (core/wrapper/bind.cpp:144-151: CPU
    tensors in, CPU tensors out) but the work runs on the current CUDA device."""
    if not row_ptr.device.type == "cpu":
        raise RuntimeError("row_ptr must be on CPU")
    dev = torch.device("cuda", torch.cuda.current_device())
    wo, cols, vals = csr_to_bcsr(int(num_rows), row_ptr.to(dev), col_idx.to(dev), values.to(dev),
                                 int(tile_rows), int(tile_cols))
    return wo.cpu(), cols.cpu(), vals.cpu()


def bcsr_transpose(window_offset, cols, vals, num_cols, values_dtype=None, exact=True, nnz_bound=None):
    """BCSR of A^T (rows = column ids of A, ``num_cols`` of them; columns = rows of A).
    ``exact`` as in ``csr_to_bcsr``.  ``nnz_bound``: an upper bound on the number of non-zero
    entries that the caller knows without asking the device (a sampled block has at most
    rows x fanout); with it the entry count is not read back either."""
    lib = _native.lib()
    dev = vals.device
    W = window_offset.shape[0] - 1
    st = _stream(dev)
    row_ptr_t = torch.empty(num_cols + 1, dtype=torch.int64, device=dev)
    scratch = _scratch(lib.grws_bcsr_transpose_scratch_bytes(num_cols), dev)
    _native.check(lib.grws_bcsr_transpose_count(_ptr(window_offset), _ptr(cols), _ptr(vals), _DT[vals.dtype],
                                                W, num_cols, row_ptr_t.data_ptr(), scratch.data_ptr(),
                                                scratch.numel(), st))
    nnz = int(row_ptr_t[-1].item()) if nnz_bound is None else int(nnz_bound)
    col_t = torch.empty(nnz, dtype=torch.int32, device=dev)
    val_t = torch.empty(nnz, dtype=torch.float32, device=dev)
    _native.check(lib.grws_bcsr_transpose_fill(_ptr(window_offset), _ptr(cols), _ptr(vals), _DT[vals.dtype],
                                               W, num_cols, row_ptr_t.data_ptr(), _ptr(col_t), _ptr(val_t),
                                               scratch.data_ptr(), scratch.numel(), st))
    return csr_to_bcsr(num_cols, row_ptr_t, col_t, val_t, values_dtype=values_dtype or vals.dtype, exact=exact,
                       nnz_is_bound=nnz_bound is not None, num_cols=W * 16)


class _TransposeCache:
    """Keeps the transposed BCSR of the graphs recently seen by ``spmm_transpose``.  An entry
    holds references to the three source tensors, so their storage cannot be recycled while the
    entry lives, and records their versions, so an in-place edit invalidates it."""

    def __init__(self, capacity=8):
        self.capacity = capacity
        self.entries = []

    def get(self, wo, cols, vals, num_cols, dtype):
        key = (wo.data_ptr(), cols.data_ptr(), vals.data_ptr(), wo._version, cols._version, vals._version,
               wo.numel(), cols.numel(), int(num_cols), dtype)
        for i, (k, _, value) in enumerate(self.entries):
            if k == key:
                self.entries.append(self.entries.pop(i))
                return value
        value = bcsr_transpose(wo, cols, vals, num_cols, values_dtype=dtype)
        self.entries.append((key, (wo, cols, vals), value))
        if len(self.entries) > self.capacity:
            self.entries.pop(0)
        return value


_transpose_cache = _TransposeCache()


def spmm_transpose(window_offset, original_col_indices, values_condensed, grad_out, num_cols):
    """grad_in[num_cols, F] = A^T @ grad_out -- signature of core/wrapper/bind.cpp:133-140.

    The reference scatters with float atomics on every call; here A^T is built once per graph
    (cached on the identity and version of the three BCSR tensors) and multiplied with the same
    kernel as the forward pass, so the result is deterministic."""
    if not grad_out.is_cuda:
        raise RuntimeError("grad_out must be a CUDA tensor")
    if not grad_out.is_contiguous():
        raise RuntimeError("grad_out must be contiguous")
    _device_visible(window_offset, "window_offset")
    _device_visible(original_col_indices, "original_col_indices")
    _device_visible(values_condensed, "values_condensed")
    wo_t, cols_t, vals_t = _transpose_cache.get(window_offset, original_col_indices, values_condensed,
                                                int(num_cols), grad_out.dtype)
    out = _spmm_any(wo_t, cols_t, vals_t, grad_out)
    return out[:num_cols]


from .sampling import (SamplingTimingResult, bcsr_to_csr, build_block, reindex_bcsr,  # noqa: E402,F401
                       sample_all_layers, sample_hop, sample_layers_csr, sample_layers_fused,
                       sample_layers_sizes)

__all__ = ["sample_all_layers", "spmm_tc", "spmm_transpose", "csr_to_bcsr_cpu", "reindex_bcsr",
           "csr_to_bcsr", "bcsr_transpose", "spmm_raw", "set_spmm_timing", "set_spmm_algo",
           "check_device_status", "bcsr_to_csr", "sample_hop", "build_block", "sample_layers_csr", "sample_layers_fused",
           "sample_layers_sizes", "SamplingTimingResult"]
