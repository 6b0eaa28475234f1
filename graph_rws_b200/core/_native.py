"""ctypes binding of libgrws_b200.so (declared in include/grws_b200.h).

There is no fallback: if the library cannot be loaded the import fails, and every call that
returns a negative status raises RuntimeError with the library's message -- the same exception
type the reference's TORCH_CHECK produces (core/wrapper/spmm_wrapper.cu:48-51).
"""
import ctypes
import os

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
# GRWS_LIB_PATH selects another build of the same library (kernel-variant comparisons)
LIB_PATH = os.environ.get("GRWS_LIB_PATH") or os.path.join(_CSRC, "libgrws_b200.so")

c_i64, c_i32, c_sz, c_vp = ctypes.c_int64, ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p

F32, F16, BF16 = 0, 1, 2
ALGO_AUTO, ALGO_WARP_MMA, ALGO_TCGEN05 = 0, 1, 2

# name -> (restype, argtypes); must list every function include/grws_b200.h declares
SIGNATURES = {
    "grws_last_error": (ctypes.c_char_p, []),
    "grws_version": (c_i32, []),
    "grws_spmm_scratch_bytes": (c_sz, [c_i64, c_i64, c_i64, c_i32]),
    "grws_spmm_resolve_algo": (c_i32, [c_i32, c_i64, c_i32]),
    "grws_spmm_fwd": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_vp, c_i32, c_i64, c_vp, c_i32, c_i64,
                              c_i64, c_i64, c_i64, c_i64, c_vp, c_sz, c_i32, c_vp]),
    "grws_peer_ctrl_bytes": (c_sz, []),
    "grws_peer_state_bytes": (c_sz, []),
    "grws_peer_all_gather": (c_i32, [c_vp, c_i64, c_vp, c_i64, c_vp, c_vp, c_i32, c_i32, c_vp, c_vp, ctypes.c_longlong, c_vp]),
    "grws_peer_all_gather_push": (c_i32, [c_vp, c_i64, c_i64, c_vp, c_vp, c_i32, c_i32, c_vp, ctypes.c_longlong, c_vp]),
    "grws_layer_norm_scratch_bytes": (c_sz, [c_i64]),
    "grws_layer_norm_fwd": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i32, c_i32, ctypes.c_float, c_vp]),
    "grws_layer_norm_bwd": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i32, c_i32, c_vp, c_sz, c_vp]),
    "grws_spmm_plan_bytes": (c_sz, [c_i64, c_i64, c_i64, c_i64]),
    "grws_spmm_plan_build": (c_i32, [c_vp, c_i64, c_i64, c_i64, c_i64, c_vp, c_sz, c_vp]),
    "grws_spmm_fwd_planned": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_vp, c_i32, c_i64, c_vp, c_i32, c_i64,
                                      c_i64, c_i64, c_i64, c_i64, c_vp, c_sz, c_i32, c_vp, c_sz, c_vp]),
    "grws_spmm_fwd_static": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_vp, c_i32, c_i64, c_vp, c_i32, c_i64,
                                     c_i64, c_i64, c_i64, c_i64, c_vp]),
    "grws_spmm_last_status": (c_i32, [c_vp, c_i32, c_vp]),
    "grws_spmm_check": (c_i32, [c_vp]),
    "grws_spmm_set_wait_limit": (c_i32, [ctypes.c_longlong]),
    "grws_csr_to_bcsr_scratch_bytes": (c_sz, [c_i64, c_i64]),
    "grws_csr_to_bcsr_count": (c_i32, [c_i64, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "grws_csr_to_bcsr_fill": (c_i32, [c_i64, c_i64, c_vp, c_i64, c_vp, c_vp, c_i32, c_vp, c_sz, c_vp]),
    "grws_csr_to_bcsr_count_bounded": (c_i32, [c_i64, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "grws_block_build_count": (c_i32, [c_vp, c_vp, c_i64, c_i32, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "grws_bcsr_transpose_scratch_bytes": (c_sz, [c_i64]),
    "grws_bcsr_transpose_count": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "grws_bcsr_transpose_fill": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_i64, c_vp, c_vp, c_vp,
                                         c_vp, c_sz, c_vp]),
    "grws_bcsr_to_csr_scratch_bytes": (c_sz, [c_i64]),
    "grws_bcsr_to_csr_count": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "grws_bcsr_to_csr_fill": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "grws_sample_hop": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, ctypes.c_uint64, ctypes.c_uint32,
                                c_vp, c_vp, c_vp, c_vp]),
    "grws_dedup_scratch_bytes": (c_sz, [c_i64, c_i32]),
    "grws_dedup_reindex": (c_i32, [c_vp, c_i64, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "grws_block_compact": (c_i32, [c_vp, c_vp, c_i64, c_i32, c_vp, c_vp, c_vp, c_vp]),
    "grws_sample_layers_sizes": (c_i32, [c_i64, c_vp, c_i32, c_i64, c_vp, c_vp, c_vp]),
    "grws_sample_layers_scratch_bytes": (c_sz, [c_i64, c_vp, c_i32, c_i64]),
    "grws_sample_layers": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_i32, ctypes.c_uint64, c_vp, c_i64, c_i32,
                                   c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "grws_gather_rows_sharded": (c_i32, [c_vp, c_i32, c_i64, c_i64, c_i64, c_vp, c_i64, c_vp, c_vp]),
    "grws_reindex_bcsr": (c_i32, [c_vp, c_vp, c_i32, c_vp, c_i64, c_i64, c_i32, c_i32, c_vp, c_vp]),
}

_lib = None


def _build_if_possible():
    import importlib.util
    spec = importlib.util.spec_from_file_location("_grws_csrc_build", os.path.join(_CSRC, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if os.path.exists(mod.NVCC):
        mod.build()


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH) or os.environ.get("GRWS_REBUILD"):
            _build_if_possible()
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python graph_rws_b200/csrc/build.py` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this library.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)          # AttributeError if the library lacks a symbol
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int):
    if status != 0:
        msg = lib().grws_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"grws_b200 error {status}: {msg}")
