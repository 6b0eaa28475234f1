"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def bcsr_from_csr_oracle(oracle, g, dtype):
    """BCSR arrays of a synthetic CSR graph built by the CPU checker; values rounded to dtype."""
    wo, cols, vals = oracle.csr_to_bcsr(g.num_nodes, g.row_ptr, g.col_idx, g.values)
    vals_t = torch.from_numpy(vals).to(dtype)
    return wo, cols, vals_t


def check_spmm_tolerance(C_gpu, C_ref, B_ref, what=""):
    """north-star tolerance: max-abs error <= 2e-2 * ||row|| and relative Frobenius error <= 1e-3,
    against the fp32/fp64 CPU product of the same (rounded) operands."""
    C_gpu = C_gpu.astype(np.float64)
    C_ref = C_ref.astype(np.float64)
    err = np.abs(C_gpu - C_ref)
    row_norm = np.linalg.norm(C_ref, axis=1, keepdims=True)
    bound = 2e-2 * np.maximum(row_norm, 1e-30)
    assert (err <= bound + 1e-7).all(), f"{what}: max-abs {err.max():.3e} beyond 2e-2*||row||"
    fro = np.linalg.norm(C_gpu - C_ref) / max(np.linalg.norm(C_ref), 1e-30)
    assert fro <= 1e-3, f"{what}: relative Frobenius error {fro:.3e} > 1e-3"
    return fro
