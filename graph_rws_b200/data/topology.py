"""CSR topology for neighbour sampling when a full-graph BCSR is not wanted or cannot exist.

The reference samples from the BCSR tiles of the whole graph (core/include/sampling.cuh:188-394) and
keeps graphs that do not fit the GPU in pinned host memory (data/data_loader.py:1513-1564).  The
per-node sampler of this library walks CSR rows, so a graph that is only ever sampled needs no
BCSR at all: 8 bytes per node plus 4 (topology) or 8 (with weights) bytes per edge.  The
111 M-node / 3.2 B-entry configuration is 13.7 GB that way, replicated per GPU, while its BCSR
(about 4e8 tiles of 544 bytes) would not fit; only the per-hop blocks of a step are BCSR.
"""
from typing import Optional

import torch


class CSRTopology:
    def __init__(self, row_ptr: torch.Tensor, col_idx: torch.Tensor, values: Optional[torch.Tensor] = None,
                 device: Optional[torch.device] = None, block_dtype: torch.dtype = torch.float32):
        """``row_ptr`` int64 [n+1], ``col_idx`` int32 [nnz] (up to 2^63 entries: the sampler indexes
        them with 64-bit offsets), ``values`` fp32 [nnz] or None (every sampled edge then weighs 1).
        ``block_dtype`` is the value dtype of the per-hop blocks built from this topology."""
        device = torch.device(device) if device is not None else row_ptr.device
        self.row_ptr = row_ptr.to(device=device, dtype=torch.int64).contiguous()
        self.col_idx = col_idx.to(device=device, dtype=torch.int32).contiguous()
        self.values = None if values is None else values.to(device=device, dtype=torch.float32).contiguous()
        self.device = device
        self.num_nodes = self.num_rows = self.num_cols = int(self.row_ptr.numel() - 1)
        self.block_dtype = block_dtype

    @property
    def nnz(self) -> int:
        return int(self.col_idx.numel())

    def csr(self):
        return self.row_ptr, self.col_idx, self.values

    @classmethod
    def from_bcsr(cls, g, block_dtype: Optional[torch.dtype] = None) -> 'CSRTopology':
        """CSR view of a BCSRGraph (extracted on the device)."""
        from .. import core
        rp, ci, vv = core.bcsr_to_csr(g.window_offset, g.original_col_indices, g.values_condensed, g.num_rows)
        return cls(rp, ci, vv, device=rp.device, block_dtype=block_dtype or g.values_condensed.dtype)

    def __repr__(self) -> str:
        return f"CSRTopology(nodes={self.num_nodes}, nnz={self.nnz}, weighted={self.values is not None}, device={self.device})"
