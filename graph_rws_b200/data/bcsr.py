"""BCSRGraph: the reference's graph container (data/bcsr.py:23-306) over device-built arrays.

Layout (same as the reference): rows are grouped into windows of ``tile_rows`` = 16; a window
lists its sorted unique column ids ``tile_cols`` = 8 per tile, padded with -1;
``window_offset`` int64 [W+1] is the prefix sum of tiles, ``original_col_indices`` int32 [T*8],
``values_condensed`` [T*16*8] row-major per tile.

Differences from the reference, all additive:
  * CSR -> BCSR runs on the GPU (``core.csr_to_bcsr``) instead of the host OpenMP builder;
  * ``values_condensed`` may be fp16 / bf16 (``values_dtype``); the reference forces fp32
    (data/bcsr.py:48-50) and fp32 stays the default;
  * ``transposed()`` builds and caches the BCSR of A^T for the backward product, and
    ``values_as(dtype)`` caches a cast copy of the values for mixed-precision layers;
  * ``num_edges`` of ``from_components`` is counted lazily, so wrapping sampler output does not
    synchronise (the reference calls ``count_nonzero().item()``, data/bcsr.py:147).
"""
from typing import Any, Optional

import numpy as np
import torch

from ..core import bcsr_transpose, csr_to_bcsr


class BCSRGraph:
    def __init__(self,
                 num_nodes: int,
                 num_edges: Optional[int],
                 tile_rows: int,
                 tile_cols: int,
                 window_offset: torch.Tensor,
                 original_col_indices: torch.Tensor,
                 values_condensed: torch.Tensor,
                 device: Optional[torch.device] = None,
                 num_rows: Optional[int] = None,
                 num_cols: Optional[int] = None,
                 values_dtype: Optional[torch.dtype] = torch.float32) -> None:
        self.device = device
        self.window_offset = window_offset.to(device, non_blocking=True).to(torch.int64)
        self.original_col_indices = original_col_indices.to(device, non_blocking=True).to(torch.int32)
        vdt = values_dtype or values_condensed.dtype
        self.values_condensed = values_condensed.to(device, non_blocking=True).to(vdt)

        self.num_rows = int(num_rows) if num_rows is not None else int(num_nodes)
        self.num_cols = int(num_cols) if num_cols is not None else int(num_nodes)
        self.num_nodes = int(num_nodes)
        self._num_edges = None if num_edges is None else int(num_edges)
        self.tile_rows = int(tile_rows)
        self.tile_cols = int(tile_cols)

        self.num_windows = int(self.window_offset.shape[0] - 1)
        self.num_tiles = None
        # state shared by shallow copies (the model copies the graph once per layer)
        self._shared = {}

    # ------------------------------------------------------------------ derived data
    @property
    def num_edges(self) -> int:
        if self._num_edges is None:
            v = self.values_condensed
            self._num_edges = int(torch.count_nonzero(v).item()) if v.numel() > 0 else 0
        return self._num_edges

    @num_edges.setter
    def num_edges(self, v):
        self._num_edges = None if v is None else int(v)

    def _versions(self):
        return (self.window_offset.data_ptr(), self.original_col_indices.data_ptr(),
                self.values_condensed.data_ptr(), self.original_col_indices._version,
                self.values_condensed._version)

    def values_as(self, dtype: torch.dtype) -> torch.Tensor:
        """``values_condensed`` in ``dtype`` (cached until the values change)."""
        if self.values_condensed.dtype == dtype:
            return self.values_condensed
        key = ("vals", dtype)
        hit = self._shared.get(key)
        if hit is not None and hit[0] == self._versions():
            return hit[1]
        v = self.values_condensed.to(dtype)
        self._shared[key] = (self._versions(), v)
        return v

    def spmm_plan(self, K: int, N: int):
        """Plan of the tcgen05 kernel's tile ranges for products of this graph with a [K, N] operand,
        cached until the graph changes.  It is built at the second product of a shape, so a graph
        that lives for one step (a sampled block) never pays for one: None then."""
        if getattr(self, 'transient', False) or not self.window_offset.is_cuda:
            return None
        key = ("plan", int(K), int(N))
        state = (self._versions(), self.window_offset._version)
        hit = self._shared.get(key)
        if hit is None or hit[0] != state:
            self._shared[key] = (state, None)
            return None
        if hit[1] is None:
            from ..core import spmm_plan
            plan = spmm_plan(self.window_offset, self.original_col_indices.numel() // self.tile_cols, K, N)
            self._shared[key] = (state, plan)
            return plan
        return hit[1]

    def transposed(self, num_cols: Optional[int] = None, dtype: Optional[torch.dtype] = None) -> 'BCSRGraph':
        """BCSR of A^T with ``num_cols`` rows (default ``self.num_cols``), built on the device once
        and cached; the backward product ``A^T @ G`` runs the forward kernel on it."""
        n = int(self.num_cols if num_cols is None else num_cols)
        dtype = dtype or self.values_condensed.dtype
        key = ("T", n, dtype)
        hit = self._shared.get(key)
        if hit is not None and hit[0] == self._versions():
            return hit[1]
        # a block that lives for one step skips the size read-backs: its tile arrays are sized by
        # a bound, and so is its entry count when the sampler recorded one (``nnz_bound``)
        wo, cols, vals = bcsr_transpose(self.window_offset, self.original_col_indices,
                                        self.values_condensed, n, values_dtype=dtype,
                                        exact=not getattr(self, 'transient', False),
                                        nnz_bound=getattr(self, 'nnz_bound', None))
        gt = BCSRGraph(num_nodes=n, num_edges=None, tile_rows=self.tile_rows, tile_cols=self.tile_cols,
                       window_offset=wo, original_col_indices=cols, values_condensed=vals,
                       device=vals.device, num_rows=n, num_cols=self.num_windows * self.tile_rows,
                       values_dtype=dtype)
        gt.transient = getattr(self, 'transient', False)
        self._shared[key] = (self._versions(), gt)
        return gt

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_dgl(cls, g: Any, tile_rows: int = 16, tile_cols: int = 8) -> 'BCSRGraph':
        """From any object with DGLGraph's ``device / num_nodes() / edges() / edata`` interface."""
        device = g.device
        num_nodes = g.num_nodes()
        src, dst = g.edges()
        edge_weights = g.edata.get('weight', None)
        _, row_ptr, col_idx, values = cls._coo_to_csr(num_nodes, src, dst, edge_weights, device)
        return cls._from_csr(num_rows=num_nodes, row_ptr=row_ptr, col_idx=col_idx, edge_values=values,
                             tile_rows=tile_rows, tile_cols=tile_cols, device=device, num_cols=num_nodes)

    @classmethod
    def from_mtx(cls, filepath: str, index_base: int = 0, undirected: bool = False,
                 tile_rows: int = 16, tile_cols: int = 8,
                 device: Optional[torch.device] = None) -> 'BCSRGraph':
        """From a Matrix Market file, all values 1 (data/bcsr.py:90-131)."""
        import scipy.io as sio
        import scipy.sparse as sps

        if device is None:
            device = torch.device('cuda')
        coo = sio.mmread(filepath).tocoo()
        rows = coo.row.astype(np.int64)
        cols = coo.col.astype(np.int64)
        if index_base == 1:
            rows -= 1
            cols -= 1
        if undirected:
            rows, cols = np.concatenate([rows, cols]), np.concatenate([cols, rows])
        n = int(max(rows.max(), cols.max()) + 1)
        csr = sps.csr_matrix((np.ones_like(rows, dtype=np.float32), (rows, cols)), shape=(n, n))
        return cls._from_csr(num_rows=n,
                             row_ptr=torch.from_numpy(csr.indptr.astype(np.int64)),
                             col_idx=torch.from_numpy(csr.indices.astype(np.int32)),
                             edge_values=torch.from_numpy(csr.data.astype(np.float32)),
                             tile_rows=tile_rows, tile_cols=tile_cols, device=device, num_cols=n)

    @classmethod
    def from_components(cls, window_offset: torch.Tensor, original_col_indices: torch.Tensor,
                        values_condensed: torch.Tensor, num_rows: int, num_cols: int,
                        tile_rows: int, tile_cols: int,
                        device: Optional[torch.device] = None) -> 'BCSRGraph':
        """Wrap kernel output (data/bcsr.py:134-159); keeps the dtype of the values it is given."""
        if device is None:
            device = window_offset.device
        return cls(num_nodes=int(num_rows), num_edges=None, tile_rows=tile_rows, tile_cols=tile_cols,
                   window_offset=window_offset, original_col_indices=original_col_indices,
                   values_condensed=values_condensed, device=device, num_rows=int(num_rows),
                   num_cols=int(num_cols), values_dtype=values_condensed.dtype)

    @classmethod
    def from_csr(cls, num_rows: int, row_ptr, col_idx, values, num_cols: Optional[int] = None,
                 device: Optional[torch.device] = None, tile_rows: int = 16, tile_cols: int = 8,
                 values_dtype: torch.dtype = torch.float32) -> 'BCSRGraph':
        """From CSR arrays (torch tensors or numpy arrays on any device)."""
        def as_t(x, dt):
            return (torch.from_numpy(np.ascontiguousarray(x)) if isinstance(x, np.ndarray) else x).to(dt)
        if device is None:
            device = torch.device('cuda')
        return cls._from_csr(num_rows, as_t(row_ptr, torch.int64), as_t(col_idx, torch.int32),
                             as_t(values, torch.float32), tile_rows, tile_cols, device, num_cols,
                             values_dtype=values_dtype)

    @classmethod
    def _coo_to_csr(cls, num_rows: int, src: torch.Tensor, dst: torch.Tensor,
                    edge_weights: Optional[torch.Tensor], device: torch.device):
        """COO -> CSR with torch ops, rows = ``src`` (data/bcsr.py:163-187)."""
        src = src.to(device=device, dtype=torch.long)
        dst = dst.to(device=device, dtype=torch.long)
        perm = torch.argsort(src * num_rows + dst)
        src, dst = src[perm], dst[perm]
        num_edges = int(src.numel())
        if edge_weights is not None:
            values = edge_weights.to(device)[perm].to(torch.float32)
        else:
            values = torch.ones(num_edges, dtype=torch.float32, device=device)
        row_ptr = torch.zeros(num_rows + 1, dtype=torch.int64, device=device)
        torch.cumsum(torch.bincount(src, minlength=num_rows), dim=0, out=row_ptr[1:])
        return num_edges, row_ptr, dst.to(torch.int32), values

    @classmethod
    def _from_csr(cls, num_rows: int, row_ptr: torch.Tensor, col_idx: torch.Tensor,
                  edge_values: torch.Tensor, tile_rows: int, tile_cols: int, device: torch.device,
                  num_cols: Optional[int] = None,
                  values_dtype: torch.dtype = torch.float32) -> 'BCSRGraph':
        """CSR -> BCSR on the GPU (the reference goes through the host, data/bcsr.py:190-234)."""
        if num_cols is None:
            num_cols = num_rows
        device = torch.device(device)
        if device.type != 'cuda':
            raise RuntimeError("BCSRGraph is built on a CUDA device; there is no host builder")
        wo, cols, vals = csr_to_bcsr(int(num_rows), row_ptr.to(device), col_idx.to(device),
                                     edge_values.to(device), int(tile_rows), int(tile_cols),
                                     values_dtype=values_dtype)
        return cls(num_nodes=int(num_rows), num_edges=int(col_idx.numel()), tile_rows=tile_rows,
                   tile_cols=tile_cols, window_offset=wo, original_col_indices=cols,
                   values_condensed=vals, device=device, num_rows=int(num_rows),
                   num_cols=int(num_cols), values_dtype=values_dtype)

    @classmethod
    def from_dgl_block(cls, block: Any, tile_rows: int = 16, tile_cols: int = 8) -> 'BCSRGraph':
        """From a DGL message-flow block: rows = destination nodes, columns = source nodes
        (data/bcsr.py:266-306)."""
        device = block.device
        num_rows = block.num_dst_nodes()
        num_cols = block.num_src_nodes()
        src, dst = block.edges()
        edge_weights = block.edata.get('weight', None) if 'weight' in block.edata else None
        _, row_ptr, col_idx, values = cls._coo_to_csr(num_rows, dst, src, edge_weights, device)
        return cls._from_csr(num_rows=num_rows, row_ptr=row_ptr, col_idx=col_idx, edge_values=values,
                             tile_rows=tile_rows, tile_cols=tile_cols, device=device, num_cols=num_cols)

    # ------------------------------------------------------------------ utilities
    def to(self, device: torch.device, non_blocking: bool = False) -> 'BCSRGraph':
        if device == self.device:
            return self
        return BCSRGraph(num_nodes=self.num_rows, num_edges=self._num_edges, tile_rows=self.tile_rows,
                         tile_cols=self.tile_cols,
                         window_offset=self.window_offset.to(device, non_blocking=non_blocking),
                         original_col_indices=self.original_col_indices.to(device, non_blocking=non_blocking),
                         values_condensed=self.values_condensed.to(device, non_blocking=non_blocking),
                         device=device, num_rows=self.num_rows, num_cols=self.num_cols,
                         values_dtype=self.values_condensed.dtype)

    def __repr__(self) -> str:
        return (f"BCSRGraph(rows={self.num_rows}, cols={self.num_cols}, windows={self.num_windows}, "
                f"tiles={self.num_tiles}, tile={self.tile_rows}x{self.tile_cols}, device={self.device})")
