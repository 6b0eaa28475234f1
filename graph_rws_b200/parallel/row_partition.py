"""Row-partitioned full-graph SpMM: window ranges per rank, all-gather of the dense operand."""
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


class _CollectiveTimers:
    """Optional CUDA-event timing of the collectives on the path (off by default: the extra events
    cost a little).  ``start()``, run some steps, ``stop()`` returns the milliseconds spent per
    collective kind on the launching stream -- what a benchmark needs to say which part of an
    epoch is communication."""

    def __init__(self):
        self.on = False
        self.pairs = []

    def start(self):
        self.on, self.pairs = True, []

    def stop(self):
        self.on = False
        out = {}
        for name, a, b in self.pairs:
            b.synchronize()
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        self.pairs = []
        return out

    class _Span:
        def __init__(self, owner, name, device):
            self.owner, self.name, self.device = owner, name, device

        def __enter__(self):
            if self.owner.on and self.device.type == 'cuda':
                self.a = torch.cuda.Event(enable_timing=True)
                self.a.record()
            return self

        def __exit__(self, *exc):
            if self.owner.on and self.device.type == 'cuda':
                b = torch.cuda.Event(enable_timing=True)
                b.record()
                self.owner.pairs.append((self.name, self.a, b))
            return False

    def timed(self, name, device):
        return self._Span(self, name, torch.device(device))


collective_timers = _CollectiveTimers()


@dataclass
class RowPartition:
    """Contiguous window range [w_begin, w_end) of every rank and the matching row ranges."""
    window_bounds: List[int]       # world + 1 entries
    num_rows: int

    @property
    def world(self) -> int:
        return len(self.window_bounds) - 1

    def windows(self, rank: int):
        return self.window_bounds[rank], self.window_bounds[rank + 1]

    def rows(self, rank: int):
        lo, hi = self.windows(rank)
        return min(lo * 16, self.num_rows), min(hi * 16, self.num_rows)

    def max_rows(self) -> int:
        return max(self.rows(r)[1] - self.rows(r)[0] for r in range(self.world))

    def padded_ids(self, ids: torch.Tensor) -> torch.Tensor:
        """Row ids in the padded numbering of ``all_gather_rows_padded``: rank r's rows start at
        ``r * max_rows()``.  Negative ids (padding) stay as they are.  The map is increasing, so
        sorted column lists stay sorted."""
        starts = torch.tensor([self.rows(r)[0] for r in range(self.world)], dtype=torch.int64, device=ids.device)
        ends = torch.tensor([self.rows(r)[1] for r in range(self.world)], dtype=torch.int64, device=ids.device)
        idl = ids.to(torch.int64)
        owner = torch.bucketize(idl, ends, right=True).clamp_(max=self.world - 1)
        out = owner * self.max_rows() + (idl - starts[owner])
        return torch.where(idl < 0, idl, out).to(ids.dtype)


def partition_windows_by_tiles(window_offset: torch.Tensor, world: int, num_rows: Optional[int] = None) -> RowPartition:
    """Cut the windows into ``world`` contiguous ranges of (nearly) equal TILE count: the SpMM cost
    of a window is its tile count, and power-law graphs make window counts a poor proxy."""
    wo = window_offset.detach().cpu().to(torch.int64)
    W = wo.numel() - 1
    T = int(wo[-1])
    bounds = [0]
    for r in range(1, world):
        target = (T * r) // world
        # first window whose start is >= target, never behind the previous cut
        w = int(torch.searchsorted(wo[:-1].contiguous(), torch.tensor(target), right=False))
        bounds.append(min(max(w, bounds[-1]), W))
    bounds.append(W)
    return RowPartition(bounds, W * 16 if num_rows is None else int(num_rows))


def shard_bcsr(window_offset, cols, vals, part: RowPartition, rank: int):
    """The rank's slice of a BCSR graph: same column ids (global), local windows."""
    lo, hi = part.windows(rank)
    t0, t1 = int(window_offset[lo]), int(window_offset[hi])
    wo = (window_offset[lo:hi + 1] - t0).contiguous()
    return wo, cols[t0 * 8:t1 * 8].contiguous(), vals[t0 * 128:t1 * 128].contiguous()


def all_gather_rows(local: torch.Tensor, part: RowPartition, group=None) -> torch.Tensor:
    """All-gather the row shards of a dense matrix into the full [num_rows, N] matrix.

    Shards may differ in size, so each rank contributes ``max_rows`` rows (zero padded) to one
    ``all_gather_into_tensor`` and the valid parts are copied out."""
    world = part.world
    if world == 1:
        return local
    pad_rows = part.max_rows()
    n = local.shape[1]
    send = local
    if local.shape[0] != pad_rows:
        send = torch.zeros((pad_rows, n), dtype=local.dtype, device=local.device)
        send[:local.shape[0]] = local
    recv = torch.empty((world * pad_rows, n), dtype=local.dtype, device=local.device)
    with collective_timers.timed("all_gather", local.device):
        dist.all_gather_into_tensor(recv, send.contiguous(), group=group)
    if all(part.rows(r)[1] - part.rows(r)[0] == pad_rows for r in range(world)):
        return recv[:part.num_rows]
    full = torch.empty((part.num_rows, n), dtype=local.dtype, device=local.device)
    for r in range(world):
        lo, hi = part.rows(r)
        full[lo:hi] = recv[r * pad_rows:r * pad_rows + (hi - lo)]
    return full


def all_gather_rows_padded(local: torch.Tensor, part: RowPartition, group=None) -> torch.Tensor:
    """All-gather the row shards into a [world * max_rows, N] matrix in which rank r's rows start at
    ``r * max_rows`` (``RowPartition.padded_ids`` gives the numbering).  Nothing is copied out
    afterwards: the consumer's column ids are rewritten to this numbering once, when the graph is
    sharded, so the product reads the receive buffer directly.  The rows between a rank's last row
    and the next rank's first are never referenced."""
    world = part.world
    pad_rows = part.max_rows()
    n = local.shape[1]
    if world == 1:
        return local
    peer = getattr(part, 'peer_gather', None)
    if peer is not None and local.is_cuda and local.shape[1] * local.element_size() <= peer.max_row_bytes \
            and (local.shape[1] * local.element_size()) % 16 == 0:
        with collective_timers.timed("all_gather", local.device):
            return peer.gather(local)
    send = local
    if local.shape[0] != pad_rows:
        send = torch.empty((pad_rows, n), dtype=local.dtype, device=local.device)
        send[:local.shape[0]] = local
        send[local.shape[0]:] = 0
    recv = torch.empty((world * pad_rows, n), dtype=local.dtype, device=local.device)
    with collective_timers.timed("all_gather", local.device):
        dist.all_gather_into_tensor(recv, send.contiguous(), group=group)
    return recv


class DistributedSpMM:
    """C_local = A[rows of this rank, :] @ H for H sharded by the same row partition
    (a square, symmetric-pattern adjacency: rows and columns share one node numbering)."""

    def __init__(self, graph, part: RowPartition, rank: int, group=None):
        from ..data import BCSRGraph
        self.part, self.rank, self.group = part, rank, group
        wo, cols, vals = shard_bcsr(graph.window_offset, graph.original_col_indices, graph.values_condensed, part, rank)
        lo, hi = part.rows(rank)
        self.local = BCSRGraph(num_nodes=hi - lo, num_edges=None, tile_rows=16, tile_cols=8, window_offset=wo,
                               original_col_indices=cols, values_condensed=vals, device=vals.device,
                               num_rows=hi - lo, num_cols=part.num_rows, values_dtype=vals.dtype)

    def __call__(self, h_local: torch.Tensor) -> torch.Tensor:
        from .. import core
        h_full = all_gather_rows(h_local, self.part, self.group)
        g = self.local
        out = core.spmm_raw(g.window_offset, g.original_col_indices, g.values_as(h_full.dtype), h_full.contiguous(),
                            plan=g.spmm_plan(h_full.shape[0], h_full.shape[1]))
        lo, hi = self.part.rows(self.rank)
        return out[:hi - lo]


class RowShardedGraph:
    """This rank's rows of a square adjacency, usable wherever the layers take a ``BCSRGraph``.

    Forward: the row shards of the dense operand are all-gathered, then the local windows are
    multiplied.  Backward: ``transposed()`` returns the rank's rows of A^T with the same hook, so
    ``A^T @ G`` all-gathers the row shards of G and multiplies the local rows of A^T -- no
    reduce-scatter and no atomics.  Weight gradients are all-reduced by the training step."""

    def __init__(self, local, part: RowPartition, rank: int, local_t=None, group=None):
        self.local, self.part, self.rank, self.group = local, part, rank, group
        self._local_t = local_t
        # column ids in the padded numbering of the all-gathered operand (done once, here): the
        # product then reads the receive buffer of the all-gather without a compaction pass
        if part.world > 1 and not getattr(local, '_padded_cols', False):
            local.original_col_indices = part.padded_ids(local.original_col_indices)
            local._padded_cols = True
        for name in ("window_offset", "original_col_indices", "values_condensed", "tile_rows", "tile_cols",
                     "num_windows", "device"):
            setattr(self, name, getattr(local, name))
        lo, hi = part.rows(rank)
        self.num_rows = self.num_nodes = hi - lo
        self.num_cols = part.world * part.max_rows() if part.world > 1 else part.num_rows
        self._shared = local._shared

    @classmethod
    def from_full(cls, graph, part: RowPartition, rank: int, dtype=None, group=None, peer_row_bytes: int = 0):
        """Shard a full graph held by every rank (and its transposed graph) by the same row partition.

        ``peer_row_bytes`` > 0 (the widest dense row that will be exchanged, in bytes): the
        all-gathers of the products run on the library's own NVLink kernels
        (``parallel.PeerAllGather``) instead of the NCCL collective, provided the GPUs can address
        each other's memory and two probe exchanges reproduce the collective; a collective call,
        every rank must make it."""
        from ..data import BCSRGraph

        def shard(g):
            wo, cols, vals = shard_bcsr(g.window_offset, g.original_col_indices, g.values_condensed, part, rank)
            lo, hi = part.rows(rank)
            return BCSRGraph(num_nodes=hi - lo, num_edges=None, tile_rows=16, tile_cols=8, window_offset=wo,
                             original_col_indices=cols, values_condensed=vals, device=vals.device,
                             num_rows=hi - lo, num_cols=part.num_rows, values_dtype=vals.dtype)
        gt = graph.transposed(part.num_rows, dtype=dtype or graph.values_condensed.dtype)
        if peer_row_bytes and part.world > 1 and graph.window_offset.is_cuda and getattr(part, 'peer_gather', None) is None:
            from .peer_gather import make_peer_all_gather
            part.peer_gather = make_peer_all_gather(part.max_rows(), int(peer_row_bytes), graph.window_offset.device, group)
        return cls(shard(graph), part, rank, local_t=cls(shard(gt), part, rank, group=group), group=group)

    def values_as(self, dtype):
        return self.local.values_as(dtype)

    def spmm_plan(self, K, N):
        return self.local.spmm_plan(K, N)

    def gather_dense(self, dense_local):
        # a product returns whole windows: rows past the rank's last row are padding
        return all_gather_rows_padded(dense_local[:self.num_rows], self.part, self.group)

    def transposed(self, num_cols=None, dtype=None):
        if self._local_t is None:
            raise RuntimeError("this shard was built without its transposed rows")
        return self._local_t
