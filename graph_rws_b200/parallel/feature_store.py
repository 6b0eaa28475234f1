"""Feature rows sharded over the GPUs of one node and read in place over NVLink.

``ShardedFeatures`` puts this rank's block of rows into memory that every peer GPU can address
(torch's symmetric-memory allocator: one CUDA allocation per rank, mapped into all ranks of the
group) and gathers the rows of a step's input nodes with one kernel of plain loads
(``grws_gather_rows_sharded``): no collective, no host synchronisation, nothing for the owning rank
to do.  The matrix is written once, before ``rendezvous``; afterwards it is read-only, so the
steps need no cross-rank ordering.

No TMA load and no library kernel is ever given a peer's memory: the gather kernel is this
library's own and uses ordinary loads; everything downstream reads the local copy it produces.
"""
import torch
import torch.distributed as dist

from ..core import _native


class ShardedFeatures:
    def __init__(self, x_local: torch.Tensor, num_rows: int, group=None):
        """``x_local``: rows [rank * per, (rank + 1) * per) of the [num_rows, F] matrix with
        per = ceil(num_rows / world); F * element_size must be a multiple of 16 bytes."""
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.num_rows = int(num_rows)
        self.per = (self.num_rows + self.world - 1) // self.world
        self.width, self.dtype, self.device = x_local.shape[1], x_local.dtype, x_local.device
        self.row_bytes = self.width * x_local.element_size()
        if self.row_bytes % 16:
            raise ValueError("feature rows must be a multiple of 16 bytes (pad the width)")
        if x_local.shape[0] > self.per:
            raise ValueError("this rank holds more rows than its share")
        self.block = symm_mem.empty((self.per, self.width), dtype=self.dtype, device=self.device)
        self.block[:x_local.shape[0]].copy_(x_local)
        self.block[x_local.shape[0]:].zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.block, self.group.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.shards = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        dist.barrier(self.group)          # every rank's block is filled before anybody reads it

    def gather(self, node_ids: torch.Tensor) -> torch.Tensor:
        """Rows ``node_ids`` (global ids, int32; -1 gives a zero row) as a local [n, F] matrix."""
        ids = node_ids.to(device=self.device, dtype=torch.int32).contiguous()
        out = torch.empty((ids.numel(), self.width), dtype=self.dtype, device=self.device)
        _native.check(_native.lib().grws_gather_rows_sharded(
            self.shards.data_ptr(), self.world, self.per, self.row_bytes, self.row_bytes, ids.data_ptr(), ids.numel(),
            out.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream))
        return out

    __call__ = gather
