"""One process per GPU over torch.distributed (NCCL on NVLink / NVSwitch; gloo in the CPU tests).

The reference is single-GPU (helper/utils.py:19-24); this module covers the two places where its
hot path shards naturally:

* full-graph SpMM: contiguous window ranges per rank, balanced by tile count; every rank owns
  the matching rows of the dense operands; one all-gather of H before the local product (and one
  of G before the local rows of the transposed product);
* sampled training: seeds are sharded per rank, sampling is keyed by (seed, node, hop) so the
  result does not depend on the number of ranks; feature rows of a hop's input nodes are
  fetched from the ranks that own them.

Nothing here issues a TMA multicast load, and no TMA load or library kernel is handed a peer GPU's
memory: remote rows land in local HBM first, through the collective or through this library's own
copy kernels (plain loads: ``ShardedFeatures``, ``PeerAllGather``).
"""
from .row_partition import (RowPartition, all_gather_rows, all_gather_rows_padded, collective_timers,  # noqa: F401
                            partition_windows_by_tiles, shard_bcsr, DistributedSpMM, RowShardedGraph)
from .seed_shard import exchange_rows, owner_of, shard_seeds  # noqa: F401
from .feature_store import ShardedFeatures  # noqa: F401,E402
from .peer_gather import PeerAllGather, make_peer_all_gather  # noqa: F401,E402
