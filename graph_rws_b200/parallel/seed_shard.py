"""Seed sharding and sharded-feature row exchange for sampled training."""
from typing import Optional

import torch
import torch.distributed as dist


def shard_seeds(seeds: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Contiguous, near-equal split of a step's seeds; sampling is keyed by (seed, node, hop), so
    every rank draws the same neighbours for a node as a single GPU would."""
    n = seeds.numel()
    lo, hi = (n * rank) // world, (n * (rank + 1)) // world
    return seeds[lo:hi]


def owner_of(node_ids: torch.Tensor, num_nodes: int, world: int) -> torch.Tensor:
    """Rank that owns each node's feature row when rows are split into ``world`` contiguous blocks of
    ceil(num_nodes / world) rows."""
    per = (num_nodes + world - 1) // world
    return torch.div(node_ids, per, rounding_mode='floor').clamp_(0, world - 1)


def exchange_rows(x_local: torch.Tensor, node_ids: torch.Tensor, num_nodes: int, group=None,
                  use_all_to_all: Optional[bool] = None) -> torch.Tensor:
    """Rows ``node_ids`` (global ids) of a feature matrix whose rows are sharded in contiguous blocks.

    Index exchange + row exchange.  With NCCL this is two ``all_to_all_single`` calls over NVLink;
    backends without all-to-all (gloo, used by the CPU tests) take an all-gather of padded request
    lists instead, which moves more data but has the same result."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    per = (num_nodes + world - 1) // world
    if world == 1:
        return x_local[node_ids.long()]
    dev, f = x_local.device, x_local.shape[1]
    ids = node_ids.long()
    owner = owner_of(ids, num_nodes, world)
    order = torch.argsort(owner, stable=True)
    sorted_ids = ids[order]
    send_counts = torch.bincount(owner, minlength=world)
    if use_all_to_all is None:
        use_all_to_all = dist.get_backend(group) == "nccl"
    if use_all_to_all:
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        req = torch.empty(sum(rc), dtype=torch.long, device=dev)
        dist.all_to_all_single(req, sorted_ids, output_split_sizes=rc, input_split_sizes=sc, group=group)
        rows = x_local[req - rank * per]
        got = torch.empty((sum(sc), f), dtype=x_local.dtype, device=dev)
        dist.all_to_all_single(got, rows, output_split_sizes=sc, input_split_sizes=rc, group=group)
    else:
        n_max = torch.tensor([ids.numel()], device=dev)
        dist.all_reduce(n_max, op=dist.ReduceOp.MAX, group=group)
        n_max = int(n_max)
        mine = torch.full((n_max,), -1, dtype=torch.long, device=dev)
        mine[:ids.numel()] = sorted_ids
        everyone = torch.empty((world, n_max), dtype=torch.long, device=dev)
        dist.all_gather_into_tensor(everyone.view(-1), mine, group=group)
        lo = rank * per
        hit = (everyone >= lo) & (everyone < lo + x_local.shape[0])
        served = torch.zeros((world, n_max, f), dtype=x_local.dtype, device=dev)
        served[hit] = x_local[(everyone[hit] - lo)]
        # every rank needs the sum over owners of what was served for its own request list
        collected = torch.empty((world, world, n_max, f), dtype=x_local.dtype, device=dev)
        dist.all_gather_into_tensor(collected.view(-1), served.view(-1), group=group)
        got = collected[:, rank].sum(dim=0)[:ids.numel()]
    out = torch.empty((ids.numel(), f), dtype=x_local.dtype, device=dev)
    out[order] = got
    return out
