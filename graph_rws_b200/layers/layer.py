"""BCSRGraphConv and its autograd function (reference: layers/layer.py:28-191).

``BCSRSPMMFunction`` computes ``A @ (X @ W)`` with the forward SpMM kernel and, in backward,
``A^T @ dY`` with the same kernel on the graph's cached transposed BCSR (the reference scatters
with float atomics over the forward graph, layers/layer.py:71-77), followed by the two dense
products of layers/layer.py:86,90.  The layer itself is the reference's GraphSAGE-style
``A (X W_neigh) + X_target W_self`` (layers/layer.py:143-191).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.autograd import Function

from .. import core
from ..helper import record_spmm_time


def _spmm_graph(graph, dense):
    """A @ dense for a BCSRGraph, values cast (and cached) to the dense dtype, N padded to 8.

    A graph may bring its own product through a ``gather_dense`` hook: a row-sharded graph
    (parallel.RowShardedGraph) all-gathers the row shards of ``dense`` before its local product."""
    gather = getattr(graph, 'gather_dense', None)
    if gather is not None:
        dense = gather(dense)
    dense = dense.contiguous()
    vals = graph.values_as(dense.dtype)
    n = dense.shape[1]
    pad = (-n) % 8
    if pad:
        dense = F.pad(dense, (0, pad))
    planner = getattr(graph, 'spmm_plan', None)
    plan = planner(dense.shape[0], dense.shape[1]) if planner is not None else None
    out = core.spmm_raw(graph.window_offset, graph.original_col_indices, vals, dense, plan=plan)
    return out[:, :n] if pad else out


class BCSRSPMMFunction(Function):
    @staticmethod
    def forward(ctx, graph, features, weight, warps_per_block):
        x_mult_w = torch.matmul(features, weight)
        if core._timing_enabled and not hasattr(graph, 'gather_dense'):
            output, timing = core.spmm_tc(graph.window_offset, graph.original_col_indices,
                                          graph.values_as(x_mult_w.dtype), x_mult_w.contiguous(),
                                          warps_per_block)
        else:
            output, timing = _spmm_graph(graph, x_mult_w), 0.0
        record_spmm_time(timing)
        ctx.save_for_backward(features, weight)
        ctx.graph = graph
        ctx.warps_per_block = warps_per_block
        return output

    @staticmethod
    def backward(ctx, grad_output):
        features, weight = ctx.saved_tensors
        graph = ctx.graph
        num_input_nodes = features.shape[0]
        grad_output = grad_output.contiguous()
        g_t = graph.transposed(num_input_nodes, dtype=grad_output.dtype)
        grad_input_aggr = _spmm_graph(g_t, grad_output)[:num_input_nodes]
        grad_features = grad_weight = None
        if ctx.needs_input_grad[1]:
            grad_features = torch.matmul(grad_input_aggr, weight.t())
        if ctx.needs_input_grad[2]:
            grad_weight = torch.matmul(features.t(), grad_input_aggr)
        return None, grad_features, grad_weight, None


class BCSRAggregateFirstFunction(Function):
    """``(A @ X) @ W`` for an input ``X`` that needs no gradient (the features of the first layer).

    Same value as ``A @ (X @ W)`` (layers/layer.py:40-49 of the reference computes the latter, over
    every row of X), but the SpMM runs at the narrower width when ``in_feats <= out_feats``, and
    the backward pass needs no transposed product at all: ``dW = (A X)^T dY`` is one small GEMM over
    the layer's output rows.  For a sampled block this removes the largest transposed block of the
    step (as many rows as the hop has input nodes) and its construction."""

    @staticmethod
    def forward(ctx, graph, features, weight, warps_per_block):
        aggregated = _spmm_graph(graph, features)
        record_spmm_time(0.0)
        ctx.save_for_backward(aggregated, weight)
        return torch.matmul(aggregated, weight)

    @staticmethod
    def backward(ctx, grad_output):
        aggregated, weight = ctx.saved_tensors
        grad_weight = torch.matmul(aggregated.t(), grad_output) if ctx.needs_input_grad[2] else None
        return None, None, grad_weight, None


class BCSRGraphConv(nn.Module):
    """Aggregation only; activation, normalisation and dropout live in the model."""

    def __init__(self, in_feats: int, out_feats: int, dropout: float = 0.5, warps_per_block: int = 8):
        super().__init__()
        self.in_feats = in_feats
        self.out_feats = out_feats
        self.warps_per_block = warps_per_block
        self.weight_neigh = nn.Parameter(torch.empty(in_feats, out_feats))
        self.weight_self = nn.Parameter(torch.empty(in_feats, out_feats))
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.xavier_uniform_(self.weight_neigh)
        nn.init.xavier_uniform_(self.weight_self)

    def forward(self, graph, features: torch.Tensor, features_target: torch.Tensor = None) -> torch.Tensor:
        aggregate_first = (not features.requires_grad and features.shape[1] <= self.out_feats
                           and not hasattr(graph, 'gather_dense') and not core._timing_enabled)
        fn = BCSRAggregateFirstFunction if aggregate_first else BCSRSPMMFunction
        # An output width that is no multiple of 8 (41 or 47 classes) is computed at the next multiple
        # with zero weight columns and cut at the end: the SpMM needs 16-byte rows anyway, and the
        # GEMMs around it (X W, dY W^T, X^T dY) otherwise fall to unaligned library kernels several
        # times slower (0.46 ms instead of 0.07 ms each on 233 k rows x 256 -> 41).
        pad = (-self.out_feats) % 8
        w_neigh = F.pad(self.weight_neigh, (0, pad)) if pad else self.weight_neigh
        w_self = F.pad(self.weight_self, (0, pad)) if pad else self.weight_self
        h_neigh = fn.apply(graph, features, w_neigh, self.warps_per_block)
        target_rows = h_neigh.shape[0]
        if features_target is not None:
            h_in_self = features_target
        elif features.shape[0] >= target_rows:
            h_in_self = features[:target_rows]          # target nodes first
        else:
            h_in_self = F.pad(features, (0, 0, 0, target_rows - features.shape[0]))
        h_self = torch.matmul(h_in_self, w_self)
        # the SpMM returns whole windows (W*16 rows); trim or pad to the self path
        if h_neigh.shape[0] > h_self.shape[0]:
            h_neigh = h_neigh[:h_self.shape[0]]
        elif h_neigh.shape[0] < h_self.shape[0]:
            h_neigh = F.pad(h_neigh, (0, 0, 0, h_self.shape[0] - h_neigh.shape[0]))
        out = h_neigh + h_self
        return out[:, :self.out_feats] if pad else out
