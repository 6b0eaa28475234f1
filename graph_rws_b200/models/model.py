"""GCN_BCSR with the reference's constructor, parameter names and forward contract
(models/model.py:13-285): a stack of BCSRGraphConv layers with LayerNorm, optional residual
projections, dropout and activation checkpointing.  Checkpoints interchange with the reference
(``layers.N.weight_neigh / weight_self``, ``norms.N.*``, ``residual_projs.N.weight``).

Graph handling per layer follows models/model.py:96-210:
  * a graph flagged ``is_local_input`` is used as is;
  * layer 0 of a global-id graph gets out-of-range / -1 column ids masked (ids -> 0, their value
    columns -> 0).  The reference repeats those three full-array passes on every forward
    (models/model.py:118-125); here the result is remembered per graph and feature count;
  * layers > 0 whose previous graph carries ``active_windows`` get their column ids localised by
    ``reindex_bcsr``;
  * a row shard of a full graph (parallel.RowShardedGraph) keeps its global column ids; the
    layer all-gathers the feature rows of all ranks before the product;
  * the rows fed to the self path are gathered by window when ``active_windows`` exist, by the
    block's ``self_rows`` index when its columns are global ids, else the target-first slice
    ``h[:target_rows]`` (what per-seed sampled blocks use).
"""
import copy
from typing import List, Union

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .. import core
from ..data import BCSRGraph
from ..layers import BCSRGraphConv
from ..layers.norm import act_layer_norm

_ACTIVATIONS = {'relu': F.relu, 'elu': F.elu, 'gelu': F.gelu}


class GCN_BCSR(nn.Module):
    def __init__(self, in_feats: int, hidden_size: int, num_classes: int, num_layers: int,
                 dropout: float = 0.5, activation: str = 'relu', residual: bool = False,
                 warps_per_block: int = 8, use_checkpoint: bool = True):
        super().__init__()
        assert num_layers >= 2, "num_layers must be >= 2"
        if activation not in _ACTIVATIONS:
            raise ValueError(f"Unsupported activation: {activation}")
        self.in_feats, self.hidden_size, self.num_classes = in_feats, hidden_size, num_classes
        self.num_layers, self.dropout, self.residual = num_layers, dropout, residual
        self.warps_per_block, self.use_checkpoint = warps_per_block, use_checkpoint
        self.activation = _ACTIVATIONS[activation]

        dims = [in_feats] + [hidden_size] * (num_layers - 1) + [num_classes]
        self.layers = nn.ModuleList(
            BCSRGraphConv(dims[i], dims[i + 1], warps_per_block=warps_per_block) for i in range(num_layers))
        self.dropout_layer = nn.Dropout(dropout) if dropout > 0 else None
        self.norms = nn.ModuleList(nn.LayerNorm(hidden_size) for _ in range(num_layers - 1))
        if residual:
            self.residual_projs = nn.ModuleList(
                nn.Linear(dims[i], hidden_size, bias=False) if dims[i] != hidden_size else None
                for i in range(num_layers - 1))
        else:
            self.residual_projs = None
        self._init_parameters()

    def _init_parameters(self):
        for layer in self.layers:
            layer.reset_parameters()
        if self.residual_projs is not None:
            for proj in self.residual_projs:
                if proj is not None:
                    nn.init.kaiming_uniform_(proj.weight, nonlinearity='relu')
        for norm in self.norms:
            norm.reset_parameters()

    def _ensure_graph_list(self, graphs: Union[BCSRGraph, List[BCSRGraph]]) -> List[BCSRGraph]:
        if isinstance(graphs, BCSRGraph) or hasattr(graphs, 'gather_dense'):
            # independent wrappers so that per-layer metadata edits do not leak between layers
            return [copy.copy(graphs) for _ in range(len(self.layers))]
        if isinstance(graphs, list):
            assert len(graphs) == len(self.layers)
            return graphs
        raise TypeError(f"graphs must be BCSRGraph or List[BCSRGraph], got {type(graphs)}")

    @staticmethod
    def _sanitize_layer0(g, num_src: int):
        shared = getattr(g, '_shared', None)
        key = ('sanitized', num_src)
        state = (g.original_col_indices.data_ptr(), g.values_condensed.data_ptr())
        if shared is not None and shared.get(key) == state:
            return
        cols = g.original_col_indices
        bad = (cols == -1) | (cols >= num_src)
        cols.masked_fill_(bad, 0)
        vals = g.values_condensed.view(-1, g.tile_rows, g.tile_cols)
        vals.masked_fill_(bad.view(-1, 1, g.tile_cols), 0.0)
        if shared is not None:
            shared[key] = state

    def _sanitize_and_reindex(self, layer_idx, curr_g, prev_g, h_in_shape):
        if hasattr(curr_g, 'gather_dense'):
            return          # row shard of a square graph: global column ids, rows gathered before the product
        if getattr(curr_g, 'is_local_input', False):
            curr_g.num_cols = h_in_shape[0]
            return
        fwd_g = curr_g.fwd if hasattr(curr_g, 'fwd') else curr_g
        if layer_idx == 0:
            if hasattr(fwd_g, 'original_col_indices'):
                self._sanitize_layer0(fwd_g, h_in_shape[0])
        else:
            if getattr(prev_g, 'active_windows', None) is not None:
                fwd_g.original_col_indices = core.reindex_bcsr(
                    fwd_g.original_col_indices, fwd_g.values_condensed, prev_g.active_windows,
                    fwd_g.tile_rows, fwd_g.tile_cols)
            fwd_g.num_cols = h_in_shape[0]

    def _get_residual(self, layer_idx, curr_g, prev_g, h_in, target_rows):
        """Rows of ``h_in`` aligned with the layer's output rows (models/model.py:145-210)."""
        self_rows = getattr(curr_g, 'self_rows', None)
        if layer_idx == 0 and self_rows is not None:
            return h_in[self_rows]          # a block whose columns are global ids names its own rows
        if h_in.shape[0] == target_rows:
            return h_in
        device = h_in.device
        curr_wins = getattr(curr_g, 'active_windows', None)
        if layer_idx == 0:
            if getattr(curr_g, 'is_local_input', False):
                return torch.zeros((target_rows, h_in.shape[1]), device=device, dtype=h_in.dtype)
            if curr_wins is not None:
                t_rows = curr_g.tile_rows
                idx = (curr_wins.unsqueeze(1) * t_rows + torch.arange(t_rows, device=device).unsqueeze(0)).view(-1)
                valid = idx < h_in.shape[0]
                res = h_in[torch.where(valid, idx, torch.zeros_like(idx))]
                res.masked_fill_((~valid).unsqueeze(1), 0.0)
                return res
        elif curr_wins is not None:
            t_rows = curr_g.tile_rows
            prev_wins = prev_g.active_windows
            win_idx = torch.searchsorted(prev_wins, curr_wins).clamp_(0, max(0, prev_wins.size(0) - 1))
            idx = (win_idx.unsqueeze(1) * t_rows + torch.arange(t_rows, device=device).unsqueeze(0)).view(-1)
            return h_in[idx]
        if target_rows > h_in.shape[0]:
            return F.pad(h_in, (0, 0, 0, target_rows - h_in.shape[0]))
        return h_in[:target_rows]          # target nodes come first

    def forward(self, graphs: Union[BCSRGraph, List[BCSRGraph]], features: torch.Tensor) -> torch.Tensor:
        if features.device.type != 'cuda':
            features = features.to('cuda', non_blocking=True)
        graph_list = self._ensure_graph_list(graphs)
        h = features
        for l, (layer, g) in enumerate(zip(self.layers, graph_list)):
            prev_g = graph_list[l - 1] if l > 0 else None
            self._sanitize_and_reindex(l, g, prev_g, h.shape)     # edits the graph: outside checkpoint
            h_target = self._get_residual(l, g, prev_g, h, g.num_rows)

            def run_curr_layer(h_curr, layer=layer, g=g, h_tgt=h_target):
                return layer(g, h_curr, features_target=h_tgt)

            if self.use_checkpoint and self.training and h.requires_grad:
                h_out = checkpoint(run_curr_layer, h, use_reentrant=False)
            else:
                h_out = run_curr_layer(h)

            if self.residual and l < len(self.layers) - 1:
                h_res = h
                if self.residual_projs is not None and self.residual_projs[l] is not None:
                    h_res = self.residual_projs[l](h_res)
                h_out = h_out + self._get_residual(l, g, prev_g, h_res, h_out.shape[0])
            h = h_out
            if l < len(self.layers) - 1:
                if self.norms:
                    # activation and normalisation in one pass over the rows when the activation is ReLU
                    relu = self.activation is F.relu
                    h = act_layer_norm(h if relu else self.activation(h), self.norms[l], relu)
                else:
                    h = self.activation(h)
                if self.dropout_layer is not None:
                    h = self.dropout_layer(h)
        return h

    def inference(self, graph: BCSRGraph, features: torch.Tensor, batch_size: int = 0) -> torch.Tensor:
        if features.device.type != 'cuda':
            features = features.to('cuda', non_blocking=True)
        h = features
        g_copy = copy.copy(graph)
        self._sanitize_and_reindex(0, g_copy, None, h.shape)
        for l, layer in enumerate(self.layers):
            h = layer(g_copy, h)
            if l < len(self.layers) - 1:
                if self.norms:
                    relu = self.activation is F.relu
                    h = act_layer_norm(h if relu else self.activation(h), self.norms[l], relu)
                else:
                    h = self.activation(h)
        return h
