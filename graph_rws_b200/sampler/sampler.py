"""BCSRSampler with the reference's constructor and ``sample_layers`` contract
(sampler/sampler.py:32-279): a full ``BCSRGraph`` and seed nodes in, one ``BCSRGraph`` per model
layer out, input layer first.

What differs, on purpose: the reference picks, per 16-row window, the top-K columns by edge weight
(a deterministic choice) and returns whole windows with global column ids plus ``active_windows``;
here every frontier node draws ``fanout`` neighbours uniformly without replacement from a
counter-based Philox stream keyed by (seed, node, hop), and each hop is a compact block:
rows = the hop's destination nodes (``output_nodes``), columns = positions in ``input_nodes``,
whose first ``num_rows`` entries are the destination nodes themselves.  ``GCN_BCSR`` consumes such
blocks through its target-first slicing path; the features to pass are ``X[blocks[0].input_nodes]``
and the logits rows line up with the seeds.  Edge values are the graph's own weights (the
reference does not renormalise sampled blocks either).

The importance-score options (HACS, locality bonus; sampler.py:101-153) and the partition
samplers (sampler.py:307-756) are not part of this library.
"""
from typing import List

import torch

from .. import core
from ..data import BCSRGraph, CSRTopology


class BCSRSampler:
    def __init__(self,
                 fanouts: List[int],
                 tile_rows: int = 16,
                 tile_cols: int = 8,
                 warps_per_block: int = 8,
                 partition_book: list = None,
                 verbose: bool = True,
                 static_scores: torch.Tensor = None,
                 window_part_ids: torch.Tensor = None,
                 part_ranges: torch.Tensor = None,
                 hacs_enabled: bool = False,
                 alpha: float = 1.0,
                 beta: float = 10.0,
                 delta: float = 0.0,
                 gamma_bonus: float = 0.0,
                 score_scale: float = 100.0,
                 locality_enabled: bool = False,
                 seed: int = core.sampling.DEFAULT_SEED,
                 pad_to: int = 0,
                 fused: bool = None):
        if hacs_enabled or locality_enabled:
            raise ValueError("importance-score sampling is not part of this library; sampling is uniform")
        if tile_rows != 16 or tile_cols != 8:
            raise ValueError("Currently only supports tile 16x8")
        self.fanouts = list(fanouts)
        self.tile_rows = tile_rows
        self.tile_cols = tile_cols
        self.warps_per_block = warps_per_block
        self.partition_book = partition_book
        self.verbose = verbose
        self.time_tracker = {}
        self.seed = int(seed)
        # > 0: every hop's node list is padded with -1 entries to a multiple of this, so that the
        # dense products of a training step see recurring shapes (input_nodes then contains -1s)
        self.pad_to = int(pad_to)
        self.step = 0          # callers may bump this to decorrelate epochs: the stream key is seed + step
        # fused: all hops in one library call, buffers sized by bounds, no size read-back (the
        # blocks then have the sizes of core.sample_layers_sizes, their unused tails hold -1
        # nodes).  Default: fused unless per-phase timings are wanted (``verbose``), which need
        # a host synchronisation per phase anyway.
        self.fused = (not verbose) if fused is None else bool(fused)

    @staticmethod
    def _to_cuda_int(x, device=None) -> torch.Tensor:
        if not isinstance(x, torch.Tensor):
            x = torch.tensor(x)
        if device is None:
            device = torch.device('cuda')
        return x.to(device=device, dtype=torch.int32, non_blocking=True).contiguous()

    @staticmethod
    def graph_csr(g: BCSRGraph):
        """CSR view of the full graph, extracted on the device once and cached on the graph."""
        hit = g._shared.get('csr')
        state = (g.original_col_indices.data_ptr(), g.values_condensed.data_ptr(),
                 g.original_col_indices._version, g.values_condensed._version)
        if hit is not None and hit[0] == state:
            return hit[1]
        csr = core.bcsr_to_csr(g.window_offset, g.original_col_indices, g.values_condensed, g.num_rows)
        g._shared['csr'] = (state, csr)
        return csr

    def sample_layers(self, g, seed_nodes: torch.Tensor, seed_dev: torch.Tensor = None) -> List[BCSRGraph]:
        """``g`` is the full graph: a ``BCSRGraph`` (its CSR view is extracted once and cached) or a
        ``CSRTopology`` (no BCSR of the whole graph is ever built).  ``seed_dev``: optional device
        uint64 tensor holding the Philox seed (fused path only), for step loops that replay one
        captured launch sequence with a new seed each time."""
        if isinstance(g, CSRTopology):
            device = g.device
            row_ptr, col_idx, values = g.csr()
            block_dtype = g.block_dtype
        else:
            device = g.window_offset.device if g.window_offset.is_cuda else torch.device('cuda')
            row_ptr, col_idx, values = self.graph_csr(g)
            block_dtype = g.values_condensed.dtype
        seed_nodes = self._to_cuda_int(seed_nodes, device=device)
        # model layers run input -> output, sampling runs from the seeds outwards (sampler.py:200-204)
        reversed_fanouts = list(reversed(self.fanouts))
        if self.fused:
            hops = core.sample_layers_fused(row_ptr, col_idx, values, seed_nodes, reversed_fanouts,
                                            seed=self.seed + self.step, values_dtype=block_dtype,
                                            pad_to=self.pad_to, seed_dev=seed_dev)
            timing_list = []
        else:
            hops, timing_list = core.sample_layers_csr(row_ptr, col_idx, values, seed_nodes, reversed_fanouts,
                                                       seed=self.seed + self.step,
                                                       values_dtype=block_dtype, timing=self.verbose,
                                                       pad_to=self.pad_to, exact=False)
        if self.verbose:
            num_layers = len(self.fanouts)
            for i, t in enumerate(timing_list):
                stats = self.time_tracker.setdefault((num_layers - 1) - i, {
                    'count': 0, 'p1_sample': 0.0, 'p2_map': 0.0, 'p3_recomp': 0.0, 'total': 0.0})
                stats['count'] += 1
                stats['p1_sample'] += t.phase1_sampling_time
                stats['p2_map'] += t.phase2_mapping_time
                stats['p3_recomp'] += t.phase3_recompression_time
                stats['total'] += t.total_time
        layers: List[BCSRGraph] = []
        for (wo, cols, vals, dst, src), fanout in zip(hops, reversed_fanouts):
            sub = BCSRGraph.from_components(wo, cols, vals, num_rows=dst.numel(), num_cols=src.numel(),
                                            tile_rows=self.tile_rows, tile_cols=self.tile_cols, device=wo.device)
            sub.nnz_bound = dst.numel() * fanout   # lets the transposed block be built without a read-back
            sub.output_nodes = dst          # global ids of the block's rows
            sub.input_nodes = src           # global ids of the block's columns; starts with output_nodes
            sub.transient = True            # lives for one step: its arrays and its transposed graph skip exact sizing
            layers.insert(0, sub)           # keep input -> output order
        return layers

    def __repr__(self):
        return (f"BCSRSampler(fanouts={self.fanouts}, tile={self.tile_rows}x{self.tile_cols}, "
                f"warps_per_block={self.warps_per_block}, seed={self.seed:#x})")

    def print_avg_timing(self):
        print("\n" + "-" * 60 + "\n [Average Sampling Performance Summary]\n" + "-" * 60)
        for layer_id in sorted(self.time_tracker):
            s = self.time_tracker[layer_id]
            c = max(s['count'], 1)
            print(f"  layer {layer_id}: sample {s['p1_sample'] / c:8.3f} ms  dedup/reindex {s['p2_map'] / c:8.3f} ms  "
                  f"block build {s['p3_recomp'] / c:8.3f} ms  total {s['total'] / c:8.3f} ms")

    def sample_partitions(self, *args, **kwargs):
        raise NotImplementedError("partition samplers are outside this library's scope")
