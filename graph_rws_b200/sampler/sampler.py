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

The importance-score options (HACS, locality bonus; sampler.py:101-153) are not part of this
library.  The partition samplers (sampler.py:307-756: ``sample_partitions``, ``repack_subgraph``,
``sample_dps_online``) keep their signatures and the attributes of what they return.
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

    # ------------------------------------------------------------------ partition samplers
    # The reference's two partition-based mini-batch modes (sampler/sampler.py:307-756): a batch is
    # a set of whole 16-row windows of the full graph, taken with all their tiles, the column ids
    # relabelled to the batch's own node list.  Written here as a handful of device-wide tensor
    # operations (window -> tile ranges by a segmented arange, relabelling through one lookup
    # table) instead of per-partition host loops.

    def _gather_windows(self, g: BCSRGraph, window_ids: torch.Tensor):
        """Tiles of the given windows, in order: (new window_offset, cols [T, 8], vals [T, 16, 8] or None)."""
        dev = window_ids.device

        def at(src, idx):           # the graph's arrays may live in pinned host memory
            return src[idx.to(src.device)].to(dev) if src.device != idx.device else src[idx]
        starts, ends = at(g.window_offset, window_ids), at(g.window_offset, window_ids + 1)
        lengths = ends - starts
        new_wo = torch.zeros(window_ids.numel() + 1, dtype=torch.int64, device=dev)
        torch.cumsum(lengths, 0, out=new_wo[1:])
        total = int(new_wo[-1])                                   # the one size read-back of a batch
        owner = torch.repeat_interleave(torch.arange(window_ids.numel(), device=dev), lengths, output_size=total)
        tile_idx = starts[owner] + (torch.arange(total, device=dev) - new_wo[owner])
        cols = at(g.original_col_indices.view(-1, self.tile_cols), tile_idx)
        vals = None
        if g.values_condensed is not None:
            vals = at(g.values_condensed.view(-1, self.tile_rows, self.tile_cols), tile_idx)
        return new_wo, cols, vals

    def sample_partitions(self, g: BCSRGraph, partition_ids: torch.Tensor) -> BCSRGraph:
        """The sub-BCSR induced by whole partitions of ``partition_book`` (entries with ``start_idx`` /
        ``end_idx`` node ranges on window boundaries): rows and columns are the partitions' nodes,
        numbered in the order the partitions are given; edges that leave the selection keep a -1
        column id and contribute nothing (sampler/sampler.py:307-410)."""
        if self.partition_book is None:
            raise ValueError("Partition book is missing! Please set sampler.partition_book.")
        dev = partition_ids.device
        parts = [self.partition_book[int(p)] for p in partition_ids.tolist()]
        lo = torch.tensor([p['start_idx'] for p in parts], dtype=torch.int64, device=dev)
        hi = torch.tensor([p['end_idx'] for p in parts], dtype=torch.int64, device=dev)
        sizes = hi - lo
        first_local = torch.cumsum(sizes, 0) - sizes
        n_local = int(sizes.sum())
        part_of = torch.repeat_interleave(torch.arange(len(parts), device=dev), sizes, output_size=n_local)
        nodes = lo[part_of] + (torch.arange(n_local, device=dev) - first_local[part_of])        # global id of local node i
        node_map = torch.full((g.num_nodes,), -1, dtype=torch.int32, device=dev)
        node_map[nodes] = torch.arange(n_local, dtype=torch.int32, device=dev)
        w_lo, w_hi = lo // self.tile_rows, hi // self.tile_rows
        w_sizes = w_hi - w_lo
        w_first = torch.cumsum(w_sizes, 0) - w_sizes
        n_win = int(w_sizes.sum())
        wp = torch.repeat_interleave(torch.arange(len(parts), device=dev), w_sizes, output_size=n_win)
        window_ids = w_lo[wp] + (torch.arange(n_win, device=dev) - w_first[wp])
        new_wo, cols, vals = self._gather_windows(g, window_ids)
        valid = (cols >= 0) & (cols < g.num_nodes)
        local = torch.where(valid, node_map[cols.clamp(0, g.num_nodes - 1).long()], torch.full_like(cols, -1))
        if vals is not None:
            vals = vals.clone()
            vals.masked_fill_((local < 0).unsqueeze(1), 0.0)
        sub = BCSRGraph.from_components(new_wo, local.reshape(-1).contiguous(),
                                        vals.reshape(-1) if vals is not None else None, num_rows=n_local,
                                        num_cols=n_local, tile_rows=self.tile_rows, tile_cols=self.tile_cols, device=dev)
        sub.active_windows = torch.arange(n_win, device=dev, dtype=torch.int32)
        sub.is_local_input = True
        return sub

    def repack_subgraph(self, g: BCSRGraph, window_ids: torch.Tensor, max_external_ratio: float = 5.0,
                        dry_run: bool = False):
        """Halo-aware batch: the rows are the nodes of ``window_ids`` ("internal"), the columns are the
        internal nodes followed by the neighbours outside them ("halo", at most
        ``max_external_ratio`` x internal, a random subset beyond that); ``inner_graph`` is the same
        block with the halo edges masked, for the layers after the first
        (sampler/sampler.py:413-690)."""
        from types import SimpleNamespace
        dev = window_ids.device
        window_ids = torch.sort(window_ids).values
        window_ids = window_ids[(window_ids >= 0) & (window_ids < g.num_windows)]
        R = self.tile_rows
        if dry_run:                                               # sizes only, nothing is gathered
            wo = g.window_offset
            idx = window_ids.to(wo.device)
            total_tiles = int((wo[idx + 1] - wo[idx]).sum()) if idx.numel() else 0
            return SimpleNamespace(original_window_ids=window_ids, num_internal_nodes=window_ids.numel() * R,
                                   total_tiles=total_tiles, approx_values=total_tiles * R * self.tile_cols,
                                   approx_cols=total_tiles * self.tile_cols, values_condensed=None,
                                   original_col_indices=None)
        new_wo, cols, vals = self._gather_windows(g, window_ids)
        internal = (window_ids.unsqueeze(1) * R + torch.arange(R, device=dev).unsqueeze(0)).reshape(-1)
        internal = internal[internal < g.num_nodes]
        n_int = int(internal.numel())
        lookup = torch.full((g.num_nodes,), -1, dtype=torch.int32, device=dev)       # global id -> local id
        lookup[internal] = torch.arange(n_int, dtype=torch.int32, device=dev)
        valid = (cols >= 0) & (cols < g.num_nodes)
        safe = cols.clamp(0, max(g.num_nodes - 1, 0)).long()
        outside = valid & (lookup[safe] < 0)
        halo = torch.unique(cols[outside].long())                 # ascending
        budget = int(n_int * max_external_ratio)
        if halo.numel() > budget:                                 # the out-of-memory guard of the reference
            halo = torch.sort(halo[torch.randperm(halo.numel(), device=dev)[:budget]]).values
        lookup[halo] = torch.arange(n_int, n_int + halo.numel(), dtype=torch.int32, device=dev)
        input_nodes = torch.cat([internal, halo])
        local = torch.where(valid, lookup[safe], torch.full_like(cols, -1))
        if vals is not None:
            vals = vals.clone()
            vals.masked_fill_((local < 0).unsqueeze(1), 0.0)
            vals.nan_to_num_(0.0)
        sub = BCSRGraph.from_components(new_wo, local.reshape(-1).contiguous(),
                                        vals.reshape(-1) if vals is not None else None, num_rows=n_int,
                                        num_cols=int(input_nodes.numel()), tile_rows=R, tile_cols=self.tile_cols, device=dev)
        sub.original_node_ids = input_nodes
        sub.original_window_ids = window_ids
        sub.is_local_input = True
        sub.num_internal_nodes = n_int
        inner_cols = torch.where(local >= n_int, torch.full_like(local, -1), local)
        inner_vals = None
        if vals is not None:
            inner_vals = vals.clone()
            inner_vals.masked_fill_((inner_cols < 0).unsqueeze(1), 0.0)
        sub.inner_graph = BCSRGraph.from_components(new_wo, inner_cols.reshape(-1).contiguous(),
                                                    inner_vals.reshape(-1) if inner_vals is not None else None,
                                                    num_rows=n_int, num_cols=n_int, tile_rows=R,
                                                    tile_cols=self.tile_cols, device=dev)
        return sub

    def sample_dps_online(self, g: BCSRGraph, seed_window_ids: torch.Tensor, fanouts: List[int] = [5, 5],
                          dry_run: bool = False):
        """Probe + repack (sampler/sampler.py:693-756): sample from the nodes of the seed windows,
        take every window the sampled hops touch, and repack those windows as one halo-aware batch."""
        dev = seed_window_ids.device
        R = self.tile_rows
        seeds = (seed_window_ids.unsqueeze(1) * R + torch.arange(R, device=dev).unsqueeze(0)).reshape(-1)
        seeds = seeds[seeds < g.num_nodes]
        if seeds.numel() == 0:
            return self.repack_subgraph(g, torch.empty(0, dtype=torch.long, device=dev), dry_run=dry_run)
        probe = BCSRSampler(fanouts, self.tile_rows, self.tile_cols, self.warps_per_block, verbose=False,
                            seed=self.seed, fused=True)
        probe.step = self.step
        touched = [seed_window_ids.to(torch.int64)]
        for block in probe.sample_layers(g, seeds):
            ids = block.input_nodes
            touched.append(torch.div(ids[ids >= 0], R, rounding_mode='floor').to(torch.int64))
        windows = torch.unique(torch.cat(touched))
        windows = windows[(windows >= 0) & (windows < g.num_windows)]
        return self.repack_subgraph(g, windows, dry_run=dry_run)
