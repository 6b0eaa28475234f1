"""Sampling operators over the C ABI: BCSR -> CSR, one sampling hop, dedup / reindex, block build,
and the reference-named ``sample_all_layers`` / ``reindex_bcsr``."""
import time

import torch

from . import _native

_DT = {torch.float32: _native.F32, torch.float16: _native.F16, torch.bfloat16: _native.BF16}
DEFAULT_SEED = 0x5EED


def _ptr(t):
    return 0 if t is None or t.numel() == 0 else t.data_ptr()


def _stream(device):
    return torch.cuda.current_stream(device).cuda_stream


def _scratch(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def bcsr_to_csr(window_offset, cols, vals, num_rows):
    """CSR (row_ptr i64, col_idx i32, values f32) of a BCSR matrix, rows ascending in column id."""
    lib = _native.lib()
    dev = vals.device
    W = window_offset.shape[0] - 1
    st = _stream(dev)
    row_ptr = torch.empty(num_rows + 1, dtype=torch.int64, device=dev)
    scratch = _scratch(lib.grws_bcsr_to_csr_scratch_bytes(num_rows), dev)
    _native.check(lib.grws_bcsr_to_csr_count(_ptr(window_offset), _ptr(cols), _ptr(vals), _DT[vals.dtype], W,
                                             num_rows, row_ptr.data_ptr(), scratch.data_ptr(), scratch.numel(), st))
    nnz = int(row_ptr[-1].item())
    col_idx = torch.empty(nnz, dtype=torch.int32, device=dev)
    values = torch.empty(nnz, dtype=torch.float32, device=dev)
    _native.check(lib.grws_bcsr_to_csr_fill(_ptr(window_offset), _ptr(cols), _ptr(vals), _DT[vals.dtype], W,
                                            num_rows, row_ptr.data_ptr(), _ptr(col_idx), _ptr(values), st))
    return row_ptr, col_idx, values


def sample_hop(row_ptr, col_idx, values, nodes, fanout, seed=DEFAULT_SEED, hop=0):
    """(nbr i32 [n, fanout] with -1 padding, w f32 [n, fanout], cnt i32 [n]) for int32 ``nodes``."""
    lib = _native.lib()
    dev = nodes.device
    n = nodes.numel()
    nbr = torch.empty((n, fanout), dtype=torch.int32, device=dev)
    w = torch.empty((n, fanout), dtype=torch.float32, device=dev)
    cnt = torch.empty(n, dtype=torch.int32, device=dev)
    _native.check(lib.grws_sample_hop(_ptr(row_ptr), _ptr(col_idx), _ptr(values), _ptr(nodes), n, int(fanout),
                                      int(seed) & 0xFFFFFFFFFFFFFFFF, int(hop), _ptr(nbr), _ptr(w), _ptr(cnt),
                                      _stream(dev)))
    return nbr, w, cnt


def build_block(dst, nbr, w, values_dtype=torch.float32, _marks=None, exact=True):
    """Dedup + reindex + BCSR build of one hop.

    Returns (src i32 [n_src], window_offset, cols, vals): rows are the ``dst`` nodes in order,
    columns are positions in ``src`` = dst ++ ascending new nodes.  ``exact=False`` saves the
    read-back of the tile count (see ``csr_to_bcsr``): cols / vals then end in unused tiles."""
    from . import csr_to_bcsr
    lib = _native.lib()
    dev = dst.device
    n_dst = dst.numel()
    fanout = nbr.shape[1]
    st = _stream(dev)
    src = torch.empty(n_dst + n_dst * fanout, dtype=torch.int32, device=dev)
    local = torch.empty((n_dst, fanout), dtype=torch.int32, device=dev)
    row_ptr = torch.empty(n_dst + 1, dtype=torch.int64, device=dev)
    counts = torch.empty(2, dtype=torch.int64, device=dev)
    scratch = _scratch(lib.grws_dedup_scratch_bytes(n_dst, fanout), dev)
    _native.check(lib.grws_dedup_reindex(_ptr(dst), n_dst, _ptr(nbr), fanout, src.data_ptr(), _ptr(local),
                                         row_ptr.data_ptr(), counts.data_ptr(), scratch.data_ptr(),
                                         scratch.numel(), st))
    n_src, n_edges = (int(x) for x in counts.tolist())          # size read-back of the hop
    if _marks is not None:
        _marks.append(time.perf_counter())
    col = torch.empty(n_edges, dtype=torch.int32, device=dev)
    val = torch.empty(n_edges, dtype=torch.float32, device=dev)
    _native.check(lib.grws_block_compact(_ptr(local), _ptr(w), n_dst, fanout, row_ptr.data_ptr(), _ptr(col),
                                         _ptr(val), st))
    wo, cols, vals = csr_to_bcsr(n_dst, row_ptr, col, val, values_dtype=values_dtype, exact=exact)
    return src[:n_src], wo, cols, vals


class SamplingTimingResult:
    """Attribute-compatible with the reference's timing object (core/wrapper/bind.cpp:81-96);
    phase 1 = sampling, phase 2 = dedup / reindex, phase 3 = BCSR block build, in milliseconds
    of host wall time (each phase ends with a size read-back, so it covers the device work)."""

    def __init__(self, p1=0.0, p2=0.0, p3=0.0):
        self.phase1_sampling_time = p1
        self.phase2_mapping_time = p2
        self.phase3_recompression_time = p3
        self.total_time = p1 + p2 + p3

    def to_dict(self):
        return {"phase1_sampling_time": self.phase1_sampling_time, "phase2_mapping_time": self.phase2_mapping_time,
                "phase3_recompression_time": self.phase3_recompression_time, "total_time": self.total_time}

    def __repr__(self):
        return (f"<SamplingTimingResult total={self.total_time:.2f}ms (P1={self.phase1_sampling_time:.2f}, "
                f"P2={self.phase2_mapping_time:.2f}, P3={self.phase3_recompression_time:.2f})>")


def sample_layers_csr(row_ptr, col_idx, values, seeds, fanouts, seed=DEFAULT_SEED, values_dtype=torch.float32,
                      timing=False, pad_to=0, exact=True):
    """Multi-hop sampling over a CSR graph.  ``fanouts`` are consumed in the order given (the caller
    passes them output layer first, like sampler/sampler.py:202-204).  Returns one
    [window_offset, cols, vals, dst_nodes, src_nodes] list per hop and one timing object per hop.

    ``pad_to`` > 0 rounds every hop's source list up to a multiple of ``pad_to`` with -1 entries
    (nodes without neighbours that nothing refers to), so that the dense products of the training
    step see a small set of recurring shapes instead of a new one every step."""
    out, timings = [], []
    dst = seeds.to(torch.int32).contiguous()
    dev = dst.device
    for hop, f in enumerate(fanouts):
        t0 = time.perf_counter()
        nbr, w, _ = sample_hop(row_ptr, col_idx, values, dst, int(f), seed, hop)
        if timing:
            torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        marks = []
        src, wo, cols, vals = build_block(dst, nbr, w, values_dtype=values_dtype, _marks=marks, exact=exact)
        t3 = time.perf_counter()
        if pad_to > 0 and src.numel() % pad_to:
            pad = pad_to - src.numel() % pad_to
            src = torch.cat([src, torch.full((pad,), -1, dtype=torch.int32, device=dev)])
        out.append([wo, cols, vals, dst, src])
        timings.append(SamplingTimingResult((t1 - t0) * 1e3, (marks[0] - t1) * 1e3, (t3 - marks[0]) * 1e3))
        dst = src
    return out, timings


def sample_layers_sizes(num_seeds, fanouts, pad_to=0):
    """(n_dst, n_src, tiles_bound) per hop of ``sample_layers_fused``: the sizes every buffer of a
    mini-batch gets, known from the seed count and the fanouts alone."""
    import ctypes
    lib = _native.lib()
    L = len(fanouts)
    fan = (ctypes.c_int * L)(*[int(f) for f in fanouts])
    a, b, c = ((ctypes.c_int64 * L)() for _ in range(3))
    _native.check(lib.grws_sample_layers_sizes(int(num_seeds), fan, L, int(pad_to), a, b, c))
    return list(a), list(b), list(c)


def sample_layers_fused(row_ptr, col_idx, values, seeds, fanouts, seed=DEFAULT_SEED, values_dtype=torch.float32,
                        pad_to=0, seed_dev=None, want_counts=False):
    """All hops of a mini-batch in ONE library call and without any size read-back.

    Same sampling, dedup and block layout as ``sample_layers_csr``; what differs is the sizing: every
    hop's arrays have the bound sizes of ``sample_layers_sizes`` (the frontier of hop h+1 is the
    whole source list of hop h, its unused tail filled with -1 nodes that sample nothing), so the
    shapes of a step depend only on (number of seeds, fanouts) and recur from step to step.  The
    call queues about twenty kernels per hop on the current stream and returns; ctypes releases the
    interpreter lock for its duration, so a sampling thread does not hold up the training thread.

    Returns one [window_offset, cols, vals, dst_nodes, src_nodes] list per hop (fanouts in the order
    given) and, with ``want_counts``, an int64 [hops, 4] device tensor {source nodes, sampled edges,
    tiles, real frontier nodes} per hop."""
    import ctypes
    lib = _native.lib()
    dev = row_ptr.device
    seeds = seeds.to(device=dev, dtype=torch.int32).contiguous()
    L = len(fanouts)
    n_dst, n_src, tiles = sample_layers_sizes(seeds.numel(), fanouts, pad_to)
    fan = (ctypes.c_int * L)(*[int(f) for f in fanouts])
    vsize = torch.empty((), dtype=values_dtype).element_size()
    # one allocation for all int32 outputs, one for the values, one for the offsets, one for scratch
    i32_sizes = [n for h in range(L) for n in (n_src[h], tiles[h] * 8)]
    i32 = torch.empty(sum(-(-n // 64) * 64 for n in i32_sizes) + 64, dtype=torch.int32, device=dev)
    vals_all = torch.empty(sum(t * 128 for t in tiles) + 8, dtype=values_dtype, device=dev)
    wo_sizes = [(n + 15) // 16 + 1 for n in n_dst]
    wo_all = torch.empty(sum(-(-n // 32) * 32 for n in wo_sizes) + 4 * L, dtype=torch.int64, device=dev)
    scratch = _scratch(lib.grws_sample_layers_scratch_bytes(seeds.numel(), fan, L, int(pad_to)), dev)
    srcs, cols, vals, wos = [], [], [], []
    o32 = ov = ow = 0
    for h in range(L):
        srcs.append(i32[o32:o32 + n_src[h]]); o32 += -(-n_src[h] // 64) * 64
        cols.append(i32[o32:o32 + tiles[h] * 8]); o32 += -(-(tiles[h] * 8) // 64) * 64
        vals.append(vals_all[ov:ov + tiles[h] * 128]); ov += tiles[h] * 128
        wos.append(wo_all[ow:ow + wo_sizes[h]]); ow += -(-wo_sizes[h] // 32) * 32
    counts = wo_all[ow:ow + 4 * L].view(L, 4) if want_counts else None
    ptrs = lambda ts: (ctypes.c_void_p * L)(*[t.data_ptr() for t in ts])      # noqa: E731
    _native.check(lib.grws_sample_layers(
        _ptr(row_ptr), _ptr(col_idx), _ptr(values), _ptr(seeds), seeds.numel(), fan, L,
        int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(seed_dev), int(pad_to), _DT[values_dtype],
        ptrs(srcs), ptrs(wos), ptrs(cols), ptrs(vals), _ptr(counts) if want_counts else 0,
        scratch.data_ptr(), scratch.numel(), _stream(dev)))
    out, dst = [], seeds
    for h in range(L):
        out.append([wos[h], cols[h], vals[h], dst, srcs[h]])
        dst = srcs[h]
    return (out, counts) if want_counts else out


class _CsrCache:
    """CSR views of the BCSR graphs recently passed to ``sample_all_layers`` (keyed on tensor
    identity and version; entries keep the tensors alive so storage cannot be recycled)."""

    def __init__(self, capacity=4):
        self.capacity, self.entries = capacity, []

    def get(self, wo, cols, vals, num_rows):
        key = (wo.data_ptr(), cols.data_ptr(), vals.data_ptr(), cols._version, vals._version, wo.numel(),
               cols.numel(), int(num_rows))
        for i, (k, _, value) in enumerate(self.entries):
            if k == key:
                self.entries.append(self.entries.pop(i))
                return value
        value = bcsr_to_csr(wo, cols, vals, num_rows)
        self.entries.append((key, (wo, cols, vals), value))
        if len(self.entries) > self.capacity:
            self.entries.pop(0)
        return value


_csr_cache = _CsrCache()


def sample_all_layers(window_offset, original_col_indices, values_condensed, initial_seeds, fanouts,
                      num_global_nodes, static_scores=None, window_part_ids=None, part_starts=None, part_ends=None,
                      alpha=1.0, beta=10.0, delta=0.0, gamma_bonus=0.0, score_scale=100.0, use_hacs=0,
                      locality_enabled=0, tile_rows=16, tile_cols=8, warps_per_block=8, seed=DEFAULT_SEED):
    """Argument list of the reference's ``sample_all_layers`` (core/wrapper/bind.cpp:99-121).

    The importance-score arguments (HACS / locality) are accepted and unused: sampling is uniform.
    Each returned layer is [window_offset, cols, vals, dst_nodes, src_nodes]; the reference's
    fourth and fifth entries are window-level ``active_windows`` / masks, which per-node sampling
    does not have."""
    if tile_rows != 16 or tile_cols != 8:
        raise RuntimeError("Currently only supports tile 16x8")
    if use_hacs or locality_enabled:
        raise RuntimeError("importance-score sampling is not part of this library; sampling is uniform")
    if not initial_seeds.is_cuda:
        raise RuntimeError("initial_seeds must be a CUDA tensor")
    num_rows = min(int(num_global_nodes), (window_offset.shape[0] - 1) * 16) if num_global_nodes > 0 else (window_offset.shape[0] - 1) * 16
    row_ptr, col_idx, values = _csr_cache.get(window_offset, original_col_indices, values_condensed, num_rows)
    return sample_layers_csr(row_ptr, col_idx, values, initial_seeds, list(fanouts), seed=seed,
                             values_dtype=values_condensed.dtype, timing=True)


def reindex_bcsr(col_indices, values_condensed, active_windows, tile_rows=16, tile_cols=8):
    """New int32 column ids; ``values_condensed`` is pruned in place (core/wrapper/bind.cpp:153-159)."""
    lib = _native.lib()
    if not col_indices.is_cuda:
        raise RuntimeError("col_indices must be a CUDA tensor")
    col_indices = col_indices.contiguous()
    active_windows = active_windows.to(torch.int32).contiguous()
    out = torch.empty_like(col_indices)
    _native.check(lib.grws_reindex_bcsr(_ptr(col_indices), _ptr(values_condensed), _DT[values_condensed.dtype],
                                        _ptr(active_windows), col_indices.numel(), active_windows.numel(),
                                        int(tile_rows), int(tile_cols), _ptr(out), _stream(col_indices.device)))
    return out
