"""On-disk BCSR in the reference's cache format, and a chunked loader to the GPU.

The reference caches a converted graph as four files next to ``<name>.pt``
(data/data_loader.py:282-406): ``<name>_bcsr_meta.pt`` (a ``torch.save``d dict with the scalar
attributes and the three array lengths), ``<name>_bcsr_window_offset.bin`` (int64),
``<name>_bcsr_col_indices.bin`` (int32) and ``<name>_bcsr_values.bin`` (float32), raw
little-endian arrays.  ``save_bcsr_bins`` writes exactly those, so caches interchange both ways.

``load_bcsr_bins`` never materialises the value array in host memory: the files are memory-mapped
and moved to the device in fixed-size pieces through one pinned staging buffer, and the fp32 values
are narrowed to the requested ``values_dtype`` on the GPU piece by piece (the 114.6 M-nnz graph has
4.2 GB of fp32 tile values and 2.1 GB after narrowing to bf16).  With ``device='cpu'`` the arrays
stay memory-mapped, which is what the reference does when host memory is short
(data/data_loader.py:363-371).
"""
import os
import warnings
from typing import Optional

import numpy as np
import torch

from .bcsr import BCSRGraph

_CHUNK_BYTES = 64 << 20


def bcsr_bin_paths(cache_path: str):
    """(meta, window_offset, col_indices, values) file names of ``cache_path``
    (data/data_loader.py:282-287)."""
    return (cache_path.replace('.pt', '_bcsr_meta.pt'),
            cache_path.replace('.pt', '_bcsr_window_offset.bin'),
            cache_path.replace('.pt', '_bcsr_col_indices.bin'),
            cache_path.replace('.pt', '_bcsr_values.bin'))


def save_bcsr_bins(bcsr: BCSRGraph, cache_path: str) -> bool:
    """Write the graph in the reference's layout; values are stored as fp32 whatever the graph holds."""
    meta_path, off_path, col_path, val_path = bcsr_bin_paths(cache_path)
    window_offset = bcsr.window_offset.detach().cpu().to(torch.int64).contiguous()
    col_indices = bcsr.original_col_indices.detach().cpu().to(torch.int32).contiguous()
    window_offset.numpy().tofile(off_path)
    col_indices.numpy().tofile(col_path)
    values = bcsr.values_condensed.detach()
    with open(val_path, 'wb') as f:           # piecewise: no second full-size fp32 copy
        step = _CHUNK_BYTES // 4
        for lo in range(0, values.numel(), step):
            values[lo:lo + step].to(device='cpu', dtype=torch.float32).contiguous().numpy().tofile(f)
    meta = {
        'num_nodes': int(bcsr.num_nodes),
        'num_edges': int(bcsr.num_edges),
        'num_rows': int(bcsr.num_rows),
        'num_cols': int(bcsr.num_cols),
        'tile_rows': int(bcsr.tile_rows),
        'tile_cols': int(bcsr.tile_cols),
        'num_windows': int(bcsr.num_windows),
        'window_offset_len': int(window_offset.numel()),
        'col_indices_len': int(col_indices.numel()),
        'values_len': int(values.numel()),
    }
    torch.save(meta, meta_path)
    return True


def _to_device_chunked(arr: np.ndarray, device: torch.device, out_dtype: torch.dtype) -> torch.Tensor:
    """Copy a (memory-mapped) host array to ``device`` through one pinned buffer, casting on the GPU."""
    src_dtype = torch.from_numpy(np.empty(0, dtype=arr.dtype)).dtype
    out = torch.empty(arr.shape[0], dtype=out_dtype, device=device)
    step = max(1, _CHUNK_BYTES // arr.dtype.itemsize)
    stage = [torch.empty(min(step, max(arr.shape[0], 1)), dtype=src_dtype).pin_memory() for _ in range(2)]
    done = [None, None]
    for i, lo in enumerate(range(0, arr.shape[0], step)):
        buf, n = stage[i & 1], min(step, arr.shape[0] - lo)
        if done[i & 1] is not None:
            done[i & 1].synchronize()               # the copy that last used this buffer has finished
        buf[:n].numpy()[:] = arr[lo:lo + n]         # page-fault the mapped file into the pinned buffer
        out[lo:lo + n].copy_(buf[:n], non_blocking=True)
        done[i & 1] = torch.cuda.Event()
        done[i & 1].record()
    torch.cuda.current_stream(device).synchronize()
    return out


def load_bcsr_bins(cache_path: str, device='cuda', values_dtype: Optional[torch.dtype] = torch.float32) -> Optional[BCSRGraph]:
    """Load a cache written by ``save_bcsr_bins`` or by the reference.  Returns ``None`` when a file
    is missing or a length disagrees with the meta data (the reference then rebuilds the graph,
    data/data_loader.py:345-381)."""
    meta_path, off_path, col_path, val_path = bcsr_bin_paths(cache_path)
    if not all(os.path.exists(p) for p in (meta_path, off_path, col_path, val_path)):
        return None
    meta = torch.load(meta_path, weights_only=False)
    off_len, col_len, val_len = (int(meta.get(k, 0)) for k in ('window_offset_len', 'col_indices_len', 'values_len'))
    if off_len <= 0 or col_len <= 0 or val_len <= 0:
        return None
    if (os.path.getsize(off_path) != off_len * 8 or os.path.getsize(col_path) != col_len * 4
            or os.path.getsize(val_path) != val_len * 4):
        return None
    off_np = np.memmap(off_path, dtype=np.int64, mode='r', shape=(off_len,))
    col_np = np.memmap(col_path, dtype=np.int32, mode='r', shape=(col_len,))
    val_np = np.memmap(val_path, dtype=np.float32, mode='r', shape=(val_len,))
    device = torch.device(device)
    vdt = values_dtype or torch.float32
    if device.type == 'cuda':
        wo = _to_device_chunked(off_np, device, torch.int64)
        cols = _to_device_chunked(col_np, device, torch.int32)
        vals = _to_device_chunked(val_np, device, vdt)
    else:
        with warnings.catch_warnings():      # read-only maps: nothing on this path writes to them
            warnings.simplefilter("ignore", UserWarning)
            wo, cols = torch.from_numpy(off_np), torch.from_numpy(col_np)
            vals = torch.from_numpy(val_np)
        if vdt != torch.float32:
            vals = vals.to(vdt)
    g = BCSRGraph(num_nodes=int(meta['num_nodes']), num_edges=int(meta['num_edges']),
                  tile_rows=int(meta['tile_rows']), tile_cols=int(meta['tile_cols']),
                  window_offset=wo, original_col_indices=cols, values_condensed=vals, device=device,
                  num_rows=int(meta['num_rows']), num_cols=int(meta['num_cols']), values_dtype=vdt)
    g.num_windows = int(meta.get('num_windows', g.num_windows))
    return g
