"""Seeded synthetic graphs with the shapes of the benchmark configurations.

The real datasets the reference trains on (Cora, ogbn-arxiv, Reddit, ogbn-products,
ogbn-papers100M; configs/*.yaml) cannot be downloaded, so every measurement and parity case runs
on Chung-Lu power-law graphs of the same node / edge counts.  Edge weights follow the reference's
symmetric normalisation ``deg^-1/2[src] * deg^-1/2[dst]`` with self-loops added
(data/data_loader.py:980-986).

Everything here is host-side numpy: it prepares inputs, it is not part of the timed path.
"""
from dataclasses import dataclass

import numpy as np


@dataclass
class CSRGraph:
    num_nodes: int
    row_ptr: np.ndarray   # int64 [n+1]
    col_idx: np.ndarray   # int32 [nnz], ascending inside each row
    values: np.ndarray    # float32 [nnz]

    @property
    def nnz(self) -> int:
        return int(self.col_idx.shape[0])


def chung_lu_edges(n: int, e_target: int, gamma: float, seed: int, directed: bool = False):
    """Draw ``e_target`` distinct node pairs (no self pairs) with expected degrees
    ``w_i ~ (rank_i + 1)^(-1/(gamma-1))``; ranks are scattered over the id space by a seeded
    permutation so that hubs are not clustered in the first windows."""
    rng = np.random.Generator(np.random.Philox(seed))
    w = (np.arange(n, dtype=np.float64) + 1.0) ** (-1.0 / (gamma - 1.0))
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    perm = rng.permutation(n)
    got = np.empty(0, dtype=np.int64)
    while got.size < e_target:
        m = int((e_target - got.size) * 1.3) + 1024
        u = perm[np.searchsorted(cdf, rng.random(m))]
        v = perm[np.searchsorted(cdf, rng.random(m))]
        keep = u != v
        u, v = u[keep], v[keep]
        if directed:
            key = u.astype(np.int64) * n + v
        else:
            key = np.minimum(u, v).astype(np.int64) * n + np.maximum(u, v)
        got = np.unique(np.concatenate([got, key]))
        if got.size > e_target:
            got = np.sort(rng.permutation(got)[:e_target])
    return got // n, got % n


def community_edges(n: int, e_target: int, num_comm: int, intra: float, seed: int):
    """Planted contiguous-id communities with a power-law degree profile inside each community
    (the Reddit-shaped dense graph): an edge picks a community, then both endpoints by local rank;
    with probability ``1 - intra`` the second endpoint comes from a random community."""
    rng = np.random.Generator(np.random.Philox(seed))
    bounds = np.linspace(0, n, num_comm + 1).astype(np.int64)
    size = np.diff(bounds)
    w = (np.arange(size.max(), dtype=np.float64) + 1.0) ** (-1.0 / 1.5)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]

    def draw_local(comm, m):
        loc = np.minimum(np.searchsorted(cdf, rng.random(m)), size[comm] - 1)
        return bounds[comm] + loc

    got = np.empty(0, dtype=np.int64)
    while got.size < e_target:
        m = int((e_target - got.size) * 1.5) + 4096
        cu = rng.integers(0, num_comm, m)
        u = draw_local(cu, m)
        same = rng.random(m) < intra
        cv = np.where(same, cu, rng.integers(0, num_comm, m))
        v = draw_local(cv, m)
        keep = u != v
        u, v = u[keep], v[keep]
        got = np.unique(np.concatenate([got, np.minimum(u, v) * n + np.maximum(u, v)]))
        if got.size > e_target:
            got = np.sort(rng.permutation(got)[:e_target])
    return got // n, got % n


def sym_normalized_csr(n: int, u: np.ndarray, v: np.ndarray) -> CSRGraph:
    """Symmetrise, add self-loops, weight every entry ``deg^-1/2[row] * deg^-1/2[col]``."""
    r = np.concatenate([u, v, np.arange(n, dtype=np.int64)])
    c = np.concatenate([v, u, np.arange(n, dtype=np.int64)])
    key = np.unique(r.astype(np.int64) * n + c)
    r, c = key // n, key % n
    deg = np.maximum(np.bincount(r, minlength=n), 1).astype(np.float64)
    val = (deg[r] ** -0.5 * deg[c] ** -0.5).astype(np.float32)
    rp = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(r, minlength=n), out=rp[1:])
    return CSRGraph(n, rp, c.astype(np.int32), val)


def graph_for_config(name: str, scale: float = 1.0) -> CSRGraph:
    """Named workloads.  ``scale`` shrinks node and edge counts together (parity-test sizes)."""
    if name == "small_gcn":            # 2,708 nodes, 5,278 undirected edges, exponent 2.5
        n, e = int(2708 * scale), int(5278 * scale)
        return sym_normalized_csr(n, *chung_lu_edges(n, e, 2.5, 1001))
    if name == "spmm_mid":             # 169,343 nodes, 1,166,243 directed edges, exponent 2.5
        n, e = int(169343 * scale), int(1166243 * scale)
        return sym_normalized_csr(n, *chung_lu_edges(n, e, 2.5, 1002, directed=True))
    if name == "dense_community":      # 232,965 nodes, ~114.6M nnz, 50 communities, 0.8 intra
        n = int(232965 * scale)
        e = int((114_600_000 * scale * scale - n) // 2) if scale < 1.0 else (114_600_000 - n) // 2
        return sym_normalized_csr(n, *community_edges(n, e, 50, 0.8, 1003))
    if name == "sampled_mid":          # 2,449,029 nodes, 61.86M undirected edges
        n, e = int(2449029 * scale), int(61_860_000 * scale)
        return sym_normalized_csr(n, *chung_lu_edges(n, e, 2.5, 1004))
    raise ValueError(f"unknown workload {name!r}")


def community_csr_torch(n: int, e_target: int, num_comm: int, intra: float, seed: int, device):
    """``community_edges`` + ``sym_normalized_csr`` with torch ops on ``device`` (seconds on a GPU
    at the 114.6 M-nnz size, where the numpy pair takes minutes).  Same distribution, another
    random stream: undirected pairs are drawn in one oversampled batch and the first ``e_target``
    distinct ones in key order of a seeded shuffle are kept.  Returns
    (row_ptr int64 [n+1], col_idx int32 [nnz], values float32 [nnz]) on ``device``."""
    import torch
    gen = torch.Generator(device=device).manual_seed(seed)
    bounds = torch.linspace(0, n, num_comm + 1, dtype=torch.float64).long().to(device)
    size = bounds[1:] - bounds[:-1]
    w = (torch.arange(int(size.max()), dtype=torch.float64, device=device) + 1.0) ** (-1.0 / 1.5)
    cdf = torch.cumsum(w, 0)
    cdf /= cdf[-1].clone()

    def draw_local(comm, m):
        loc = torch.searchsorted(cdf, torch.rand(m, generator=gen, device=device, dtype=torch.float64))
        return bounds[comm] + torch.minimum(loc, size[comm] - 1)

    got = torch.empty(0, dtype=torch.int64, device=device)
    while got.numel() < e_target:
        m = int((e_target - got.numel()) * 1.5) + 4096
        cu = torch.randint(0, num_comm, (m,), generator=gen, device=device)
        u = draw_local(cu, m)
        same = torch.rand(m, generator=gen, device=device) < intra
        cv = torch.where(same, cu, torch.randint(0, num_comm, (m,), generator=gen, device=device))
        v = draw_local(cv, m)
        keep = u != v
        u, v = u[keep], v[keep]
        got = torch.unique(torch.cat([got, torch.minimum(u, v) * n + torch.maximum(u, v)]))
        del u, v, cu, cv, same, keep
        if got.numel() > e_target:
            got = got[torch.randperm(got.numel(), generator=gen, device=device)[:e_target]]
    u, v = got // n, got % n
    loops = torch.arange(n, dtype=torch.int64, device=device)
    key = torch.unique(torch.cat([u * n + v, v * n + u, loops * n + loops]))
    del got, u, v
    r, c = key // n, key % n
    del key
    counts = torch.bincount(r, minlength=n)
    dinv = counts.clamp(min=1).double() ** -0.5
    val = (dinv[r] * dinv[c]).float()
    rp = torch.zeros(n + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=rp[1:])
    return rp, c.int(), val


def chung_lu_csr_torch(n: int, e_target: int, gamma: float, seed: int, device):
    """``chung_lu_edges`` + ``sym_normalized_csr`` with torch ops on ``device``: the power-law graph
    of the sampled-training configurations at full size (2.45 M nodes, 61.86 M undirected edges)
    takes seconds on a GPU, minutes with numpy.  Same distribution, another random stream; every
    device of one type draws the same graph from the same seed.  Returns
    (row_ptr int64 [n+1], col_idx int32 [nnz], values float32 [nnz]) on ``device``."""
    import torch
    gen = torch.Generator(device=device).manual_seed(seed)
    w = (torch.arange(n, dtype=torch.float64, device=device) + 1.0) ** (-1.0 / (gamma - 1.0))
    cdf = torch.cumsum(w, 0)
    cdf /= cdf[-1].clone()
    del w
    perm = torch.randperm(n, generator=gen, device=device)
    got = torch.empty(0, dtype=torch.int64, device=device)
    while got.numel() < e_target:
        m = int((e_target - got.numel()) * 1.3) + 4096
        u = perm[torch.searchsorted(cdf, torch.rand(m, generator=gen, device=device, dtype=torch.float64)).clamp_(max=n - 1)]
        v = perm[torch.searchsorted(cdf, torch.rand(m, generator=gen, device=device, dtype=torch.float64)).clamp_(max=n - 1)]
        keep = u != v
        u, v = u[keep], v[keep]
        got = torch.unique(torch.cat([got, torch.minimum(u, v) * n + torch.maximum(u, v)]))
        del u, v, keep
        if got.numel() > e_target:
            got = got[torch.randperm(got.numel(), generator=gen, device=device)[:e_target]]
    del cdf, perm
    u, v = got // n, got % n
    loops = torch.arange(n, dtype=torch.int64, device=device)
    key = torch.unique(torch.cat([u * n + v, v * n + u, loops * n + loops]))
    del got, u, v, loops
    r, c = key // n, key % n
    del key
    counts = torch.bincount(r, minlength=n)
    dinv = counts.clamp(min=1).double() ** -0.5
    val = (dinv[r] * dinv[c]).float()
    rp = torch.zeros(n + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=rp[1:])
    return rp, c.int(), val


def sampling_algorithmic_bytes(frontier_sizes, sampled_edges, block_tiles, block_windows, val_bytes: int = 4) -> dict:
    """Compulsory traffic of the sampling side of one mini-batch step, per hop h with frontier F_h,
    sampled edges S_h and a block of T_h tiles in W_h windows.  Sampling: two int64 row offsets per
    frontier node, one column id read and one neighbour id + weight written per sampled edge
    (16 F + 4 S + 8 S).  Dedup / reindex / block build: every sampled id read and its local id
    written (8 S), then the block (32 + 128 * sizeof(value) bytes per tile, 8 bytes per window)."""
    sample = sum(16 * f + 12 * s for f, s in zip(frontier_sizes, sampled_edges))
    build = sum(8 * s + t * (32 + 128 * val_bytes) + 8 * (w + 1)
                for s, t, w in zip(sampled_edges, block_tiles, block_windows))
    return {"sample": int(sample), "build": int(build), "total": int(sample + build)}


def spmm_algorithmic_bytes(num_windows: int, num_tiles: int, k_touched: int, n: int,
                           val_bytes: int, b_bytes: int, c_bytes: int) -> int:
    """Compulsory traffic of one BCSR SpMM: offsets + column ids + tile values + every touched
    row of the dense operand once + the output once (gathers served by L2 are not counted)."""
    return (8 * (num_windows + 1) + 32 * num_tiles + 128 * num_tiles * val_bytes
            + k_touched * n * b_bytes + 16 * num_windows * n * c_bytes)
