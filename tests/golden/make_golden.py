"""Generates tests/golden/*.npz by running the REFERENCE's own code in this container.

Needs oracle/_ref/core_lib.so (python oracle/build_ref.py), which is compiled from the
reference sources; the fixtures it writes are what travels.  Every case stores the CSR input and
the three arrays returned by the reference's csr_to_bcsr_cpu
(core/wrapper/convert_wrapper.cpp:27-180, binding core/wrapper/bind.cpp:144-151).

Usage: python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref  # noqa: E402
from graph_rws_b200.data import synthetic  # noqa: E402


def random_csr(rng, rows, cols, density, dup=False, sort_rows=True):
    rp = [0]
    ci, vv = [], []
    for _ in range(rows):
        k = rng.binomial(cols, density)
        c = rng.choice(cols, size=min(k, cols), replace=False)
        if dup and c.size:
            c = np.concatenate([c, c[: max(1, c.size // 3)]])     # duplicate (row, col) entries
        c = np.sort(c) if (sort_rows and not dup) else rng.permutation(c)
        ci.append(c)
        vv.append(rng.standard_normal(c.size).astype(np.float32))
        rp.append(rp[-1] + c.size)
    return (np.asarray(rp, np.int64), np.concatenate(ci).astype(np.int32) if ci else np.zeros(0, np.int32),
            np.concatenate(vv).astype(np.float32) if vv else np.zeros(0, np.float32))


def cases():
    rng = np.random.default_rng(20240611)
    # the 3x3 known-answer example
    yield "kat3x3", 3, (np.array([0, 2, 3, 5], np.int64), np.array([0, 2, 1, 0, 2], np.int32),
                        np.array([.5, .25, 1, .125, .75], np.float32))
    yield "ragged_37x50", 37, random_csr(rng, 37, 50, 0.2)
    yield "unsorted_64x300", 64, random_csr(rng, 64, 300, 0.05, sort_rows=False)
    yield "duplicates_40x30", 40, random_csr(rng, 40, 30, 0.3, dup=True)
    rp, ci, vv = random_csr(rng, 80, 64, 0.1)
    # empty windows: rows 16..47 have no entries
    keep = np.ones(ci.size, bool)
    keep[rp[16]:rp[48]] = False
    cnt = np.diff(rp)
    cnt[16:48] = 0
    rp2 = np.zeros_like(rp)
    np.cumsum(cnt, out=rp2[1:])
    yield "empty_windows_80x64", 80, (rp2, ci[keep], vv[keep])
    yield "all_empty_20", 20, (np.zeros(21, np.int64), np.zeros(0, np.int32), np.zeros(0, np.float32))
    yield "dense_row_16x2000", 16, random_csr(rng, 16, 2000, 0.6)
    g = synthetic.sym_normalized_csr(600, *synthetic.chung_lu_edges(600, 1500, 2.5, 7))
    yield "chunglu_600", 600, (g.row_ptr, g.col_idx, g.values)


def main():
    ref = build_ref.load()
    if ref is None:
        raise SystemExit("oracle/_ref/core_lib.so not built: run python oracle/build_ref.py")
    for name, num_rows, (rp, ci, vv) in cases():
        wo, cols, vals = ref.csr_to_bcsr_cpu(num_rows, torch.from_numpy(rp), torch.from_numpy(ci),
                                             torch.from_numpy(vv), 16, 8)
        out = os.path.join(HERE, f"bcsr_{name}.npz")
        np.savez_compressed(out, num_rows=np.int64(num_rows), row_ptr=rp, col_idx=ci, values=vv,
                            window_offset=wo.numpy(), cols=cols.numpy(), vals=vals.numpy())
        print(f"{name}: rows={num_rows} nnz={ci.size} tiles={int(wo[-1])} -> {os.path.getsize(out)} bytes")


if __name__ == "__main__":
    main()
