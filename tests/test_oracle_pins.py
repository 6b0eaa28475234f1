"""Pins the CPU checker itself: against outputs of the reference's own code (tests/golden/, made by
tests/golden/make_golden.py), against published known-answer vectors, and against dense algebra."""
import ctypes
import ctypes.util
import os

import numpy as np
import pytest

from conftest import golden_cases, load_case


@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: os.path.basename(p)[5:-4])
def test_csr_to_bcsr_matches_reference_output(oracle, path):
    c = load_case(path)
    wo, cols, vals = oracle.csr_to_bcsr(int(c["num_rows"]), c["row_ptr"], c["col_idx"], c["values"])
    assert np.array_equal(wo, c["window_offset"])
    assert np.array_equal(cols, c["cols"])
    assert np.array_equal(vals.view(np.uint32), c["vals"].view(np.uint32))      # bit-exact


def test_known_answer_3x3(oracle):
    # a 3x3 CSR matrix and what the reference's csr_to_bcsr_cpu returns for it
    wo, cols, vals = oracle.csr_to_bcsr(3, [0, 2, 3, 5], [0, 2, 1, 0, 2], [.5, .25, 1, .125, .75])
    assert wo.tolist() == [0, 1]
    assert cols.tolist() == [0, 1, 2, -1, -1, -1, -1, -1]
    v = vals.reshape(16, 8)
    assert v[0, :3].tolist() == [.5, 0, .25] and v[1, :3].tolist() == [0, 1, 0] and v[2, :3].tolist() == [.125, 0, .75]
    assert not v[3:].any() and not v[:, 3:].any()


# Philox4x32-10 known-answer vectors published with Random123 (kat_vectors)
PHILOX_KAT = [
    ((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
    ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
    ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
     (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
]


@pytest.mark.parametrize("ctr,key,want", PHILOX_KAT)
def test_philox_known_answers(oracle, ctr, key, want):
    assert tuple(int(x) for x in oracle.philox4x32_10(ctr, key)) == want


def test_philox_matches_curand_host_generator(oracle):
    """cuRAND's host Philox4_32_10 generator gives every group of four outputs its own subsequence:
    output i is philox(counter = (0, 0, i / 4, 0), key = seed)[i % 4]."""
    path = None
    for cand in ("/usr/local/cuda/lib64/libcurand.so", ctypes.util.find_library("curand")):
        if cand and (os.path.exists(cand) or not os.path.isabs(cand)):
            path = cand
            break
    if path is None:
        pytest.skip("libcurand not found")
    try:
        cr = ctypes.CDLL(path)
    except OSError:
        pytest.skip("libcurand not loadable")
    gen = ctypes.c_void_p()
    CURAND_RNG_PSEUDO_PHILOX4_32_10 = 161
    if cr.curandCreateGeneratorHost(ctypes.byref(gen), CURAND_RNG_PSEUDO_PHILOX4_32_10) != 0:
        pytest.skip("curandCreateGeneratorHost unavailable here")
    seed = 0x5EED0123456789AB
    assert cr.curandSetPseudoRandomGeneratorSeed(gen, ctypes.c_ulonglong(seed)) == 0
    n = 64
    out = (ctypes.c_uint32 * n)()
    assert cr.curandGenerate(gen, out, ctypes.c_size_t(n)) == 0
    cr.curandDestroyGenerator(gen)
    got = np.frombuffer(out, dtype=np.uint32)
    key = (seed & 0xffffffff, seed >> 32)
    want = np.concatenate([oracle.philox4x32_10((0, 0, i, 0), key) for i in range(n // 4)])
    assert np.array_equal(got, want)


def _dense_from_bcsr(wo, cols, vals, num_cols):
    W = wo.shape[0] - 1
    A = np.zeros((W * 16, num_cols), dtype=np.float64)
    for w in range(W):
        for t in range(wo[w], wo[w + 1]):
            for c in range(8):
                col = cols[t * 8 + c]
                if col >= 0:
                    A[w * 16:(w + 1) * 16, col] += vals[t * 128 + c: (t + 1) * 128: 8]
    return A


@pytest.mark.parametrize("name", ["ragged_37x50", "empty_windows_80x64", "chunglu_600"])
def test_spmm_restatement_equals_dense_product(oracle, name):
    from conftest import GOLDEN
    c = load_case(os.path.join(GOLDEN, f"bcsr_{name}.npz"))
    num_cols = int(c["col_idx"].max()) + 1
    rng = np.random.default_rng(3)
    B = rng.standard_normal((num_cols, 24)).astype(np.float32)
    A = _dense_from_bcsr(c["window_offset"], c["cols"], c["vals"], num_cols)
    C = oracle.spmm_fwd(c["window_offset"], c["cols"], c["vals"], B)
    np.testing.assert_allclose(C, A @ B.astype(np.float64), rtol=1e-6, atol=1e-6)
    G = rng.standard_normal((A.shape[0], 24)).astype(np.float32)
    Gin = oracle.spmm_transpose(c["window_offset"], c["cols"], c["vals"], G, num_cols)
    np.testing.assert_allclose(Gin, A.T @ G.astype(np.float64), rtol=1e-6, atol=1e-6)


def test_reindex_restatement(oracle):
    # windows 2 and 5 active; column 37 (window 2, offset 5) -> 0*16+5; column 83 (window 5) -> 16+3;
    # column 100 (window 6, inactive) -> 0 with its value column zeroed; -1 -> window 0 inactive -> 0
    cols = np.array([37, 83, 100, -1, 80, 95, 32, 47], np.int32)
    vals = np.arange(128, dtype=np.float32) + 1
    new, pruned = oracle.reindex(cols, vals, np.array([2, 5], np.int32))
    assert new.tolist() == [5, 19, 0, 0, 16, 31, 0, 15]
    v = pruned.reshape(16, 8)
    assert not v[:, 2].any() and not v[:, 3].any() and v[:, [0, 1, 4, 5, 6, 7]].all()
    # with window 0 active a -1 id is looked up as window 0 and stays -1 (C division, reindex.cuh:48-51)
    new2, _ = oracle.reindex(np.array([-1, 3], np.int32).repeat(4), np.ones(128, np.float32), np.array([0], np.int32))
    assert new2.tolist() == [-1] * 4 + [3] * 4


def test_windows_and_masks(oracle):
    w, m = oracle.windows_and_masks(np.array([35, 32, -1, 5, 47, 5], np.int32))
    assert w.tolist() == [0, 2] and m.tolist() == [1 << 5, (1 << 3) | 1 | (1 << 15)]


def test_sampler_replay_properties(oracle):
    from graph_rws_b200.data import synthetic
    g = synthetic.sym_normalized_csr(500, *synthetic.chung_lu_edges(500, 4000, 2.5, 11))
    nodes = np.arange(0, 500, 3, dtype=np.int32)
    nbr, w, cnt = oracle.sample_hop(g.row_ptr, g.col_idx, g.values, nodes, 5, 0x5EED, 1)
    deg = np.diff(g.row_ptr)[nodes]
    assert np.array_equal(cnt, np.minimum(deg, 5))
    for i, v in enumerate(nodes):
        row = g.col_idx[g.row_ptr[v]:g.row_ptr[v + 1]]
        picked = nbr[i, :cnt[i]]
        assert len(set(picked.tolist())) == cnt[i] and set(picked.tolist()) <= set(row.tolist())
        assert (nbr[i, cnt[i]:] == -1).all()
        if deg[i] <= 5:
            assert np.array_equal(picked, row)
    # keyed: same (seed, node, hop) -> same list regardless of the batch it is sampled in
    nbr2, _, _ = oracle.sample_hop(g.row_ptr, g.col_idx, g.values, nodes[::-1].copy(), 5, 0x5EED, 1)
    assert np.array_equal(nbr2[::-1], nbr)
    nbr3, _, _ = oracle.sample_hop(g.row_ptr, g.col_idx, g.values, nodes, 5, 0x5EED, 2)
    assert not np.array_equal(nbr3, nbr)


def test_sampler_replay_is_uniform(oracle):
    """chi-square of the selection counts of one 40-neighbour node over many keys."""
    deg, fanout, trials = 40, 5, 4000
    row_ptr = np.array([0, deg], np.int64)
    col = np.arange(deg, dtype=np.int32)
    counts = np.zeros(deg)
    for s in range(trials):
        nbr, _, _ = oracle.sample_hop(row_ptr, col, None, np.array([0], np.int32), fanout, 1000 + s, 0)
        counts[nbr[0]] += 1
    expect = trials * fanout / deg
    chi2 = ((counts - expect) ** 2 / expect).sum()
    assert chi2 < 72.1      # chi-square 39 dof, p = 0.001


def test_block_build_is_csr_to_bcsr_of_local_edges(oracle):
    from graph_rws_b200.data import synthetic
    g = synthetic.sym_normalized_csr(400, *synthetic.chung_lu_edges(400, 3000, 2.5, 5))
    seeds = np.array([7, 300, 12, 5, 99], np.int32)
    blocks = oracle.sample_layers(g.row_ptr, g.col_idx, g.values, seeds, [4, 3], 42)
    assert len(blocks) == 2
    outer, inner = blocks[0], blocks[1]
    assert np.array_equal(inner["dst"], seeds)
    assert np.array_equal(inner["src"][:5], seeds)                       # target nodes first
    assert np.array_equal(outer["dst"], inner["src"])
    tail = inner["src"][5:]
    assert np.array_equal(tail, np.unique(tail)) and not set(tail.tolist()) & set(seeds.tolist())
    # every stored value is the global edge weight of (dst, src[col])
    wo, cols, vals = inner["window_offset"], inner["cols"], inner["vals"].reshape(-1, 16, 8)
    for t in range(wo[-1]):
        for r in range(16):
            for c in range(8):
                if vals[t, r, c] != 0:
                    u, v = seeds[r], inner["src"][cols[t * 8 + c]]
                    row = g.col_idx[g.row_ptr[u]:g.row_ptr[u + 1]]
                    assert vals[t, r, c] == g.values[g.row_ptr[u] + np.searchsorted(row, v)]
