"""GPU sampler against the host Philox replay: neighbour lists, dedup / reindex and the per-hop
BCSR blocks are all bit-exact; the selection is uniform (chi-square)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def graph():
    from graph_rws_b200.data import synthetic
    return synthetic.sym_normalized_csr(5000, *synthetic.chung_lu_edges(5000, 60000, 2.3, 31))


def _dev_csr(g):
    dev = torch.device("cuda")
    return (torch.from_numpy(g.row_ptr).to(dev), torch.from_numpy(g.col_idx).to(dev), torch.from_numpy(g.values).to(dev))


@pytest.mark.parametrize("fanout", [1, 5, 15, 32, 40, 200])
def test_sample_hop_is_bit_exact(oracle, graph, fanout):
    from graph_rws_b200 import core
    rp, ci, vv = _dev_csr(graph)
    rng = np.random.default_rng(fanout)
    nodes = rng.permutation(graph.num_nodes)[:700].astype(np.int32)
    nodes[5] = -1                                     # an empty entry
    nbr, w, cnt = core.sample_hop(rp, ci, vv, torch.from_numpy(nodes).cuda(), fanout, seed=0x5EED, hop=2)
    nbr_r, w_r, cnt_r = oracle.sample_hop(graph.row_ptr, graph.col_idx, graph.values, nodes, fanout, 0x5EED, 2)
    assert np.array_equal(nbr.cpu().numpy(), nbr_r)
    assert np.array_equal(w.cpu().numpy(), w_r)
    assert np.array_equal(cnt.cpu().numpy(), cnt_r)


def test_sample_hop_does_not_depend_on_batch(graph):
    from graph_rws_b200 import core
    rp, ci, vv = _dev_csr(graph)
    a = torch.arange(0, 3000, 3, dtype=torch.int32, device="cuda")
    n1, _, _ = core.sample_hop(rp, ci, vv, a, 10, seed=7, hop=1)
    n2, _, _ = core.sample_hop(rp, ci, vv, a.flip(0).contiguous(), 10, seed=7, hop=1)
    assert torch.equal(n1, n2.flip(0))
    n3, _, _ = core.sample_hop(rp, ci, vv, a, 10, seed=8, hop=1)
    assert not torch.equal(n1, n3)


def test_uniformity_chi_square():
    from graph_rws_b200 import core
    deg, fanout, trials = 40, 5, 4000
    rp = torch.tensor([0, deg], dtype=torch.int64, device="cuda")
    ci = torch.arange(deg, dtype=torch.int32, device="cuda")
    node = torch.zeros(1, dtype=torch.int32, device="cuda")
    counts = np.zeros(deg)
    for s in range(trials):
        nbr, _, _ = core.sample_hop(rp, ci, None, node, fanout, seed=1000 + s, hop=0)
        counts[nbr[0].cpu().numpy()] += 1
    expect = trials * fanout / deg
    assert ((counts - expect) ** 2 / expect).sum() < 72.1          # chi-square, 39 dof, p = 0.001


def test_block_build_is_bit_exact(oracle, graph):
    from graph_rws_b200 import core
    rp, ci, vv = _dev_csr(graph)
    rng = np.random.default_rng(3)
    dst = rng.permutation(graph.num_nodes)[:333].astype(np.int32)
    nbr_r, w_r, _ = oracle.sample_hop(graph.row_ptr, graph.col_idx, graph.values, dst, 7, 99, 0)
    src_r, wo_r, cols_r, vals_r = oracle.build_block(dst, nbr_r, w_r)
    src, wo, cols, vals = core.build_block(torch.from_numpy(dst).cuda(), torch.from_numpy(nbr_r).cuda(),
                                           torch.from_numpy(w_r).cuda())
    assert np.array_equal(src.cpu().numpy(), src_r)
    assert np.array_equal(wo.cpu().numpy(), wo_r)
    assert np.array_equal(cols.cpu().numpy(), cols_r)
    assert np.array_equal(vals.cpu().numpy().view(np.uint32), vals_r.view(np.uint32))


def test_multi_hop_sampler_matches_replay(oracle, graph):
    """BCSRSampler.sample_layers over a BCSRGraph: CSR extraction + 3 hops + blocks, all bit-exact."""
    from graph_rws_b200 import BCSRGraph
    from graph_rws_b200.sampler import BCSRSampler
    g = BCSRGraph.from_csr(graph.num_nodes, graph.row_ptr, graph.col_idx, graph.values, device=torch.device("cuda"))
    rp, ci, vv = BCSRSampler.graph_csr(g)
    assert np.array_equal(rp.cpu().numpy(), graph.row_ptr)
    assert np.array_equal(ci.cpu().numpy(), graph.col_idx)
    assert np.array_equal(vv.cpu().numpy(), graph.values)
    seeds = np.random.default_rng(1).permutation(graph.num_nodes)[:256].astype(np.int32)
    sampler = BCSRSampler(fanouts=[15, 10, 5], verbose=False, seed=0x5EED, fused=False)      # exactly sized hops
    layers = sampler.sample_layers(g, torch.from_numpy(seeds))
    blocks = oracle.sample_layers(graph.row_ptr, graph.col_idx, graph.values, seeds, [15, 10, 5], 0x5EED)
    assert len(layers) == 3
    for sub, ref in zip(layers, blocks):
        assert np.array_equal(sub.output_nodes.cpu().numpy(), ref["dst"])
        assert np.array_equal(sub.input_nodes.cpu().numpy(), ref["src"])
        assert sub.num_rows == ref["dst"].size and sub.num_cols == ref["src"].size
        assert np.array_equal(sub.window_offset.cpu().numpy(), ref["window_offset"])
        # the sampler sizes a block's tile arrays by a bound instead of reading the tile count back:
        # the tiles the offsets cover equal the checker's, the unused tail is empty (-1 / 0)
        cols, vals = sub.original_col_indices.cpu().numpy(), sub.values_condensed.cpu().numpy()
        assert cols.size >= ref["cols"].size and cols.size % 8 == 0 and vals.size == cols.size * 16
        assert np.array_equal(cols[:ref["cols"].size], ref["cols"]) and (cols[ref["cols"].size:] == -1).all()
        assert np.array_equal(vals[:ref["vals"].size], ref["vals"]) and (vals[ref["vals"].size:] == 0).all()
    assert np.array_equal(layers[-1].output_nodes.cpu().numpy(), seeds)
    # target-first layout: a block's rows are the first entries of its columns
    for sub in layers:
        assert torch.equal(sub.input_nodes[:sub.num_rows], sub.output_nodes)


def test_reference_named_sampling_entry_points(oracle, graph):
    from graph_rws_b200 import BCSRGraph, core
    g = BCSRGraph.from_csr(graph.num_nodes, graph.row_ptr, graph.col_idx, graph.values, device=torch.device("cuda"))
    seeds = torch.arange(100, 164, dtype=torch.int32, device="cuda")
    dummy = torch.ones(1, device="cuda")
    layers, timings = core.sample_all_layers(g.window_offset, g.original_col_indices, g.values_condensed, seeds,
                                             [5, 10], g.num_nodes, dummy, dummy.int(), dummy.int(), dummy.int())
    assert len(layers) == 2 and len(layers[0]) == 5 and len(timings) == 2
    assert timings[0].total_time >= 0 and "total_time" in timings[0].to_dict()
    blocks = oracle.sample_layers(graph.row_ptr, graph.col_idx, graph.values, seeds.cpu().numpy(), [10, 5], 0x5EED)
    assert np.array_equal(layers[0][4].cpu().numpy(), blocks[1]["src"])       # hop 0 = the seeds' hop
    assert np.array_equal(layers[1][1].cpu().numpy(), blocks[0]["cols"])
    # reindex_bcsr: reference semantics including pruning and the -1 quirk
    cols = torch.tensor([37, 83, 100, -1, 80, 95, 32, 47], dtype=torch.int32, device="cuda")
    vals = (torch.arange(128, dtype=torch.float32, device="cuda") + 1)
    new = core.reindex_bcsr(cols, vals, torch.tensor([2, 5], dtype=torch.int32, device="cuda"))
    new_r, vals_r = oracle.reindex(cols.cpu().numpy(), (np.arange(128) + 1).astype(np.float32), np.array([2, 5], np.int32))
    assert np.array_equal(new.cpu().numpy(), new_r) and np.array_equal(vals.cpu().numpy(), vals_r)
    new2 = core.reindex_bcsr(torch.tensor([-1, 3] * 4, dtype=torch.int32, device="cuda"), torch.ones(128, device="cuda"),
                             torch.tensor([0], dtype=torch.int32, device="cuda"))
    assert new2.cpu().tolist() == [-1, 3] * 4


def test_padded_hops_keep_the_real_part_identical(graph):
    """pad_to only appends -1 nodes: the real rows / columns of every block are unchanged."""
    from graph_rws_b200 import BCSRGraph
    from graph_rws_b200.sampler import BCSRSampler
    g = BCSRGraph.from_csr(graph.num_nodes, graph.row_ptr, graph.col_idx, graph.values, device=torch.device("cuda"))
    seeds = torch.arange(0, 600, 3, dtype=torch.int32)
    exact = BCSRSampler([4, 3], verbose=False, seed=5, fused=False).sample_layers(g, seeds)
    padded = BCSRSampler([4, 3], verbose=False, seed=5, pad_to=512, fused=False).sample_layers(g, seeds)
    inner_e, inner_p = exact[1], padded[1]
    assert inner_p.num_cols % 512 == 0 and inner_p.num_cols >= inner_e.num_cols
    n = inner_e.num_cols
    assert torch.equal(inner_p.input_nodes[:n], inner_e.input_nodes) and (inner_p.input_nodes[n:] == -1).all()
    assert torch.equal(inner_p.original_col_indices, inner_e.original_col_indices)
    outer_e, outer_p = exact[0], padded[0]
    assert outer_p.num_rows == inner_p.num_cols
    te = int(outer_e.window_offset[-1])
    # the padded rows have no neighbours: same tiles, only more (empty) windows
    assert int(outer_p.window_offset[-1]) == te
    # ... and new source nodes are numbered after the (longer, padded) destination list
    ce = outer_e.original_col_indices[:te * 8]
    shifted = torch.where(ce >= n, ce + (inner_p.num_cols - n), ce)
    assert torch.equal(outer_p.original_col_indices[:te * 8], shifted)


@pytest.mark.parametrize("pad_to", [0, 512])
def test_fused_all_hops_call_matches_replay(oracle, graph, pad_to):
    """grws_sample_layers: every hop's source list, offsets, column ids and values equal the host
    replay run on the same (padded) frontiers; buffers have the bound sizes and empty tails."""
    from graph_rws_b200 import core
    rp, ci, vv = _dev_csr(graph)
    seeds = np.random.default_rng(11).permutation(graph.num_nodes)[:300].astype(np.int32)
    fanouts = [5, 10, 15]                                  # in the order the hops consume them
    n_dst, n_src, tiles = core.sample_layers_sizes(seeds.size, fanouts, pad_to)
    assert n_dst[0] == seeds.size and all(n_dst[h + 1] == n_src[h] for h in range(2))
    if pad_to:
        assert all(n % pad_to == 0 for n in n_src)
    hops, counts = core.sample_layers_fused(rp, ci, vv, torch.from_numpy(seeds), fanouts, seed=77, pad_to=pad_to,
                                            want_counts=True)
    torch.cuda.synchronize()
    core.check_device_status()
    counts = counts.cpu().numpy()
    dst = seeds
    for h, f in enumerate(fanouts):
        wo, cols, vals, dst_g, src_g = (t.cpu().numpy() for t in hops[h])
        assert np.array_equal(dst_g, dst) and src_g.size == n_src[h] and cols.size == tiles[h] * 8
        nbr_r, w_r, _ = oracle.sample_hop(graph.row_ptr, graph.col_idx, graph.values, dst, f, 77, h)
        src_r, wo_r, cols_r, vals_r = oracle.build_block(dst, nbr_r, w_r)
        assert np.array_equal(src_g[:src_r.size], src_r) and (src_g[src_r.size:] == -1).all()
        assert np.array_equal(wo, wo_r)
        assert np.array_equal(cols[:cols_r.size], cols_r) and (cols[cols_r.size:] == -1).all()
        assert np.array_equal(vals[:vals_r.size].view(np.uint32), vals_r.view(np.uint32)) and (vals[vals_r.size:] == 0).all()
        assert counts[h].tolist() == [src_r.size, int((nbr_r >= 0).sum()), int(wo_r[-1]), int((dst >= 0).sum())]
        dst = src_g                                        # the next frontier keeps the -1 padding


def test_fused_blocks_train_like_exact_blocks(graph):
    """A 3-layer GCN sees the same logits and weight gradients for the seeds through the bound-sized
    blocks of the fused call (sampled from a CSR topology, no full-graph BCSR) as through the
    exactly sized blocks of the hop-by-hop path; the transposed blocks are built without read-backs."""
    from graph_rws_b200 import BCSRGraph, GCN_BCSR
    from graph_rws_b200.data import CSRTopology
    from graph_rws_b200.sampler import BCSRSampler
    dev = torch.device("cuda")
    g = BCSRGraph.from_csr(graph.num_nodes, graph.row_ptr, graph.col_idx, graph.values, device=dev)
    topo = CSRTopology(*_dev_csr(graph))
    x = torch.randn(graph.num_nodes, 24, generator=torch.Generator().manual_seed(3)).to(dev)
    seeds = torch.arange(7, 2007, 10, dtype=torch.int32)
    torch.manual_seed(5)
    model = GCN_BCSR(24, 32, 5, num_layers=3, dropout=0.0, use_checkpoint=False).to(dev)
    out = []
    for sampler, gg in ((BCSRSampler([6, 4, 3], verbose=False, seed=9, fused=False), g),
                        (BCSRSampler([6, 4, 3], verbose=False, seed=9, fused=True, pad_to=256), topo)):
        blocks = sampler.sample_layers(gg, seeds)
        ids = blocks[0].input_nodes.clamp(min=0)
        model.zero_grad(set_to_none=True)
        logits = model(blocks, x[ids.long()])[:seeds.numel()]
        logits.square().sum().backward()
        out.append((logits.detach().clone(), [p.grad.clone() for p in model.parameters()]))
    torch.testing.assert_close(out[0][0], out[1][0], rtol=2e-3, atol=2e-3)      # TF32 products, other summation order
    for a, b in zip(out[0][1], out[1][1]):
        torch.testing.assert_close(a, b, rtol=5e-3, atol=5e-3)


def test_first_block_with_global_ids_equals_gathered_rows(graph):
    """helper.layer0_inputs: reading the feature rows in place through global column ids gives the
    logits and weight gradients of the gather-then-multiply path."""
    from graph_rws_b200 import GCN_BCSR
    from graph_rws_b200.data import CSRTopology
    from graph_rws_b200.helper import layer0_inputs
    from graph_rws_b200.sampler import BCSRSampler
    dev = torch.device("cuda")
    topo = CSRTopology(*_dev_csr(graph), block_dtype=torch.float16)
    x = torch.randn(graph.num_nodes, 128, generator=torch.Generator().manual_seed(3)).half().to(dev)
    seeds = torch.arange(3, 1803, 9, dtype=torch.int32)
    torch.manual_seed(6)
    model = GCN_BCSR(128, 128, 7, num_layers=3, dropout=0.0, use_checkpoint=False).to(dev).half()
    blocks = BCSRSampler([5, 4, 3], verbose=False, seed=3, pad_to=256).sample_layers(topo, seeds)
    out = []
    for bl, xx in ((blocks, x[blocks[0].input_nodes.clamp(min=0).long()]), layer0_inputs(blocks, x)):
        model.zero_grad(set_to_none=True)
        logits = model(bl, xx)[:seeds.numel()]
        logits.float().square().sum().backward()
        out.append((logits.detach().float(), [p.grad.float().clone() for p in model.parameters()]))
    torch.testing.assert_close(out[0][0], out[1][0], rtol=1e-2, atol=1e-2)
    for a, b in zip(out[0][1], out[1][1]):
        torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2)


def test_two_branch_graph_step_trains_like_the_one_chain_graph_step(graph):
    """helper.graphed_sampled_step: with ``pipelined=True`` the sampler of the next batch runs as a
    second branch of the graph that trains on the current one.  Batch by batch the losses are those
    of the one-chain graph (sampling depends on seeds and step index only), one call later."""
    import copy
    from graph_rws_b200 import GCN_BCSR
    from graph_rws_b200.data import CSRTopology
    from graph_rws_b200.helper import graphed_sampled_step
    from graph_rws_b200.sampler import BCSRSampler
    dev = torch.device("cuda")
    n = graph.num_nodes
    topo = CSRTopology(*_dev_csr(graph), block_dtype=torch.float16)
    x = torch.randn(n, 128, generator=torch.Generator().manual_seed(3)).half().to(dev)
    y = torch.randint(0, 7, (n,), generator=torch.Generator().manual_seed(4)).to(dev)
    torch.manual_seed(6)
    base = GCN_BCSR(128, 128, 7, num_layers=3, dropout=0.0, use_checkpoint=False).to(dev).half()
    batches = [((torch.arange(256) * 7 + 3 + 11 * i) % n).to(torch.int32).to(dev) for i in range(5)]
    losses = {}
    for mode in ("chain", "branches"):
        model = copy.deepcopy(base)
        opt = torch.optim.Adam(model.parameters(), lr=1e-3, eps=1e-4, capturable=True)
        sampler = BCSRSampler([5, 4, 3], verbose=False, seed=3, pad_to=256)
        step = graphed_sampled_step(model, sampler, topo, x, y, opt, 256, pipelined=(mode == "branches"))
        out = []
        if mode == "chain":
            for i, b in enumerate(batches[:4]):
                out.append(float(step(b, i)))
        else:
            step.prime(batches[0], 0)
            for i in range(1, 5):
                out.append(float(step(batches[i], i)))      # the loss of batch i - 1
        losses[mode] = out
    torch.cuda.synchronize()
    assert all(np.isfinite(losses["chain"]))
    np.testing.assert_allclose(losses["branches"], losses["chain"], rtol=2e-3, atol=2e-3)


def test_full_size_sampled_blocks_have_the_sampling_properties():
    """The sampled workload at its stated size (2,449,029 nodes, 126 M CSR entries, fan-out 15-10-5,
    1,024 seeds), where the host replay would take minutes: properties that hold whatever the size.
    Every row of a block holds min(degree, fan-out) distinct neighbours of its node with the graph's
    weights; the source list starts with the destination nodes and continues with new ids in
    ascending order; the frontier of the next hop is that source list, padding entries included."""
    from graph_rws_b200.core.sampling import bcsr_to_csr
    from graph_rws_b200.data import CSRTopology, synthetic
    from graph_rws_b200.sampler import BCSRSampler
    dev = torch.device("cuda")
    n, e = 2449029, 61_860_000
    rp, ci, vv = synthetic.chung_lu_csr_torch(n, e, 2.5, 1004, dev)
    topo = CSRTopology(rp, ci, vv, device=dev, block_dtype=torch.float32)
    rows_of = torch.repeat_interleave(torch.arange(n, device=dev), rp[1:] - rp[:-1])
    graph_keys = rows_of * n + ci.long()                  # sorted: rows ascending, columns ascending in a row
    assert bool((graph_keys[1:] > graph_keys[:-1]).all())
    deg = (rp[1:] - rp[:-1])
    seeds = torch.randperm(n, generator=torch.Generator().manual_seed(12))[:1024].to(torch.int32).to(dev)
    fanouts = [15, 10, 5]
    blocks = BCSRSampler(fanouts, verbose=False, seed=77, pad_to=256).sample_layers(topo, seeds)
    assert torch.equal(blocks[-1].output_nodes[:1024], seeds)
    for b, fanout in zip(blocks, fanouts):               # blocks run input -> output, like the model's layers
        dst, src = b.output_nodes.long(), b.input_nodes.long()
        real = dst >= 0                               # a frontier has -1 entries wherever the list above it had them
        # source list: the destination list as it is, then new ids ascending, then padding
        assert torch.equal(src[:dst.numel()], dst)
        tail = src[dst.numel():]
        n_new = int((tail >= 0).sum())
        assert bool((tail[:n_new] >= 0).all()) and bool((tail[1:n_new] > tail[:n_new - 1]).all())
        assert torch.unique(src[src >= 0]).numel() == int((src >= 0).sum()), "a node appears once"
        # the block's entries as (row, global column, weight)
        brp, bci, bvv = bcsr_to_csr(b.window_offset, b.original_col_indices, b.values_condensed, dst.numel())
        cnt = brp[1:] - brp[:-1]
        want = torch.minimum(deg[dst.clamp(min=0)], torch.tensor(fanout, device=dev))
        assert torch.equal(cnt, torch.where(real, want, torch.zeros_like(want)))
        rows = torch.repeat_interleave(torch.arange(dst.numel(), device=dev), cnt)
        u = src[bci.long()]
        assert bool((u >= 0).all())
        keys = dst[rows] * n + u
        pos = torch.searchsorted(graph_keys, keys)
        assert bool((graph_keys[pos.clamp(max=graph_keys.numel() - 1)] == keys).all()), "a sampled edge is not in the graph"
        assert torch.equal(bvv, vv[pos]), "weights are the graph's"
        # (row, column) pairs are distinct: rows of the CSR view ascend strictly in column id
        same_row = rows[1:] == rows[:-1]
        assert bool((bci[1:][same_row] > bci[:-1][same_row]).all())
    for lower, upper in zip(blocks[1:], blocks[:-1]):     # the frontier of a hop is the source list of the hop above it
        assert torch.equal(upper.output_nodes, lower.input_nodes)
