"""BCSRGraphConv / GCN_BCSR over the CUDA path against the same algebra with a dense fp32 adjacency."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small():
    from graph_rws_b200 import BCSRGraph
    from graph_rws_b200.data import synthetic
    g = synthetic.graph_for_config("small_gcn")
    dev = torch.device("cuda")
    graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev)
    A = torch.zeros(g.num_nodes, g.num_nodes, dtype=torch.float64)
    rows = np.repeat(np.arange(g.num_nodes), np.diff(g.row_ptr))
    A[torch.from_numpy(rows), torch.from_numpy(g.col_idx.astype(np.int64))] = torch.from_numpy(g.values).double()
    return g, graph, A.to(dev)


def test_graphconv_forward_backward_matches_dense(small):
    from graph_rws_b200 import BCSRGraphConv
    g, graph, A = small
    torch.manual_seed(0)
    layer = BCSRGraphConv(48, 24).cuda()
    x = torch.randn(g.num_nodes, 48, device="cuda", requires_grad=True)
    # called on its own the layer returns whole windows (W*16 rows), like the reference's
    # (layers/layer.py:157-165 pads the self path); the model trims through features_target
    out = layer(graph, x)
    assert out.shape == (graph.num_windows * 16, 24)
    out = out[:g.num_nodes]
    xd = x.detach().double().requires_grad_(True)
    wn, ws = layer.weight_neigh.detach().double().requires_grad_(True), layer.weight_self.detach().double().requires_grad_(True)
    ref = A @ (xd @ wn) + xd @ ws
    # operands are rounded to TF32 inside the SpMM, like the reference kernel
    assert torch.allclose(out.double(), ref, rtol=2e-2, atol=2e-3)
    go = torch.randn_like(out)
    out.backward(go)
    ref.backward(go.double())
    for got, want in ((x.grad, xd.grad), (layer.weight_neigh.grad, wn.grad), (layer.weight_self.grad, ws.grad)):
        err = (got.double() - want).norm() / want.norm()
        assert err < 5e-3, err
    # the transposed graph was built once and is reused
    assert graph.transposed(g.num_nodes, dtype=torch.float32) is graph.transposed(g.num_nodes, dtype=torch.float32)


def test_gcn_full_graph_training_step(small):
    """Config-1-shaped run: 2-layer GCN, hidden 16, 7 classes, one full-batch step; loss goes down."""
    from graph_rws_b200 import GCN_BCSR
    g, graph, A = small
    torch.manual_seed(1)
    x = (torch.rand(g.num_nodes, 1440, device="cuda") < 0.013).float()
    y = torch.randint(0, 7, (g.num_nodes,), device="cuda")
    model = GCN_BCSR(1440, 16, 7, num_layers=2, dropout=0.0, use_checkpoint=True).cuda()
    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        logits = model(graph, x)
        assert logits.shape == (g.num_nodes, 7)
        loss = torch.nn.functional.cross_entropy(logits, y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    with torch.no_grad():
        # inference() calls the layers without aligned self features, so it returns whole windows,
        # as the reference's does (models/model.py:268-285)
        assert model.inference(graph, x).shape == (graph.num_windows * 16, 7)
    # parameter names interchange with the reference's checkpoints
    names = set(model.state_dict())
    assert {"layers.0.weight_neigh", "layers.1.weight_self", "norms.0.weight"} <= names


def test_sampled_blocks_train_a_gcn():
    """Blocks from BCSRSampler feed GCN_BCSR through its target-first slicing path; half-precision
    tiles and features take the tcgen05 kernel for the 128/256-wide layers."""
    from graph_rws_b200 import BCSRGraph, GCN_BCSR
    from graph_rws_b200.data import synthetic
    from graph_rws_b200.sampler import BCSRSampler
    g = synthetic.sym_normalized_csr(20000, *synthetic.chung_lu_edges(20000, 200000, 2.5, 77))
    dev = torch.device("cuda")
    graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev)
    X = torch.randn(g.num_nodes, 100, device=dev)
    Y = torch.randint(0, 47, (g.num_nodes,), device=dev)
    model = GCN_BCSR(100, 256, 47, num_layers=3, dropout=0.0, use_checkpoint=False).cuda()
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    sampler = BCSRSampler([15, 10, 5], verbose=False)
    seeds = torch.randperm(g.num_nodes, device=dev)[:512].int()
    blocks = sampler.sample_layers(graph, seeds)
    assert [b.num_rows for b in blocks][-1] == 512
    feats = X[blocks[0].input_nodes.long()]
    losses = []
    for _ in range(5):
        opt.zero_grad()
        logits = model(blocks, feats)[:seeds.numel()]
        loss = torch.nn.functional.cross_entropy(logits, Y[seeds.long()])
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert np.isfinite(losses).all() and losses[-1] < losses[0]


def test_pipelined_epoch_equals_serial_epoch():
    """The producer-thread / side-stream epoch trains on the same batches as the serial one: the
    sampler is keyed by (seed, node, hop, step), so both orders of execution see identical blocks
    and the mean losses agree."""
    import copy
    from graph_rws_b200 import BCSRGraph, GCN_BCSR
    from graph_rws_b200.data import synthetic
    from graph_rws_b200.helper import train_epoch_node_sampling
    from graph_rws_b200.sampler import BCSRSampler
    g = synthetic.sym_normalized_csr(20000, *synthetic.chung_lu_edges(20000, 200000, 2.5, 78))
    dev = torch.device("cuda")
    graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev)
    X = torch.randn(g.num_nodes, 100, device=dev)
    Y = torch.randint(0, 47, (g.num_nodes,), device=dev)
    train_idx = torch.randperm(g.num_nodes, device=dev)[:2048]
    torch.manual_seed(9)
    model_a = GCN_BCSR(100, 128, 47, num_layers=3, dropout=0.0, use_checkpoint=False).cuda()
    model_b = copy.deepcopy(model_a)
    out = []
    for model, pipe in ((model_a, False), (model_b, True)):
        opt = torch.optim.SGD(model.parameters(), lr=0.05)
        sampler = BCSRSampler([10, 5, 5], verbose=False, seed=4)
        loss, seen = train_epoch_node_sampling(model, graph, X, Y, train_idx, opt, sampler, batch_size=512, pipeline=pipe)
        torch.cuda.synchronize()
        assert seen == 2048
        out.append(float(loss))
    assert np.isfinite(out).all()
    assert abs(out[0] - out[1]) < 1e-3 * abs(out[0]), out
    for pa, pb in zip(model_a.parameters(), model_b.parameters()):
        assert torch.allclose(pa, pb, rtol=1e-3, atol=1e-4)


def test_window_style_graphs_with_active_windows(oracle, small):
    """Graphs in the reference sampler's format -- rows are whole 16-row windows of the global graph,
    column ids are global, ``active_windows`` names the windows (sampler/sampler.py:261-277) -- go
    through the model's window branches: the layer-0 self rows gathered by window, the per-layer
    ``reindex_bcsr`` against the previous graph's windows, the window lookup of the later self rows
    (models/model.py:118-143,183-194).  With every tile of the chosen windows kept, the result on
    those windows equals the full-graph forward pass."""
    from graph_rws_b200 import BCSRGraph, GCN_BCSR
    g, graph, A = small
    dev = torch.device("cuda")
    wo = graph.window_offset.cpu().numpy()
    cols = graph.original_col_indices.cpu().numpy().reshape(-1, 8)
    vals = graph.values_condensed.cpu().numpy().reshape(-1, 128)

    def window_subgraph(wins):
        tiles = np.concatenate([np.arange(wo[w], wo[w + 1]) for w in wins])
        sub_wo = np.concatenate([[0], np.cumsum([wo[w + 1] - wo[w] for w in wins])]).astype(np.int64)
        sub = BCSRGraph.from_components(torch.from_numpy(sub_wo).to(dev), torch.from_numpy(cols[tiles].reshape(-1)).to(dev),
                                        torch.from_numpy(vals[tiles].reshape(-1)).to(dev), num_rows=len(wins) * 16,
                                        num_cols=g.num_nodes, tile_rows=16, tile_cols=8, device=dev)
        sub.active_windows = torch.from_numpy(np.asarray(wins, dtype=np.int32)).to(dev)
        return sub

    seeds = np.random.default_rng(2).permutation(2600)[:40].astype(np.int32)
    win1, masks = oracle.windows_and_masks(seeds)                   # sorted unique windows of the seeds
    assert win1.size < seeds.size + 1 and (np.diff(win1) > 0).all() and masks.size == win1.size
    g1 = window_subgraph(win1)
    c1 = g1.original_col_indices.cpu().numpy()
    win0 = np.unique(c1[c1 >= 0] // 16).astype(np.int32)           # every window the output layer reads from
    assert np.isin(win1, win0).all()                                # self-loops: a window is among its own sources
    g0 = window_subgraph(win0)
    torch.manual_seed(4)
    model = GCN_BCSR(40, 24, 5, num_layers=2, dropout=0.0, use_checkpoint=False).to(dev)
    x = torch.randn(g.num_nodes, 40, generator=torch.Generator().manual_seed(5)).to(dev)
    model.eval()
    with torch.no_grad():
        full = model(graph, x)                                     # [num_nodes, 5], checked against dense algebra above
        sub = model([g0, g1], x)
    assert sub.shape == (win1.size * 16, 5)
    rows = (win1[:, None].astype(np.int64) * 16 + np.arange(16)[None, :]).reshape(-1)
    keep = rows < g.num_nodes
    got, want = sub[torch.from_numpy(np.nonzero(keep)[0]).to(dev)], full[torch.from_numpy(rows[keep]).to(dev)]
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-3), float((got - want).abs().max())
    # the output layer's column ids were localised against the first graph's windows
    assert int(g1.original_col_indices.max()) < win0.size * 16
