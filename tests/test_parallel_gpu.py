"""Row-partitioned SpMM and sharded-feature exchange on two GPUs over NCCL (skipped with fewer)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from graph_rws_b200 import BCSRGraph, core
        from graph_rws_b200.data import synthetic
        from graph_rws_b200.parallel import DistributedSpMM, exchange_rows, partition_windows_by_tiles
        g = synthetic.sym_normalized_csr(9000, *synthetic.chung_lu_edges(9000, 120000, 2.2, 13))
        graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev, values_dtype=torch.float16)
        H = torch.randn(g.num_nodes, 128, generator=torch.Generator().manual_seed(4)).half().to(dev)
        full = core.spmm_raw(graph.window_offset, graph.original_col_indices, graph.values_condensed, H)[:g.num_nodes]
        part = partition_windows_by_tiles(graph.window_offset, world, num_rows=g.num_nodes)
        lo, hi = part.rows(rank)
        local = DistributedSpMM(graph, part, rank)(H[lo:hi].contiguous())
        # the shard cuts its tile array at other places than the full graph does, so windows that
        # are split between CTAs are summed in other groupings: equal up to fp32 rounding and the
        # final fp16 rounding
        err = (local.float() - full[lo:hi].float()).norm() / full[lo:hi].float().norm()
        assert err < 1e-3, float(err)
        # feature rows sharded in contiguous blocks, fetched by global id with all_to_all_single
        per = (g.num_nodes + world - 1) // world
        ids = torch.randint(0, g.num_nodes, (5000,), generator=torch.Generator().manual_seed(rank)).int().to(dev)
        rows = exchange_rows(H[rank * per:(rank + 1) * per].contiguous(), ids, g.num_nodes)
        assert torch.equal(rows, H[ids.long()])
        torch.cuda.synchronize()
        out[rank] = 1
    finally:
        dist.destroy_process_group()


def _gcn_worker(rank, world, port, out):
    """Row-sharded full-graph GCN step == the single-GPU step: loss, logits, weight gradients."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import torch.nn.functional as F
        from graph_rws_b200 import BCSRGraph, GCN_BCSR
        from graph_rws_b200.data import synthetic
        from graph_rws_b200.helper.engine import _allreduce_grads
        from graph_rws_b200.parallel import RowShardedGraph, partition_windows_by_tiles
        n = 7003                                            # last window is partial
        g = synthetic.sym_normalized_csr(n, *synthetic.chung_lu_edges(n, 90000, 2.2, 5))
        graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev, values_dtype=torch.float16)
        gen = torch.Generator().manual_seed(8)
        X = torch.randn(n, 64, generator=gen).to(dev)
        y = torch.randint(0, 10, (n,), generator=gen).to(dev)
        train = torch.randperm(n, generator=gen)[:3000].sort().values.to(dev)
        torch.manual_seed(3)
        # checkpointing re-runs a layer's all-gather in backward: the same setting on every rank
        model = GCN_BCSR(64, 128, 10, 3, dropout=0.0, use_checkpoint=True).to(dev)
        for p in model.parameters():
            dist.broadcast(p.data, 0)

        def grads():
            return torch.cat([p.grad.reshape(-1) for p in model.parameters()]).clone()

        ref_logits = model(graph, X)                     # fp32 features: the TF32 warp-MMA kernel
        ref_loss = F.cross_entropy(ref_logits[train].float(), y[train])
        ref_loss.backward()
        ref_grads = grads()
        model.zero_grad(set_to_none=True)

        part = partition_windows_by_tiles(graph.window_offset, world, num_rows=n)
        lo, hi = part.rows(rank)
        # the all-gathers of the layers go through the library's own NVLink kernels (rows of up to 512 bytes)
        from graph_rws_b200.parallel import make_peer_all_gather
        part.peer_gather = make_peer_all_gather(part.max_rows(), 512, dev, keep_if_slower=True)
        assert part.peer_gather is not None, "these GPUs address each other's memory: the peer all-gather must come up"
        shard = RowShardedGraph.from_full(graph, part, rank, peer_row_bytes=512)
        mine = train[(train >= lo) & (train < hi)] - lo
        logits = model(shard, X[lo:hi].contiguous())
        assert logits.shape[0] == hi - lo
        loss = F.cross_entropy(logits[mine].float(), y[lo:hi][mine], reduction='sum') / train.numel()
        loss.backward()
        _allreduce_grads(model, average=False)
        dist.all_reduce(loss)
        assert (logits.float() - ref_logits[lo:hi].float()).norm() / ref_logits[lo:hi].float().norm() < 5e-3
        assert abs(float(loss) - float(ref_loss)) < 2e-3 * abs(float(ref_loss))
        assert (grads() - ref_grads).norm() / ref_grads.norm() < 2e-2
        part.peer_gather.check()
        torch.cuda.synchronize()
        out[rank] = 1
    finally:
        dist.destroy_process_group()


def _peer_gather_worker(rank, world, port, out):
    """parallel.PeerAllGather == all_gather_into_tensor on zero-padded shards: uneven shards, two
    widths, eagerly and as replays of one CUDA graph with new inputs every time."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from graph_rws_b200.parallel import make_peer_all_gather
        pad_rows = 4099
        gen = torch.Generator(device=dev).manual_seed(100 + rank)
        for push in (True, False):
            _peer_gather_checks(make_peer_all_gather(pad_rows, 512, dev, push=push, keep_if_slower=True), pad_rows, world, rank, dev, gen)
        out[rank] = 1
    finally:
        dist.destroy_process_group()


def _peer_gather_checks(pg, pad_rows, world, rank, dev, gen):
    assert pg is not None

    def reference(local):
        send = torch.zeros((pad_rows, local.shape[1]), dtype=local.dtype, device=dev)
        send[:local.shape[0]] = local
        want = torch.empty((world * pad_rows, local.shape[1]), dtype=local.dtype, device=dev)
        dist.all_gather_into_tensor(want, send)
        return want

    for i, (rows, width, dtype) in enumerate([(pad_rows, 256, torch.bfloat16), (pad_rows - 17 * rank, 48, torch.float16),
                                              (pad_rows - 3, 128, torch.float32), (1, 8, torch.float16)]):
        local = torch.randn((rows, width), generator=gen, device=dev).to(dtype)
        assert torch.equal(pg.gather(local), reference(local)), f"exchange {i}"
    # replays of a captured sequence of three exchanges; the inputs change between replays
    bufs = [torch.zeros((pad_rows - rank, 256), dtype=torch.bfloat16, device=dev),
            torch.zeros((pad_rows, 48), dtype=torch.bfloat16, device=dev),
            torch.zeros((pad_rows - 5, 256), dtype=torch.bfloat16, device=dev)]
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for b in bufs:
            pg.gather(b)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = [pg.gather(b).clone() for b in bufs]      # (the push form returns its inbox: valid until the next exchange)
    for step in range(4):
        for b in bufs:
            b.copy_(torch.randn(b.shape, generator=gen, device=dev).to(b.dtype))
        graph.replay()
        torch.cuda.synchronize()
        for b, o in zip(bufs, outs):
            assert torch.equal(o, reference(b)), f"replay {step}"
    pg.check()


def _sampled_worker(rank, world, port, out):
    """Seed-sharded sampled step with the feature rows sharded over the ranks: the rows a rank reads
    from its peers' memory equal the rows of the full matrix, the blocks a rank samples equal the
    blocks one GPU samples for the same seeds (keyed Philox), and a data-parallel step runs."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from graph_rws_b200 import GCN_BCSR
        from graph_rws_b200.data import CSRTopology, synthetic
        from graph_rws_b200.helper import train_step_sampled
        from graph_rws_b200.parallel import ShardedFeatures, shard_seeds
        from graph_rws_b200.sampler import BCSRSampler
        g = synthetic.sym_normalized_csr(12000, *synthetic.chung_lu_edges(12000, 150000, 2.3, 19))
        topo = CSRTopology(torch.from_numpy(g.row_ptr), torch.from_numpy(g.col_idx), torch.from_numpy(g.values), device=dev,
                           block_dtype=torch.float16)
        n = g.num_nodes
        X = torch.randn(n, 128, generator=torch.Generator().manual_seed(4)).half().to(dev)
        per = (n + world - 1) // world
        store = ShardedFeatures(X[rank * per:(rank + 1) * per].contiguous(), n)
        ids = torch.randint(-1, n, (7000,), generator=torch.Generator().manual_seed(rank)).int().to(dev)
        rows = store.gather(ids)
        want = X[ids.clamp(min=0).long()]
        want[ids < 0] = 0
        assert torch.equal(rows, want)
        # the blocks of this rank's seeds do not depend on the rank count
        all_seeds = torch.randperm(n, generator=torch.Generator().manual_seed(8))[:1024].int().to(dev)
        mine = shard_seeds(all_seeds, rank, world)
        sampler = BCSRSampler([6, 4, 3], verbose=False, seed=21, pad_to=256)
        blocks = sampler.sample_layers(topo, mine)
        whole = sampler.sample_layers(topo, all_seeds)
        lo = (all_seeds.numel() * rank) // world
        # per-node neighbour lists are keyed by (seed, node, hop): the first-hop sources of this
        # rank's seeds are a subset of what the one-GPU batch reaches
        assert set(blocks[-1].input_nodes[blocks[-1].input_nodes >= 0].tolist()) <= \
            set(whole[-1].input_nodes[whole[-1].input_nodes >= 0].tolist())
        assert torch.equal(blocks[-1].output_nodes, all_seeds[lo:lo + mine.numel()])
        torch.manual_seed(5)
        model = GCN_BCSR(128, 64, 7, num_layers=3, dropout=0.0, use_checkpoint=False).to(dev).half()
        for p_ in model.parameters():
            dist.broadcast(p_.data, 0)
        y = torch.randint(0, 7, (n,), generator=torch.Generator().manual_seed(9)).to(dev)
        opt = torch.optim.SGD(model.parameters(), lr=0.01)
        loss = train_step_sampled(model, sampler, topo, None, y, mine, opt, fetch_rows=store)
        assert torch.isfinite(loss).item()
        # after the gradient all-reduce every rank holds the same weights
        w = torch.cat([p_.detach().float().reshape(-1) for p_ in model.parameters()])
        ws = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(ws, w)
        assert torch.equal(ws[0], ws[1])
        torch.cuda.synchronize()
        out[rank] = 1
    finally:
        dist.destroy_process_group()


def _run(worker):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Array("i", world)
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    for p in procs:
        if p.is_alive():            # a rank stuck in a collective: end exactly the processes started here
            p.kill()
            p.join()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(out) == [1] * world


def test_row_partitioned_spmm_and_row_exchange_on_two_gpus():
    _run(_worker)


def test_row_sharded_gcn_step_matches_single_gpu():
    _run(_gcn_worker)


def test_sampled_step_with_features_read_from_peer_memory():
    _run(_sampled_worker)


def test_peer_all_gather_matches_the_collective():
    _run(_peer_gather_worker)
