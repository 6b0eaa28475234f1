"""Minimal training steps: the callers that turn kernel throughput into "epoch ms" and "seeds/s".

Restates, for the two modes the hot path serves, the reference's ``train_epoch_full``
(helper/engine.py:44-83) and the consumer half of ``train_epoch_node_sampling``
(helper/engine.py:156-201): forward, cross-entropy on the training rows, backward, gradient-norm
clipping at 1.0, optimizer step.  With per-node sampled blocks the seed -> logit-row mapping of
helper/engine.py:175-183 (a searchsorted over ``active_windows``) becomes the identity on the first
``len(seeds)`` rows.  Data-parallel ranks all-reduce the gradients (NCCL) before the step.
"""
import queue
import threading

import torch
import torch.distributed as dist
import torch.nn.functional as F


class _FlatGrads:
    """All gradients of a model as views into one flat buffer, so that the data-parallel all-reduce
    is a single collective on that buffer with no gather / scatter passes around it."""

    def __init__(self, params):
        self.params = [p for p in params if p.requires_grad]
        dtype, device = self.params[0].dtype, self.params[0].device
        self.flat = torch.zeros(sum(p.numel() for p in self.params), dtype=dtype, device=device)
        off = 0
        for p in self.params:
            p.grad = self.flat[off:off + p.numel()].view_as(p)
            off += p.numel()

    def valid(self):
        return all(p.grad is not None and p.grad.untyped_storage().data_ptr() == self.flat.untyped_storage().data_ptr()
                   for p in self.params)


def _flat_grads(model):
    params = list(model.parameters())
    fg = getattr(model, '_grws_flat_grads', None)
    if fg is None or not fg.valid() or len({p.dtype for p in params}) != 1:
        if len({p.dtype for p in params}) != 1 or not params:
            return None
        fg = _FlatGrads(params)
        try:
            model._grws_flat_grads = fg
        except AttributeError:
            pass
    return fg


def _zero_grads(model, optimizer):
    """Gradients := 0, kept as views of one flat buffer when the model allows it."""
    fg = _flat_grads(model) if hasattr(model, 'parameters') else None
    if fg is None:
        optimizer.zero_grad(set_to_none=True)
    else:
        fg.flat.zero_()


def _allreduce_grads(model, group=None, average=True):
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    from ..parallel.row_partition import collective_timers
    fg = getattr(model, '_grws_flat_grads', None)
    if fg is not None and fg.valid():
        with collective_timers.timed("all_reduce", fg.flat.device):
            dist.all_reduce(fg.flat, group=group)
        if average:
            fg.flat /= dist.get_world_size(group)
        return
    grads = [p.grad for p in model.parameters() if p.grad is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1) for g in grads])
    with collective_timers.timed("all_reduce", flat.device):
        dist.all_reduce(flat, group=group)
    if average:
        flat /= dist.get_world_size(group)
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()


def train_step_full(model, graph, features, labels, train_idx, optimizer):
    """One full-graph epoch (= one step); returns the loss tensor (no host sync)."""
    model.train()
    _zero_grads(model, optimizer)
    logits = model(graph, features)
    loss = F.cross_entropy(logits[train_idx].float(), labels[train_idx])
    loss.backward()
    _allreduce_grads(model)
    torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
    optimizer.step()
    return loss.detach()


def train_step_full_sharded(model, graph, features_local, labels_local, train_idx_local, num_train, optimizer):
    """One full-graph epoch with the rows of the graph, features and labels sharded over the ranks
    (``graph`` is a parallel.RowShardedGraph).  The loss is the global mean over ``num_train``
    training rows: every rank sums its own rows' terms, so the weight gradients ADD across ranks."""
    model.train()
    _zero_grads(model, optimizer)
    logits = model(graph, features_local)
    loss = F.cross_entropy(logits[train_idx_local].float(), labels_local[train_idx_local], reduction='sum') / num_train
    loss.backward()
    _allreduce_grads(model, average=False)
    torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
    optimizer.step()
    return loss.detach()


def layer0_inputs(blocks, features, fetch_rows=None):
    """(blocks, x) to hand to the model for a sampled step.

    With sharded features the rows of the input nodes are fetched (``fetch_rows``: the real node ids
    only, padding entries get zero rows).  With the whole feature matrix on this GPU nothing is
    gathered at all: the first block gets its column ids rewritten to global node ids (one gather
    over the block's ids) and the product reads the feature rows in place -- the reference
    multiplies and gathers over every row of the matrix instead (layers/layer.py:40,
    helper/engine.py:170-171)."""
    import copy
    b0 = blocks[0]
    if fetch_rows is not None:
        ids = b0.input_nodes
        if hasattr(fetch_rows, 'gather'):           # a row store that takes padding ids itself (zero rows)
            return blocks, fetch_rows.gather(ids)
        real = ids >= 0
        rows = fetch_rows(ids[real])
        x = torch.zeros((ids.numel(), rows.shape[1]), dtype=rows.dtype, device=rows.device)
        x[real] = rows
        return blocks, x
    g0 = copy.copy(b0)
    cols = b0.original_col_indices
    g0.original_col_indices = torch.where(cols >= 0, b0.input_nodes[cols.clamp(min=0).long()], cols)
    g0.self_rows = b0.output_nodes.clamp(min=0).long()
    g0.num_cols = features.shape[0]
    g0._shared = {}
    return [g0] + list(blocks[1:]), features


def train_step_sampled(model, sampler, graph, features, labels, seeds, optimizer, fetch_rows=None):
    """One mini-batch step: sample the blocks for ``seeds``, gather the input rows, train.

    ``fetch_rows(node_ids)`` supplies feature rows when they are sharded across ranks
    (parallel.exchange_rows); by default they are indexed from the local ``features``."""
    model.train()
    blocks, x = layer0_inputs(sampler.sample_layers(graph, seeds), features, fetch_rows)
    _zero_grads(model, optimizer)
    logits = model(blocks, x)[:seeds.numel()]
    loss = F.cross_entropy(logits.float(), labels[seeds.long()])
    loss.backward()
    _allreduce_grads(model)
    torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
    optimizer.step()
    return loss.detach()


class GraphedStep:
    """A training step captured once as a CUDA graph and replayed: the whole step -- sampling, block
    build, forward, backward, gradient all-reduce, clipping, optimizer -- becomes one graph launch.

    A sampled step queues a few hundred small kernels; issued one by one from the interpreter they
    take longer to issue than to run.  Everything in the step has fixed shapes (the fused sampler
    sizes its blocks by bounds) and reads what changes from step to step -- the seeds, the Philox
    seed -- from device buffers, so the recorded launch sequence is valid for every step.

    ``body()`` runs one step on static inputs and returns the loss tensor; the optimizer must be
    capturable (``torch.optim.Adam(..., capturable=True)``).  The first calls run eagerly on a
    side stream (libraries pick their algorithms, the allocator warms up, this library looks up
    its device symbols), then the body is captured."""

    def __init__(self, body, device, warmup: int = 3):
        self.body = body
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                body()
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = body()

    def replay(self):
        self.graph.replay()
        return self.loss


def _block_tensors(blocks):
    """The device allocations behind a list of sampled blocks, each once: the fused sampler carves a
    step's arrays out of three allocations (ids, values, offsets), so copying a batch is a handful
    of large copies rather than one per array."""
    seen, out = set(), []
    for b in blocks:
        for t in (b.window_offset, b.original_col_indices, b.values_condensed, b.output_nodes, b.input_nodes):
            base = t._base if t._base is not None else t
            if base.data_ptr() not in seen:
                seen.add(base.data_ptr())
                out.append(base)
    return out


def graphed_sampled_step(model, sampler, graph, features, labels, optimizer, num_seeds, fetch_rows=None, warmup=3,
                         pipelined=False):
    """``step(seeds, step_index) -> loss`` for sampled training, as one CUDA graph per step.

    ``pipelined=True`` overlaps the sampler with the training: the graph of a step has two branches,
    one trains on the blocks sampled during the previous step, the other samples and builds the
    blocks for the seeds passed to this call (the reference overlaps the two with a producer thread
    and a side stream, helper/engine.py:196-260; here both are branches of one graph launch, so the
    GPU runs the sampler's small kernels in the gaps of the training's).  ``step`` then returns the
    loss of the batch given to the PREVIOUS call; ``step.prime(seeds, step_index)`` samples the
    first batch.  Results per batch are the same as without pipelining: sampling depends on the
    seeds and the step index only."""
    device = labels.device
    seeds_buf = torch.zeros(num_seeds, dtype=torch.int32, device=device)
    seed_dev = torch.zeros(1, dtype=torch.int64, device=device)          # the Philox seed, read by the sampling kernels
    model.train()

    def train_on(blocks, seeds):
        blocks, x = layer0_inputs(blocks, features, fetch_rows)
        _zero_grads(model, optimizer)
        logits = model(blocks, x)[:num_seeds]
        loss = F.cross_entropy(logits.float(), labels[seeds.long()])
        loss.backward()
        _allreduce_grads(model)
        torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
        optimizer.step()
        return loss.detach()

    if not pipelined:
        def body():
            return train_on(sampler.sample_layers(graph, seeds_buf, seed_dev=seed_dev), seeds_buf)

        graphed = GraphedStep(body, device, warmup)

        def step(seeds, step_index=0):
            seeds_buf.copy_(seeds, non_blocking=True)
            seed_dev.fill_(int(sampler.seed) + int(step_index))
            return graphed.replay()
        step.graphed = graphed
        return step

    # the batch being trained on lives in arrays of its own, outside the graph's memory pool; the
    # sampler branch fills fresh arrays, which are copied over once both branches are done
    seeds_cur = torch.zeros(num_seeds, dtype=torch.int32, device=device)
    blocks_cur = sampler.sample_layers(graph, seeds_cur, seed_dev=seed_dev)
    cur_tensors = _block_tensors(blocks_cur)
    side = torch.cuda.Stream(device)
    keep = {}

    def body():
        main = torch.cuda.current_stream(device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            blocks_next = sampler.sample_layers(graph, seeds_buf, seed_dev=seed_dev)
        for b in blocks_cur:
            b._shared.clear()                  # transposed blocks of the previous batch
        loss = train_on(blocks_cur, seeds_cur)
        main.wait_stream(side)
        nxt = _block_tensors(blocks_next)
        assert len(nxt) == len(cur_tensors)
        for dst, src in zip(cur_tensors, nxt):
            dst.copy_(src)
        seeds_cur.copy_(seeds_buf)
        keep['next'] = blocks_next             # the sampler branch's arrays stay allocated as long as the graph
        return loss

    graphed = GraphedStep(body, device, warmup)

    def prime(seeds, step_index=0):
        seeds_cur.copy_(seeds, non_blocking=True)
        seed_dev.fill_(int(sampler.seed) + int(step_index))
        first = sampler.sample_layers(graph, seeds_cur, seed_dev=seed_dev)
        for dst, src in zip(cur_tensors, _block_tensors(first)):
            dst.copy_(src)

    def step(seeds, step_index=0):
        seeds_buf.copy_(seeds, non_blocking=True)
        seed_dev.fill_(int(sampler.seed) + int(step_index))
        return graphed.replay()
    step.graphed = graphed
    step.prime = prime
    return step


def graphed_full_step(model, graph, features, labels, train_idx, optimizer, num_train=None, warmup=3):
    """``step() -> loss`` for full-graph training (one GPU, or a row shard with ``num_train`` = the
    global number of training rows) as one CUDA graph per epoch."""
    device = labels.device
    sharded = num_train is not None

    def body():
        _zero_grads(model, optimizer)
        logits = model(graph, features)
        if sharded:
            loss = F.cross_entropy(logits[train_idx].float(), labels[train_idx], reduction='sum') / num_train
        else:
            loss = F.cross_entropy(logits[train_idx].float(), labels[train_idx])
        loss.backward()
        _allreduce_grads(model, average=not sharded)
        torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
        optimizer.step()
        return loss.detach()

    model.train()
    graphed = GraphedStep(body, device, warmup)
    return graphed.replay


def _record_stream(obj, stream):
    """Tell the caching allocator that ``stream`` uses the tensors of ``obj`` (a tensor, a block or a
    list of them), which were allocated on another stream."""
    if torch.is_tensor(obj):
        if obj.is_cuda:
            obj.record_stream(stream)
    elif isinstance(obj, (list, tuple)):
        for o in obj:
            _record_stream(o, stream)
    elif hasattr(obj, '__dict__'):
        for v in vars(obj).values():
            if torch.is_tensor(v) or isinstance(v, (list, tuple)):
                _record_stream(v, stream)


def train_epoch_node_sampling(model, graph, features, labels, train_idx, optimizer, sampler,
                              batch_size: int = 1024, pipeline: bool = True, fetch_rows=None, max_batches=None):
    """One epoch of mini-batch training over ``train_idx`` (helper/engine.py:86-256).

    With ``pipeline`` a producer thread samples the blocks of batch i+1 and gathers its input rows
    on a side stream while the main thread trains on batch i (the reference's producer / consumer
    pair with a queue of one, helper/engine.py:118-153); the hand-over is a CUDA event, so neither
    thread synchronises the device.  Returns (mean loss tensor, number of seeds trained on)."""
    device = labels.device
    n = train_idx.numel()
    starts = list(range(0, n, batch_size))
    if max_batches is not None:
        starts = starts[:max_batches]
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        # the gradient all-reduce pairs the batches of all ranks up: unequal counts would leave the
        # ranks with more batches waiting in a collective for ever, so refuse before the first one
        cnt = torch.tensor([len(starts), -len(starts)], device=device)
        dist.all_reduce(cnt, op=dist.ReduceOp.MAX)
        if int(cnt[0]) != -int(cnt[1]):
            raise RuntimeError(f"ranks hold different numbers of batches ({len(starts)} here, "
                               f"{-int(cnt[1])}..{int(cnt[0])} overall): shard train_idx evenly")
    main_stream = torch.cuda.current_stream(device)
    total = torch.zeros((), device=device)
    model.train()

    def make_batch(step, lo):
        seeds = train_idx[lo:lo + batch_size].to(device=device, dtype=torch.int32, non_blocking=True)
        sampler.step = step
        blocks, x = layer0_inputs(sampler.sample_layers(graph, seeds), features, fetch_rows)
        return seeds, blocks, x

    def train_on(seeds, blocks, x):
        _zero_grads(model, optimizer)
        logits = model(blocks, x)[:seeds.numel()]
        loss = F.cross_entropy(logits.float(), labels[seeds.long()])
        loss.backward()
        _allreduce_grads(model)
        torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
        optimizer.step()
        return loss.detach()

    if not pipeline:
        for step, lo in enumerate(starts):
            total += train_on(*make_batch(step, lo))
        return total / max(len(starts), 1), min(n, len(starts) * batch_size)

    side = torch.cuda.Stream(device)
    side.wait_stream(main_stream)
    q = queue.Queue(maxsize=1)
    failure = []

    def producer():
        try:
            torch.cuda.set_device(device)
            with torch.cuda.stream(side):
                for step, lo in enumerate(starts):
                    item = make_batch(step, lo)
                    ev = torch.cuda.Event()
                    ev.record(side)
                    q.put((item, ev))
        except BaseException as exc:      # hand the failure to the consumer instead of dying silently
            failure.append(exc)
        finally:
            q.put(None)

    worker = threading.Thread(target=producer, daemon=True)
    worker.start()
    while True:
        got = q.get()
        if got is None:
            break
        (seeds, blocks, x), ev = got
        main_stream.wait_event(ev)
        _record_stream([seeds, blocks, x], main_stream)
        total += train_on(seeds, blocks, x)
    worker.join()
    if failure:
        raise failure[0]
    side.wait_stream(main_stream)
    return total / max(len(starts), 1), min(n, len(starts) * batch_size)
