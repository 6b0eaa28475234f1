"""All-gather of row shards with the library's own NVLink kernels (``grws_peer_all_gather``).

Every rank keeps a staging block and a small control block in memory all ranks of the node can
address (torch's symmetric-memory allocator: one CUDA allocation per rank, mapped into every rank).
An exchange is two kernels per rank and no collective call: publish the local rows, pull everybody's
rows with plain loads.  Ordering between ranks is kept by flags in the control blocks that hold
exchange numbers; all state is on the device, so exchanges can be captured in a CUDA graph.  Waits
are bounded: ``check()`` raises if one ran out.
"""
import torch
import torch.distributed as dist

from ..core import _native


class PeerAllGather:
    """``gather(local) -> [world * pad_rows, width]`` with rank r's rows at ``r * pad_rows``
    (the layout of ``all_gather_into_tensor`` on zero-padded shards)."""

    WAIT_LIMIT = 2_000_000_000        # SM clocks, about a second

    def __init__(self, pad_rows: int, max_row_bytes: int, device, group=None, push: bool = True):
        """``push``: every rank stores its rows into an inbox on each rank and ``gather`` returns
        (a view of) this rank's inbox -- valid until the next ``gather``; otherwise every rank
        publishes its rows in a staging block and pulls everybody's into a fresh tensor."""
        import torch.distributed._symmetric_memory as symm_mem
        lib = _native.lib()
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.pad_rows, self.max_row_bytes, self.device = int(pad_rows), int(max_row_bytes), torch.device(device)
        if self.max_row_bytes % 16:
            raise ValueError("rows must be a multiple of 16 bytes")
        self.push = bool(push)
        slots = self.world if self.push else 1
        self.stage = symm_mem.empty((slots * self.pad_rows * self.max_row_bytes,), dtype=torch.uint8, device=self.device)
        self.ctrl = symm_mem.empty((int(lib.grws_peer_ctrl_bytes()) // 4,), dtype=torch.int32, device=self.device)
        self.ctrl.zero_()
        torch.cuda.synchronize(self.device)
        self._stage_handle = symm_mem.rendezvous(self.stage, self.group.group_name)
        self._ctrl_handle = symm_mem.rendezvous(self.ctrl, self.group.group_name)
        self.stages = torch.tensor([int(p) for p in self._stage_handle.buffer_ptrs], dtype=torch.int64, device=self.device)
        self.ctrls = torch.tensor([int(p) for p in self._ctrl_handle.buffer_ptrs], dtype=torch.int64, device=self.device)
        self.state = torch.zeros(int(lib.grws_peer_state_bytes()) // 4, dtype=torch.int32, device=self.device)
        dist.barrier(self.group)          # every rank's control block is zeroed before anybody signals

    def gather(self, local: torch.Tensor) -> torch.Tensor:
        rows, width = local.shape
        row_bytes = width * local.element_size()
        if rows > self.pad_rows or row_bytes > self.max_row_bytes or row_bytes % 16:
            raise ValueError("shard does not fit the staging block")
        local = local.contiguous()
        if self.push:
            _native.check(_native.lib().grws_peer_all_gather_push(
                local.data_ptr(), rows * row_bytes, self.pad_rows * row_bytes, self.stages.data_ptr(), self.ctrls.data_ptr(),
                self.world, self.rank, self.state.data_ptr(), self.WAIT_LIMIT,
                torch.cuda.current_stream(self.device).cuda_stream))
            return self.stage[:self.world * self.pad_rows * row_bytes].view(local.dtype).view(self.world * self.pad_rows, width)
        out = torch.empty((self.world * self.pad_rows, width), dtype=local.dtype, device=self.device)
        _native.check(_native.lib().grws_peer_all_gather(
            local.data_ptr(), rows * row_bytes, self.stage.data_ptr(), self.pad_rows * row_bytes,
            self.stages.data_ptr(), self.ctrls.data_ptr(), self.world, self.rank, self.state.data_ptr(),
            out.data_ptr(), self.WAIT_LIMIT, torch.cuda.current_stream(self.device).cuda_stream))
        return out

    __call__ = gather

    def check(self):
        """Synchronises and raises if a wait of an exchange ran out since the start."""
        status = int(self.state[3].item())
        if status:
            what = {1: "peers were still reading the previous exchange", 2: "peers never published their rows"}
            raise RuntimeError(f"peer all-gather gave up waiting: {what.get(status, status)}; its output is undefined")


def make_peer_all_gather(pad_rows, max_row_bytes, device, group=None, probe_dtype=torch.bfloat16, push=True,
                         keep_if_slower=False):
    """A ``PeerAllGather`` that has reproduced ``all_gather_into_tensor`` on two probe exchanges and
    is not slower than it on the widest operand (unless ``keep_if_slower``), or None (on every rank
    alike) when the node's GPUs cannot address each other's memory, a probe disagreed or the
    collective was faster -- the caller then keeps the NCCL collective."""
    group = group if group is not None else dist.group.WORLD
    ok = 1
    pg = None
    try:
        pg = PeerAllGather(pad_rows, max_row_bytes, device, group, push=push)
    except Exception:                      # noqa: BLE001  (no symmetric memory on this box)
        ok = 0
    flag = torch.tensor([ok], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if int(flag) == 0:
        return None
    width = max_row_bytes // torch.empty((), dtype=probe_dtype).element_size()
    gen = torch.Generator(device=device).manual_seed(1234 + pg.rank)
    for w in (width, max(8, width // 4 // 8 * 8)):
        rows = pad_rows - (pg.rank % 2)                        # uneven shards as well
        local = torch.randn((max(rows, 0), w), generator=gen, device=device).to(probe_dtype)
        got = pg.gather(local)
        send = torch.zeros((pad_rows, w), dtype=probe_dtype, device=device)
        send[:local.shape[0]] = local
        want = torch.empty_like(got)
        dist.all_gather_into_tensor(want, send, group=group)
        same = torch.equal(got, want) and int(pg.state[3].item()) == 0
        flag = torch.tensor([1 if same else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag) == 0:
            return None
    if not keep_if_slower:
        # which of the two is faster depends on the number of ranks and the links: time both on
        # the widest operand (slowest rank counts) and keep the collective if it wins
        local = torch.randn((pad_rows, width), generator=gen, device=device).to(probe_dtype)
        want = torch.empty((pg.world * pad_rows, width), dtype=probe_dtype, device=device)
        times = []
        for fn in (lambda: pg.gather(local), lambda: dist.all_gather_into_tensor(want, local, group=group)):
            for _ in range(2):
                fn()
            dist.barrier(group)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(5):
                fn()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
        t = torch.tensor(times, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        pg.probe_ms = (float(t[0]) / 5, float(t[1]) / 5)          # (peer kernels, collective) per exchange
        if float(t[0]) > float(t[1]):
            return None
    return pg
