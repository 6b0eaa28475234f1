"""The bounded waits of the tcgen05 SpMM kernel: a pipeline that stops making progress ends with a
status, not with a hung GPU.

The self-test build of the library (csrc/build.py: build_selftest, -DGRWS_TC5_PROFILING) can withhold
one barrier arrive in one CTA -- the batch of stage descriptors is written but never published, and
nothing was copied for it, so no copy is in flight.  Every role of that CTA then runs into its wait
limit (set to a few milliseconds here), the kernel drains and returns, the launch's status word and
the per-device word name the wait, and the context stays usable: the next launch is correct.
Nothing here faults, traps or spins without a bound.  Runs in a process of its own because the
library variant is chosen when the binding is first loaded.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import os, sys, time
sys.path.insert(0, %(root)r)
import numpy as np, torch
import oracle
from graph_rws_b200 import BCSRGraph, core
from graph_rws_b200.core import _native
from graph_rws_b200.data import synthetic
lib = _native.lib()
dev = torch.device("cuda")
g = synthetic.sym_normalized_csr(40000, *synthetic.chung_lu_edges(40000, 500000, 2.3, 5))
graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev, values_dtype=torch.float16)
H = torch.randn(g.num_nodes, 128, generator=torch.Generator().manual_seed(1)).half().to(dev)
args = (graph.window_offset, graph.original_col_indices, graph.values_condensed, H)
good = core.spmm_raw(*args, algo=core.ALGO_TCGEN05, check=True)
assert lib.grws_spmm_set_wait_limit(8000000) == 0                  # about 4 ms of SM clocks per wait
os.environ["GRWS_TC5_PROFILE"] = "1"
os.environ["GRWS_TC5_SKIP"] = "16"                                 # CTA 0 never publishes its second descriptor batch
t0 = time.perf_counter()
bad = core.spmm_raw(*args, algo=core.ALGO_TCGEN05)
torch.cuda.synchronize()                                           # the launch returns: no role waits for ever
elapsed = time.perf_counter() - t0
assert elapsed < 5.0, elapsed
st = lib.grws_spmm_check(torch.cuda.current_stream().cuda_stream)
assert st == -5, st                                                # GRWS_ERR_DEVICE
msg = lib.grws_last_error().decode()
assert "gave up waiting" in msg, msg
assert lib.grws_spmm_check(torch.cuda.current_stream().cuda_stream) == 0     # reading the word cleared it
os.environ["GRWS_TC5_SKIP"] = "0"
assert lib.grws_spmm_set_wait_limit(0) == 0
again = core.spmm_raw(*args, algo=core.ALGO_TCGEN05, check=True)   # the context is intact
assert torch.equal(again, good)
wo, cols, vals = oracle.csr_to_bcsr(g.num_nodes, g.row_ptr, g.col_idx, g.values)
ref = oracle.spmm_fwd(wo, cols, torch.from_numpy(vals).half().float().numpy(), H.float().cpu().numpy())
err = np.linalg.norm(again.float().cpu().numpy() - ref) / np.linalg.norm(ref)
assert err < 1e-3, err
print("TIMEOUT-SELFTEST-OK", round(elapsed * 1e3, 1), "ms;", msg)
"""


def test_a_withheld_arrive_ends_with_a_status_not_a_hang():
    from graph_rws_b200.core import _native
    selftest = os.path.join(os.path.dirname(_native.LIB_PATH), "libgrws_b200_selftest.so")
    if not os.path.exists(selftest):
        pytest.skip("self-test build of the library is missing (graph_rws_b200/csrc/build.py --selftest)")
    env = dict(os.environ, GRWS_LIB_PATH=selftest)
    env.pop("GRWS_TC5_SKIP", None)
    out = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "TIMEOUT-SELFTEST-OK" in out.stdout
