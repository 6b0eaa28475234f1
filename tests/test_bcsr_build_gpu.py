"""Device CSR->BCSR builder and transposed-BCSR builder: bit-exact against the reference's own
csr_to_bcsr_cpu outputs (tests/golden/) and against the CPU checker."""
import os

import numpy as np
import pytest
import torch

from conftest import golden_cases, load_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: os.path.basename(p)[5:-4])
def test_device_builder_is_bit_exact_on_golden(path):
    from graph_rws_b200 import core
    c = load_case(path)
    dev = torch.device("cuda")
    wo, cols, vals = core.csr_to_bcsr(int(c["num_rows"]), torch.from_numpy(c["row_ptr"]).to(dev),
                                      torch.from_numpy(c["col_idx"]).to(dev), torch.from_numpy(c["values"]).to(dev))
    assert np.array_equal(wo.cpu().numpy(), c["window_offset"])
    assert np.array_equal(cols.cpu().numpy(), c["cols"])
    assert np.array_equal(vals.cpu().numpy().view(np.uint32), c["vals"].view(np.uint32))


def test_csr_to_bcsr_cpu_keeps_the_reference_contract():
    from graph_rws_b200 import core
    c = load_case(golden_cases()[0])
    wo, cols, vals = core.csr_to_bcsr_cpu(int(c["num_rows"]), torch.from_numpy(c["row_ptr"]),
                                          torch.from_numpy(c["col_idx"]), torch.from_numpy(c["values"]), 16, 8)
    assert wo.device.type == "cpu" and wo.dtype == torch.int64 and cols.dtype == torch.int32
    assert np.array_equal(vals.numpy(), c["vals"])
    with pytest.raises(RuntimeError):
        core.csr_to_bcsr_cpu(3, torch.zeros(4, dtype=torch.int64, device="cuda"), torch.zeros(0, dtype=torch.int32),
                             torch.zeros(0), 16, 8)


def test_device_builder_on_power_law_graph(oracle):
    from graph_rws_b200 import core
    from graph_rws_b200.data import synthetic
    g = synthetic.graph_for_config("spmm_mid", scale=0.1)
    dev = torch.device("cuda")
    wo, cols, vals = core.csr_to_bcsr(g.num_nodes, torch.from_numpy(g.row_ptr).to(dev),
                                      torch.from_numpy(g.col_idx).to(dev), torch.from_numpy(g.values).to(dev))
    wo_r, cols_r, vals_r = oracle.csr_to_bcsr(g.num_nodes, g.row_ptr, g.col_idx, g.values)
    assert np.array_equal(wo.cpu().numpy(), wo_r)
    assert np.array_equal(cols.cpu().numpy(), cols_r)
    assert np.array_equal(vals.cpu().numpy(), vals_r)


def test_transposed_bcsr_equals_bcsr_of_transposed_csr(oracle):
    import scipy.sparse as sps
    from graph_rws_b200 import core
    from graph_rws_b200.data import synthetic
    rng = np.random.default_rng(9)
    n_rows, n_cols = 300, 190
    A = sps.random(n_rows, n_cols, density=0.03, random_state=rng, dtype=np.float32, format="csr")
    A.sort_indices()
    dev = torch.device("cuda")
    wo, cols, vals = core.csr_to_bcsr(n_rows, torch.from_numpy(A.indptr.astype(np.int64)).to(dev),
                                      torch.from_numpy(A.indices.astype(np.int32)).to(dev),
                                      torch.from_numpy(A.data).to(dev))
    wo_t, cols_t, vals_t = core.bcsr_transpose(wo, cols, vals, n_cols)
    At = A.T.tocsr()
    At.sort_indices()
    wo_r, cols_r, vals_r = oracle.csr_to_bcsr(n_cols, At.indptr.astype(np.int64), At.indices.astype(np.int32), At.data)
    assert np.array_equal(wo_t.cpu().numpy(), wo_r)
    assert np.array_equal(cols_t.cpu().numpy(), cols_r)
    assert np.array_equal(vals_t.cpu().numpy(), vals_r)
