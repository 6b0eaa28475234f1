"""Planned tile ranges of the tcgen05 SpMM (grws_spmm_plan_build / grws_spmm_fwd_planned): the plan
against a host restatement of its rules, and the planned product against the CPU checker."""
import numpy as np
import pytest
import torch

from conftest import golden_cases, load_case
from gpu_util import DT, check_spmm_tolerance

pytestmark = pytest.mark.gpu

STAGE_TILES = 8
LONG_STAGES = 16
MAGIC = 0x504c4e31


def host_plan(wo, G):
    """Cuts and piece holders the plan kernel must produce for `G` CTAs."""
    W = len(wo) - 1
    T = int(wo[-1])
    stages = (np.diff(wo) + STAGE_TILES - 1) // STAGE_TILES
    sp = np.concatenate([[0], np.cumsum(stages)]).astype(np.int64)
    S = int(sp[-1])
    long_stages = LONG_STAGES if S >= 8 * G else np.iinfo(np.int64).max
    s = np.zeros(G + 1, np.int64)
    wf = np.zeros(G + 1, np.int64)
    for k in range(G + 1):
        if k == 0:
            s[k], wf[k] = 0, 0
        elif k == G or S == 0:
            s[k], wf[k] = T, W
        else:
            tgt = (k * S) // G
            w = int(np.searchsorted(sp[:W], tgt, side='right')) - 1
            a, b, before, after = int(wo[w]), int(wo[w + 1]), tgt - int(sp[w]), int(sp[w + 1]) - tgt
            if before == 0:
                s[k], wf[k] = a, w
            elif before + after <= long_stages:
                s[k], wf[k] = (b, w + 1) if after < before else (a, w)
            else:
                s[k], wf[k] = a + before * STAGE_TILES, w
    holders = np.zeros((G + 1, 3), np.int64)
    for k in range(G + 1):
        holders[k] = k
        if k == G:
            continue
        if s[k] < s[k + 1] and wf[k] < W and s[k] > wo[wf[k]]:
            a, b = wo[wf[k]], wo[wf[k] + 1]
            j = k
            while j > 0 and s[j] > a:
                j -= 1
            holders[k, 0] = j
            j = k
            while j + 1 < G and s[j + 1] < b:
                j += 1
            holders[k, 1] = j
        if s[k] < s[k + 1] and s[k + 1] < T:
            we = wf[k + 1]
            if we < W and s[k + 1] > wo[we] and wo[we] >= s[k]:
                b = wo[we + 1]
                j = k + 1
                while j + 1 < G and s[j + 1] < b:
                    j += 1
                holders[k, 2] = j
    return s, wf, holders, sp


def read_plan(plan, W):
    p = plan.cpu().numpy().view(np.int32)
    assert p[0] == MAGIC
    G = int(p[1])
    assert int(p[2]) | (int(p[3]) << 32) == W
    T = int(np.uint32(p[4])) | (int(p[5]) << 32)
    cuts = p[8:8 + 8 * (G + 1)].reshape(G + 1, 8)
    s = cuts[:, 0].astype(np.uint32).astype(np.int64) | (cuts[:, 1].astype(np.int64) << 32)
    wf = cuts[:, 2].astype(np.uint32).astype(np.int64) | (cuts[:, 3].astype(np.int64) << 32)
    holders = cuts[:, 4:7].astype(np.int64)
    sp = plan.cpu().numpy()[16 * (2 + 2 * (G + 1)):].view(np.int64)[:W + 1]
    return G, T, s, wf, holders, sp


def power_law(oracle, n, e, gamma, seed):
    from graph_rws_b200.data import synthetic
    g = synthetic.sym_normalized_csr(n, *synthetic.chung_lu_edges(n, e, gamma, seed))
    return g, oracle.csr_to_bcsr(g.num_nodes, g.row_ptr, g.col_idx, g.values)


def stage_counts(wo, s):
    """pipeline stages of every CTA for cuts `s`"""
    out = []
    for k in range(len(s) - 1):
        lo = np.maximum(wo[:-1], s[k])
        hi = np.minimum(wo[1:], s[k + 1])
        n = np.maximum(hi - lo, 0)
        out.append(int(((n + STAGE_TILES - 1) // STAGE_TILES).sum()))
    return np.array(out)


@pytest.mark.parametrize("shape", ["power_law", "hubs", "tiny", "dense_window"])
def test_plan_matches_host_restatement(oracle, shape):
    from graph_rws_b200 import core
    dev = torch.device("cuda")
    if shape == "power_law":
        g, (wo, cols, vals) = power_law(oracle, 60000, 900000, 2.5, 31)
    elif shape == "hubs":
        g, (wo, cols, vals) = power_law(oracle, 20000, 300000, 2.1, 23)
    elif shape == "tiny":
        g, (wo, cols, vals) = power_law(oracle, 500, 2000, 2.3, 3)
    else:
        c = load_case([p for p in golden_cases() if "dense_row" in p][0])     # one window of 250 tiles
        wo = c["window_offset"]
    W, T = len(wo) - 1, int(wo[-1])
    plan = core.spmm_plan(torch.from_numpy(wo).to(dev), T, 100000, 128)
    torch.cuda.synchronize()
    G, T_plan, s, wf, holders, sp = read_plan(plan, W)
    assert T_plan == T
    hs, hwf, hh, hsp = host_plan(wo, G)
    assert np.array_equal(sp, hsp)
    assert np.array_equal(s, hs) and np.array_equal(wf, hwf)
    assert np.array_equal(holders[:G], hh[:G])
    assert s[0] == 0 and s[G] == T and (np.diff(s) >= 0).all()
    if shape == "power_law":
        # the point of the plan: stage counts of the CTAs within a window's length of each other
        st = stage_counts(wo, s)
        assert st.max() - st.min() <= 2 * LONG_STAGES + 2, (st.min(), st.max())


@pytest.mark.parametrize("dt,N,out", [("f16", 128, "f16"), ("bf16", 256, "f32"), ("bf16", 128, "f32")])
def test_planned_product_matches_oracle_with_split_windows(oracle, dt, N, out):
    """Hub windows longer than a CTA's share: planned cuts inside windows, pieces summed by the
    holders the plan names."""
    from graph_rws_b200 import core
    dev = torch.device("cuda")
    g, (wo, cols, vals) = power_law(oracle, 20000, 300000, 2.1, 23)
    dtype = DT[dt]
    W, T = len(wo) - 1, int(wo[-1])
    B = torch.randn(g.num_nodes, N, generator=torch.Generator().manual_seed(5)).to(dtype)
    vals_t = torch.from_numpy(vals).to(dtype)
    wo_d, cols_d, vals_d, B_d = torch.from_numpy(wo).to(dev), torch.from_numpy(cols).to(dev), vals_t.to(dev), B.to(dev)
    plan = core.spmm_plan(wo_d, T, g.num_nodes, N)
    G, _, s, wf, holders, _ = read_plan(plan, W)
    inside = [k for k in range(1, G) if wf[k] < W and s[k] > wo[wf[k]]]
    assert inside, "the case must split a window"
    C_ref = oracle.spmm_fwd(wo, cols, vals_t.float().numpy(), B.float().numpy())
    for _ in range(2):          # the second launch finds the split counters used by the first
        C = core.spmm_raw(wo_d, cols_d, vals_d, B_d, out_dtype=DT[out], algo=core.ALGO_TCGEN05, check=True, plan=plan)
        check_spmm_tolerance(C.float().cpu().numpy(), C_ref, None, f"planned N={N} {dt}")
    C0 = core.spmm_raw(wo_d, cols_d, vals_d, B_d, out_dtype=DT[out], algo=core.ALGO_TCGEN05, check=True)
    assert torch.allclose(C.float(), C0.float(), rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("N", [128, 256, 48])      # one slab; two slabs in one pass (one CTA per SM); the narrow variant
@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: p.split("bcsr_")[-1][:-4])
def test_planned_product_on_golden_graphs(oracle, path, N):
    from graph_rws_b200 import core
    dev = torch.device("cuda")
    c = load_case(path)
    wo, cols, vals = c["window_offset"], c["cols"], c["vals"]
    W, T = len(wo) - 1, int(wo[-1])
    K = int(max(int(cols.max()) + 1 if cols.size else 1, 16))
    B = torch.randn(K, N, generator=torch.Generator().manual_seed(9)).half()
    vals_t = torch.from_numpy(vals).half()
    wo_d = torch.from_numpy(wo).to(dev)
    plan = core.spmm_plan(wo_d, T, K, N)
    C = core.spmm_raw(wo_d, torch.from_numpy(cols).to(dev), vals_t.to(dev), B.to(dev), algo=core.ALGO_TCGEN05, check=True, plan=plan)
    C_ref = oracle.spmm_fwd(wo, cols, vals_t.float().numpy(), B.float().numpy())
    check_spmm_tolerance(C.float().cpu().numpy(), C_ref, None, "planned golden")


def test_plan_of_another_shape_is_ignored(oracle):
    """A plan built for a different number of windows must not be used: the launch searches its
    ranges and the product is right."""
    from graph_rws_b200 import core
    dev = torch.device("cuda")
    g1, (wo1, cols1, vals1) = power_law(oracle, 20000, 300000, 2.1, 23)
    g2, (wo2, cols2, vals2) = power_law(oracle, 24000, 300000, 2.3, 29)
    plan2 = core.spmm_plan(torch.from_numpy(wo2).to(dev), int(wo2[-1]), g2.num_nodes, 128)
    B = torch.randn(g1.num_nodes, 128, generator=torch.Generator().manual_seed(6)).half()
    vals_t = torch.from_numpy(vals1).half()
    C = core.spmm_raw(torch.from_numpy(wo1).to(dev), torch.from_numpy(cols1).to(dev), vals_t.to(dev), B.to(dev),
                      algo=core.ALGO_TCGEN05, check=True, plan=plan2)
    C_ref = oracle.spmm_fwd(wo1, cols1, vals_t.float().numpy(), B.float().numpy())
    check_spmm_tolerance(C.float().cpu().numpy(), C_ref, None, "foreign plan")


def test_graph_builds_its_plan_at_the_second_product():
    from graph_rws_b200 import BCSRGraph
    from graph_rws_b200.data import synthetic
    dev = torch.device("cuda")
    g = synthetic.sym_normalized_csr(5000, *synthetic.chung_lu_edges(5000, 60000, 2.3, 17))
    graph = BCSRGraph.from_csr(g.num_nodes, g.row_ptr, g.col_idx, g.values, device=dev, values_dtype=torch.float16)
    assert graph.spmm_plan(5000, 128) is None
    p = graph.spmm_plan(5000, 128)
    assert p is not None and graph.spmm_plan(5000, 128) is p
    assert graph.spmm_plan(5000, 256) is None            # another width: its own plan
    graph.transient = True
    assert graph.spmm_plan(5000, 128) is None
