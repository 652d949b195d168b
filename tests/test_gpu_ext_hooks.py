"""The PyTorch extension's single-GPU test hooks, called the way the reference's own solving test
calls them (tests/test_solving.py:30-53, 115-131, 297-334 of the reference): one solve per source
rank to simulate a whole EP group on one device, then the legality / completeness invariants and
parity with the oracle."""

import numpy as np
import pytest
import torch

import cases as Cs
import gpu_util as G
from oracle import uep_oracle as O
from ultra_ep_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C_ext(native_lib):
    from ultra_ep_b200 import build
    from ultra_ep_b200.native import load

    build.build_ext()
    return load()


@pytest.mark.parametrize("name", ["cfg1_plan_reroute", "cfg3_qwen3_235b_fp8", "ep64", "many_small_R1", "precheck_seed4"])
def test_solve_placement_for_test_hook(C_ext, cuda_device, name):
    case = next(c for c in Cs.solve_cases(True) if c.name == name)
    lpr = torch.from_numpy(case.loads_per_rank).to(cuda_device)
    loads = lpr.sum(0, dtype=torch.int32)
    prefixes = []
    for src in range(case.N):
        out = C_ext.solve_placement_for_test(loads, lpr, case.N, case.M, case.R, case.nvl, False, case.balance_threshold,
                                             case.min_tokens, case.allow_zero, case.locality, case.eps, 1, src)
        p2l, l2p, lcnts, quota, qp, rqp = (t.cpu().numpy() for t in out)
        plan = O.solve_placement(case.loads_per_rank, case.M, case.R, case.nvl, src, G.oracle_params(case))
        for got, f in zip((p2l, l2p, lcnts, quota, qp, rqp), G.PLAN_FIELDS):
            assert np.array_equal(got, getattr(plan, f)), (name, src, f)
        if src == 0:
            O.assert_plan_legal(plan, case.N, case.M, case.R, case.nvl)
        prefixes.append(rqp)
    # the last prefix of every rank equals that rank's load of the expert
    for src in range(case.N):
        O.assert_rank_quota_complete(prefixes[src], lcnts, case.loads_per_rank[src])


def test_dense_reroute_for_test_hook(C_ext, cuda_device):
    cfg = W.CONFIGS["cfg1_plan_reroute"]
    lpr_np = W.loads_per_rank(cfg)
    lpr = torch.from_numpy(lpr_np).to(cuda_device)
    P = cfg.ep * (cfg.masters + cfg.redundant)
    for src in (0, 5):
        _, l2p, lcnts, _, _, rqp = C_ext.solve_placement_for_test(lpr.sum(0, dtype=torch.int32), lpr, cfg.ep, cfg.masters,
                                                                 cfg.redundant, cfg.ep, False, 1.0, 1024, False, True,
                                                                 0.01, 1, src)
        ids = W.routing_ids(cfg, src)
        rmap = W.ids_to_map(ids, cfg.num_experts)
        probs = rmap.astype(np.float32)
        for quota, interleave in ((True, True), (True, False), (False, True)):
            ep, em = C_ext.dense_reroute_for_test(torch.from_numpy(rmap).to(cuda_device),
                                                  torch.from_numpy(probs).to(cuda_device), l2p, lcnts, rqp, P, quota,
                                                  interleave)
            assert bool((em.sum(1) == cfg.topk).all())
            plan = O.solve_placement(lpr_np, cfg.masters, cfg.redundant, cfg.ep, src)
            o_probs, o_map = O.dense_reroute_forward(rmap, probs, plan, P, interleave, quota)
            assert np.array_equal(em.cpu().numpy(), o_map) and np.array_equal(ep.cpu().numpy(), o_probs)


def test_hook_argument_errors(C_ext, cuda_device):
    loads = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    lpr = torch.zeros(4, 16, dtype=torch.int32, device=cuda_device)
    with pytest.raises(RuntimeError):
        C_ext.solve_placement_for_test(loads, lpr, 4, 4, 1, 3)        # 4 % 3 != 0
    with pytest.raises(RuntimeError):
        C_ext.solve_placement_for_test(loads.cpu(), lpr, 4, 4, 1, 4)  # host tensor
    with pytest.raises(RuntimeError):
        C_ext.Manager(1, 2, 1, 16, 16, 2, 1, 0, 0, 4, True, True)     # runtime not initialised


def test_solve_placement_for_test_hook_legacy(C_ext, cuda_device):
    """legacy_placement=True through the hook: the counts-only greedy plan, quotas zero."""
    for case in Cs.legacy_cases()[:9]:
        if case["nvl"] != case["N"]:
            continue
        N, M, R = case["N"], case["M"], case["R"]
        loads = torch.from_numpy(case["loads"]).to(cuda_device)
        lpr = torch.zeros(N, N * M, dtype=torch.int32, device=cuda_device)
        lpr[0] = loads
        p2l, l2p, lcnts, quota, qp, rqp = C_ext.solve_placement_for_test(loads, lpr, N, M, R, N, True,
                                                                         case["balance_threshold"])
        plan = O.legacy_solve_placement(case["loads"], N, M, R, N, case["balance_threshold"])
        assert np.array_equal(p2l.cpu().numpy(), plan.p2l) and np.array_equal(l2p.cpu().numpy(), plan.l2p)
        assert np.array_equal(lcnts.cpu().numpy(), plan.lcnts)
        assert not quota.any() and not qp.any() and not rqp.any()
