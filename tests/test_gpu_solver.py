"""Parity of the CUDA placement solver and histogram kernels with the CPU oracle, and (when
oracle/_ref is present) with the reference's own solver kernel. Bit-exact: integer work."""

import numpy as np
import pytest
import torch

import cases as Cs
import gpu_util as G
from oracle import uep_oracle as O
from oracle import uep_ref

pytestmark = pytest.mark.gpu

SOLVE_CASES = Cs.solve_cases(True)


def _compare(cuda_out, plan, what):
    for f in G.PLAN_FIELDS:
        got = cuda_out[f].cpu().numpy()
        exp = getattr(plan, f)
        assert np.array_equal(got, exp), f"{what}: field {f} differs at {np.argwhere(got != exp)[:5].tolist()}"


@pytest.mark.parametrize("case", SOLVE_CASES, ids=lambda c: c.name)
def test_solver_matches_oracle(native_lib, cuda_device, case):
    lpr_dev = torch.from_numpy(case.loads_per_rank).to(cuda_device)
    for rank in case.ranks:
        out = G.cuda_solve(case, rank, lpr_dev)
        torch.cuda.synchronize()
        assert out["status"].tolist() == [0, 0]
        plan = O.solve_placement(case.loads_per_rank, case.M, case.R, case.nvl, rank, G.oracle_params(case))
        _compare(out, plan, f"{case.name} rank {rank}")
        assert np.array_equal(out["global_loads"].cpu().numpy(), case.loads_per_rank.sum(0).astype(np.int32))


def test_solver_random_sweep(native_lib, cuda_device):
    """Tiny exhaustive-style sweep: 400 random small domains, every field, one rank each."""
    for case in Cs.random_small_cases(400):
        rank = case.ranks[0]
        out = G.cuda_solve(case, rank)
        plan = O.solve_placement(case.loads_per_rank, case.M, case.R, case.nvl, rank, G.oracle_params(case))
        _compare(out, plan, case.name)
        assert out["status"].tolist() == [0, 0]


@pytest.mark.skipif(not uep_ref.available(), reason="oracle/_ref/libuep_ref.so not built")
@pytest.mark.parametrize("case", SOLVE_CASES, ids=lambda c: c.name)
def test_solver_matches_reference_kernel(native_lib, cuda_device, case):
    """The new kernel against the reference's quota_placement_solve_kernel on the same device."""
    lpr_dev = torch.from_numpy(case.loads_per_rank).to(cuda_device)
    for rank in case.ranks:
        out = G.cuda_solve(case, rank, lpr_dev)
        ref = uep_ref.solve_placement(lpr_dev, case.M, case.R, case.nvl, rank, case.balance_threshold,
                                      case.min_tokens, case.allow_zero, case.locality, case.eps)
        torch.cuda.synchronize()
        for f in G.PLAN_FIELDS:
            assert torch.equal(out[f], ref[f]), f"{case.name} rank {rank}: field {f} differs from the reference"


def test_solver_plan_properties_full_size(native_lib, cuda_device):
    """Size-independent properties at the largest benchmark shape (cfg5): legality of the plan,
    completeness of every rank's quota split, and that all ranks derive the same plan."""
    case = next(c for c in SOLVE_CASES if c.name == "cfg5_dsv3_stress")
    lpr_dev = torch.from_numpy(case.loads_per_rank).to(cuda_device)
    first = None
    for rank in range(case.N):
        out = G.cuda_solve(case, rank, lpr_dev)
        host = {f: out[f].cpu().numpy() for f in G.PLAN_FIELDS}
        plan = O.Plan(*[host[f] for f in G.PLAN_FIELDS])
        O.assert_plan_legal(plan, case.N, case.M, case.R, case.nvl)
        O.assert_rank_quota_complete(plan.rank_quota_prefix, plan.lcnts, case.loads_per_rank[rank])
        if first is None:
            first = host
        else:
            for f in G.PLAN_FIELDS[:-1]:
                assert np.array_equal(first[f], host[f])


def test_solver_rejects_bad_shapes(native_lib, cuda_device):
    from ultra_ep_b200 import capi
    import ctypes as C

    prm = capi.SolverParams.defaults()
    t = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    rc = native_lib.uep_solve_placement(t.data_ptr(), t.data_ptr(), *([t.data_ptr()] * 6), 8, 3, 2, 2, 8,
                                        C.byref(prm), 0, 0, 0)
    assert rc == -1 and b"group shape" in native_lib.uep_last_error()
    rc = native_lib.uep_solve_placement(t.data_ptr(), t.data_ptr(), *([t.data_ptr()] * 6), 8, 8, 100, 2, 8,
                                        C.byref(prm), 0, 0, 0)
    assert rc == -1 and b"static limits" in native_lib.uep_last_error()


@pytest.mark.parametrize("T,L,K", [(4096, 64, 8), (8192, 128, 8), (16384, 256, 8), (1000, 48, 4), (1, 64, 8), (0, 64, 8),
                                   (300, 64, 64)])
def test_histograms(native_lib, cuda_device, T, L, K):
    rng = np.random.default_rng(T + L)
    if T:
        keys = rng.random((T, L))
        ids = np.argpartition(keys, K - 1, axis=1)[:, :K].astype(np.int32) if K < L else np.tile(np.arange(L, dtype=np.int32), (T, 1))
    else:
        ids = np.empty((0, K), np.int32)
    ids_bad = ids.copy()
    if T:
        ids_bad[0, 0] = -1
        ids_bad[-1, -1] = L + 5
    rmap = np.zeros((T, L), np.bool_)
    if T:
        rmap[np.arange(T)[:, None], ids] = True
    exp_ids = O.histogram_ids(ids_bad, L)
    exp_map = O.histogram_map(rmap)
    got32 = G.cuda_histogram(torch.from_numpy(ids_bad).to(cuda_device), L, "ids32")
    got64 = G.cuda_histogram(torch.from_numpy(ids_bad.astype(np.int64)).to(cuda_device), L, "ids64")
    gotm = G.cuda_histogram(torch.from_numpy(rmap).to(cuda_device), L, "map")
    assert np.array_equal(got32.cpu().numpy(), exp_ids)
    assert np.array_equal(got64.cpu().numpy(), exp_ids)
    assert np.array_equal(gotm.cpu().numpy(), exp_map)
    if uep_ref.available() and T:
        refm = uep_ref.histogram_map(torch.from_numpy(rmap).to(cuda_device))
        assert torch.equal(refm, gotm)
        ref64 = uep_ref.histogram_ids64(torch.from_numpy(ids_bad.astype(np.int64)).to(cuda_device), L)
        assert torch.equal(ref64, got64)


def test_init_master_placement(native_lib, cuda_device):
    N, M, R = 8, 16, 4
    D, L, P = N, N * M, N * (M + R)
    bufs = [torch.full(s, 99, dtype=torch.int32, device=cuda_device) for s in [(P,), (L, D), (L,), (L, D), (L, D), (L, D)]]
    from ultra_ep_b200 import capi

    capi.check(native_lib.uep_init_master_placement(*[b.data_ptr() for b in bufs], N, M, R, D, G.stream_ptr()))
    exp = O.init_master_placement(N, M, R)
    for b, f in zip(bufs, G.PLAN_FIELDS):
        assert np.array_equal(b.cpu().numpy(), getattr(exp, f)), f


@pytest.mark.parametrize("case", Cs.legacy_cases(), ids=lambda c: c["name"])
def test_legacy_solver_matches_oracle(native_lib, cuda_device, case):
    """legacy_placement=True: the kernel against the restatement of the reference's host-side solver (which is
    itself pinned to that solver's recorded outputs) — p2l, l2p, lcnts bit for bit, quotas zero."""
    from ultra_ep_b200 import capi

    N, M, R, nvl = case["N"], case["M"], case["R"], case["nvl"]
    L, P, D = N * M, N * (M + R), N
    plan = O.legacy_solve_placement(case["loads"], N, M, R, nvl, case["balance_threshold"])
    loads = torch.from_numpy(case["loads"]).to(cuda_device)
    out = {k: torch.full(shape, 7777, dtype=torch.int32, device=cuda_device)
           for k, shape in [("p2l", (P,)), ("l2p", (L, D)), ("lcnts", (L,)), ("quota", (L, D)), ("quota_prefix", (L, D)),
                            ("rank_quota_prefix", (L, D))]}
    status = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    capi.check(capi.lib().uep_legacy_solve_placement(
        loads.data_ptr(), out["p2l"].data_ptr(), out["l2p"].data_ptr(), out["lcnts"].data_ptr(), out["quota"].data_ptr(),
        out["quota_prefix"].data_ptr(), out["rank_quota_prefix"].data_ptr(), N, nvl, M, R, D, case["balance_threshold"],
        status.data_ptr(), G.stream_ptr()), "uep_legacy_solve_placement")
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0]
    for f in ("p2l", "l2p", "lcnts"):
        assert np.array_equal(out[f].cpu().numpy(), getattr(plan, f)), (case["name"], f)
    for f in ("quota", "quota_prefix", "rank_quota_prefix"):
        assert not out[f].any()
