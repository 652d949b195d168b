"""Pins the CPU oracle against outputs recorded from the reference's own kernels
(tests/golden/ref_golden.npz, written by tests/golden/make_golden.py on a B200).
No GPU needed: this is what makes the oracle trustworthy as the parity checker."""

import hashlib
import os

import numpy as np
import pytest

import cases as Cs
from oracle import uep_oracle as O
from ultra_ep_b200 import workloads as W

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_golden.npz")
FIELDS = ("p2l", "l2p", "lcnts", "quota", "quota_prefix", "rank_quota_prefix")


@pytest.fixture(scope="module")
def golden():
    assert os.path.exists(GOLDEN), "tests/golden/ref_golden.npz is missing (see tests/golden/make_golden.py)"
    return np.load(GOLDEN)


def _sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


def test_solver_against_recorded_reference(golden):
    names = [str(n) for n in golden["solve_names"]]
    assert len(names) >= 100
    branches = set()
    for name in names:
        key = f"solve/{name}"
        lpr = golden[f"{key}/loads_per_rank"]
        M, R, nvl, min_tokens, allow_zero, locality = (int(x) for x in golden[f"{key}/params"])
        bt, eps = (float(x) for x in golden[f"{key}/fparams"])
        ranks = [int(r) for r in golden[f"{key}/ranks"]]
        params = O.SolverParams(bt, min_tokens, bool(allow_zero), bool(locality), eps)
        for rank in ranks:
            plan = O.solve_placement(lpr, M, R, nvl, rank, params)
            branches.update(int(p) & 15 for p in plan.path)
            for f in FIELDS:
                k = f"{key}/r{rank}/{f}" if (f == "rank_quota_prefix" or rank == ranks[0]) else f"{key}/r{ranks[0]}/{f}"
                assert np.array_equal(getattr(plan, f), golden[k]), f"{name} rank {rank}: {f} differs from the reference"
    assert branches == {0, 1, 2, 3}, "golden cases must cover every branch of the threshold search"


def test_golden_inputs_match_case_generators(golden):
    """The recorded inputs are what tests/cases.py generates today (guards against silent drift)."""
    by_name = {c.name: c for c in Cs.solve_cases(True) + Cs.random_small_cases(60)}
    for name in (str(n) for n in golden["solve_names"]):
        assert name in by_name, name
        assert np.array_equal(by_name[name].loads_per_rank, golden[f"solve/{name}/loads_per_rank"]), name


def test_reroute_against_recorded_reference(golden):
    solve_by_name = {c.name: c for c in Cs.solve_cases(True)}
    names = [str(n) for n in golden["reroute_names"]]
    assert len(names) >= 8
    for name in names:
        key = f"reroute/{name}"
        rank, T, K, seed, interleave, L, P = (int(x) for x in golden[f"{key}/meta"])
        sc = solve_by_name[str(golden[f"{key}/solve"])]
        plan = O.solve_placement(sc.loads_per_rank, sc.M, sc.R, sc.nvl, rank,
                                 O.SolverParams(sc.balance_threshold, sc.min_tokens, sc.allow_zero, sc.locality, sc.eps))
        ids = golden[f"{key}/ids"]
        rmap = W.ids_to_map(ids, L)
        probs = W.probs_for_map(rmap, seed)
        out_probs, out_map = O.dense_reroute_forward(rmap, probs, plan, P, bool(interleave))
        assert np.array_equal(np.packbits(out_map), golden[f"{key}/expanded_map_bits"]), name
        assert np.array_equal(_sha(out_probs), golden[f"{key}/expanded_probs_sha256"]), name
        grad = np.random.default_rng(seed + 1).normal(size=(T, P)).astype(np.float32)
        back = O.dense_reroute_backward(grad, rmap, out_map, plan)
        assert np.array_equal(_sha(back), golden[f"{key}/grad_probs_sha256"]), name
        # the sparse form is the dense rule applied per (token, k)
        sparse = O.sparse_reroute(ids.astype(np.int32), plan, bool(interleave))
        dense_from_sparse = np.zeros((T, P), np.bool_)
        dense_from_sparse[np.arange(T)[:, None], sparse] = True
        assert np.array_equal(dense_from_sparse, out_map), name


def test_oracle_legacy_solver_matches_reference_golden():
    """The restatement of the reference's legacy host-side solver against what that solver itself produced
    (tests/golden/ref_legacy_golden.npz, written by tests/golden/make_legacy_golden.py), and live when the
    in-place build of it is present."""
    import cases as Cs
    from oracle import uep_ref

    golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_legacy_golden.npz"))
    cases = Cs.legacy_cases()
    assert sorted(golden["names"].tolist()) == sorted(c["name"] for c in cases)
    replicated = 0
    for c in cases:
        plan = O.legacy_solve_placement(c["loads"], c["N"], c["M"], c["R"], c["nvl"], c["balance_threshold"])
        for f in ("p2l", "l2p", "lcnts"):
            assert np.array_equal(getattr(plan, f), golden[f"{c['name']}/{f}"]), (c["name"], f)
        assert not plan.quota.any() and not plan.rank_quota_prefix.any()
        replicated += int((plan.lcnts > 1).sum())
        if uep_ref.legacy_available():
            p2l, l2p, lcnts = uep_ref.legacy_solve_host(c["loads"], c["N"], c["M"], c["R"], c["nvl"], c["balance_threshold"])
            assert np.array_equal(p2l, plan.p2l) and np.array_equal(l2p, plan.l2p) and np.array_equal(lcnts, plan.lcnts)
    assert replicated > 50
