"""Parity of the CUDA reroute kernels with the CPU oracle and with the reference's own dense
reroute kernels (when oracle/_ref is present). Bit-exact: routing is integer work and the
probabilities are copied, never recomputed."""

import numpy as np
import pytest
import torch

import cases as Cs
import gpu_util as G
from oracle import uep_oracle as O
from oracle import uep_ref
from ultra_ep_b200 import workloads as W

pytestmark = pytest.mark.gpu

REROUTE_CASES = Cs.reroute_cases(True)


def _setup(rc, dev):
    sc = rc.solve
    plan = O.solve_placement(sc.loads_per_rank, sc.M, sc.R, sc.nvl, rc.rank, G.oracle_params(sc))
    ids = Cs.reroute_inputs(rc)
    L, P = sc.L, sc.N * (sc.M + sc.R)
    rmap = W.ids_to_map(ids, L)
    probs = W.probs_for_map(rmap, rc.seed)
    return plan, ids, rmap, probs, L, P, G.plan_to_device(plan, dev)


@pytest.mark.parametrize("rc", REROUTE_CASES, ids=lambda c: c.name)
def test_dense_forward_backward(native_lib, cuda_device, rc):
    plan, ids, rmap, probs, L, P, pd = _setup(rc, cuda_device)
    exp_probs, exp_map = O.dense_reroute_forward(rmap, probs, plan, P, rc.interleave)
    d_map = torch.from_numpy(rmap).to(cuda_device)
    d_probs = torch.from_numpy(probs).to(cuda_device)
    got_probs, got_map = G.cuda_dense_reroute(d_map, d_probs, pd["l2p"], pd["lcnts"], pd["rank_quota_prefix"], P,
                                              rc.interleave)
    torch.cuda.synchronize()
    assert np.array_equal(got_map.cpu().numpy(), exp_map)
    assert np.array_equal(got_probs.cpu().numpy().view(np.uint32), exp_probs.view(np.uint32))
    if rc.T:
        assert bool((got_map.sum(1) == rc.K).all()), "every token must keep top-k physical experts"
    # backward: gather a random upstream gradient back to logical experts
    grad = torch.from_numpy(np.random.default_rng(rc.seed + 1).normal(size=(rc.T, P)).astype(np.float32)).to(cuda_device)
    exp_back = O.dense_reroute_backward(grad.cpu().numpy(), rmap, exp_map, plan)
    got_back = G.cuda_dense_reroute_backward(grad, d_map, got_map, pd["l2p"], pd["lcnts"])
    assert np.array_equal(got_back.cpu().numpy().view(np.uint32), exp_back.view(np.uint32))
    if uep_ref.available() and rc.T:
        ref_probs, ref_map = uep_ref.dense_reroute_forward(d_map, d_probs, pd["l2p"], pd["lcnts"],
                                                           pd["rank_quota_prefix"], P, rc.interleave)
        assert torch.equal(ref_map, got_map) and torch.equal(ref_probs, got_probs)
        ref_back = uep_ref.dense_reroute_backward(grad, d_map, ref_map, pd["l2p"], pd["lcnts"])
        assert torch.equal(ref_back, got_back)


@pytest.mark.parametrize("rc", REROUTE_CASES, ids=lambda c: c.name)
def test_round_robin_mode(native_lib, cuda_device, rc):
    plan, ids, rmap, probs, L, P, pd = _setup(rc, cuda_device)
    exp_probs, exp_map = O.dense_reroute_forward(rmap, probs, plan, P, quota=False)
    got_probs, got_map = G.cuda_dense_reroute(torch.from_numpy(rmap).to(cuda_device),
                                              torch.from_numpy(probs).to(cuda_device), pd["l2p"], pd["lcnts"],
                                              pd["rank_quota_prefix"], P, quota_mode=False)
    assert np.array_equal(got_map.cpu().numpy(), exp_map)
    assert np.array_equal(got_probs.cpu().numpy().view(np.uint32), exp_probs.view(np.uint32))


@pytest.mark.parametrize("rc", REROUTE_CASES, ids=lambda c: c.name)
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_sparse_reroute(native_lib, cuda_device, rc, dtype):
    plan, ids, rmap, probs, L, P, pd = _setup(rc, cuda_device)
    np_ids = ids.astype(np.int64 if dtype == torch.int64 else np.int32)
    exp = O.sparse_reroute(np_ids, plan, rc.interleave)
    d_ids = torch.from_numpy(np_ids).to(cuda_device)
    got = G.cuda_sparse_reroute(d_ids, pd["l2p"], pd["lcnts"], pd["rank_quota_prefix"], rc.interleave)
    assert np.array_equal(got.cpu().numpy(), exp)
    # in place gives the same answer
    inplace = G.cuda_sparse_reroute(d_ids.clone(), pd["l2p"], pd["lcnts"], pd["rank_quota_prefix"], rc.interleave,
                                    inplace=True)
    assert torch.equal(inplace, got)
    if rc.T:
        # the sparse result scattered to dense equals the dense rule (ids are distinct per token)
        _, exp_map = O.dense_reroute_forward(rmap, probs, plan, P, rc.interleave)
        dense_from_sparse = np.zeros((rc.T, P), np.bool_)
        dense_from_sparse[np.arange(rc.T)[:, None], got.cpu().numpy()] = True
        assert np.array_equal(dense_from_sparse, exp_map)
    if uep_ref.available() and rc.T and dtype == torch.int64 and not rc.interleave:
        # the reference's sparse kernel is order-nondeterministic: only per-physical counts are defined
        ref = uep_ref.sparse_reroute_quota(d_ids, pd["l2p"], pd["lcnts"], pd["rank_quota_prefix"])
        assert torch.equal(torch.bincount(ref.flatten(), minlength=P), torch.bincount(got.flatten(), minlength=P))


def test_sparse_reroute_invalid_ids(native_lib, cuda_device):
    rc = REROUTE_CASES[0]
    plan, ids, rmap, probs, L, P, pd = _setup(rc, cuda_device)
    bad = ids.copy()
    bad[5, 2] = -3
    bad[100, 0] = L
    bad[4095, 7] = 1 << 30
    exp = O.sparse_reroute(bad, plan, True)
    got = G.cuda_sparse_reroute(torch.from_numpy(bad).to(cuda_device), pd["l2p"], pd["lcnts"], pd["rank_quota_prefix"])
    assert np.array_equal(got.cpu().numpy(), exp)


@pytest.mark.parametrize("n,P", [(65536, 160), (131072, 320), (1000, 80), (1, 16), (0, 16), (5000, 2600)])
def test_dispatch_positions_and_gather(native_lib, cuda_device, n, P):
    rng = np.random.default_rng(n + P)
    phys = rng.integers(0, P, size=n).astype(np.int32)
    if n > 10:
        phys[3] = -1
        phys[7] = P + 2
    exp_pos, exp_off = O.dispatch_positions(phys, P)
    pos, off = G.cuda_dispatch_positions(torch.from_numpy(phys).to(cuda_device), P)
    if n:
        assert np.array_equal(pos.cpu().numpy(), exp_pos)
        assert np.array_equal(off.cpu().numpy(), exp_off)
        assert np.array_equal(np.sort(pos.cpu().numpy()), np.arange(n)), "positions must be a permutation"
    for hidden in (64, 4096) if n <= 5000 else (512,):
        rows = torch.from_numpy(rng.integers(0, 1 << 16, size=(max(n, 1), hidden)).astype(np.uint16)).to(cuda_device)
        if n == 0:
            continue
        got, status = G.cuda_gather_rows(rows, pos)
        assert status.tolist() == [0, 0]
        exp = O.gather_rows16(rows.cpu().numpy(), exp_pos)
        assert np.array_equal(got.cpu().numpy(), exp)


def test_gather_rows_full_size_roundtrip(native_lib, cuda_device):
    """cfg4 shape: [8192*8, 4096] bf16 rows. Scatter by the inverse permutation, gather back: identity."""
    n, hidden, P = 8192 * 8, 4096, 160
    rng = np.random.default_rng(4)
    phys = torch.from_numpy(rng.integers(0, P, size=n).astype(np.int32)).to(cuda_device)
    pos, off = G.cuda_dispatch_positions(phys, P)
    rows = torch.randn(n, hidden, device=cuda_device, dtype=torch.float32).mul_(1e-3).to(torch.bfloat16)
    permuted = torch.empty_like(rows)
    permuted[pos.long()] = rows  # what the dispatcher would deliver, grouped by physical expert
    got, status = G.cuda_gather_rows(permuted.view(torch.int16), pos)
    assert status.tolist() == [0, 0]
    assert torch.equal(got.view(torch.bfloat16), rows)
    assert int(off[-1]) == n


def test_gather_rows_unaligned_and_bad_index(native_lib, cuda_device):
    rows = torch.arange(50 * 6, dtype=torch.uint8, device=cuda_device).reshape(50, 6)  # 6-byte rows: plain path
    pos = torch.tensor([3, 0, 49, 7], dtype=torch.int32, device=cuda_device)
    got, status = G.cuda_gather_rows(rows, pos)
    assert torch.equal(got, rows[pos.long()]) and status.tolist() == [0, 0]
    rows16 = torch.arange(8 * 32, dtype=torch.uint8, device=cuda_device).reshape(8, 32)
    pos_bad = torch.tensor([1, 99, 2], dtype=torch.int32, device=cuda_device)
    got, status = G.cuda_gather_rows(rows16, pos_bad)
    assert status[0].item() == 5 and status[1].item() == 1  # bad index recorded, row clamped to 0
    assert torch.equal(got[0], rows16[1]) and torch.equal(got[1], rows16[0]) and torch.equal(got[2], rows16[2])
