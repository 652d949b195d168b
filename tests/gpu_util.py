"""Helpers that drive the CUDA path through the C ABI (ctypes) on torch device tensors."""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from ultra_ep_b200 import capi

PLAN_FIELDS = ("p2l", "l2p", "lcnts", "quota", "quota_prefix", "rank_quota_prefix")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def solver_params(case) -> capi.SolverParams:
    return capi.SolverParams(case.balance_threshold, int(case.locality), case.min_tokens, int(case.allow_zero),
                             case.eps, 1)


def cuda_solve(case, rank: int, lpr_dev=None):
    """Run uep_solve_placement for one case/rank. Returns dict of torch tensors + status."""
    L_ = capi.lib()
    N, L, M, R = case.N, case.L, case.M, case.R
    D, P = N, N * (M + R)
    dev = torch.device("cuda")
    lpr = torch.from_numpy(case.loads_per_rank).to(dev) if lpr_dev is None else lpr_dev
    out = {
        "p2l": torch.full((P,), 7777, dtype=torch.int32, device=dev),
        "l2p": torch.full((L, D), 7777, dtype=torch.int32, device=dev),
        "lcnts": torch.full((L,), 7777, dtype=torch.int32, device=dev),
        "quota": torch.full((L, D), 7777, dtype=torch.int32, device=dev),
        "quota_prefix": torch.full((L, D), 7777, dtype=torch.int32, device=dev),
        "rank_quota_prefix": torch.full((L, D), 7777, dtype=torch.int32, device=dev),
    }
    gl = torch.empty(L, dtype=torch.int32, device=dev)
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    prm = solver_params(case)
    capi.check(L_.uep_solve_placement(
        lpr.data_ptr(), gl.data_ptr(), out["p2l"].data_ptr(), out["l2p"].data_ptr(), out["lcnts"].data_ptr(),
        out["quota"].data_ptr(), out["quota_prefix"].data_ptr(), out["rank_quota_prefix"].data_ptr(),
        N, case.nvl, M, R, D, C.byref(prm), rank, status.data_ptr(), stream_ptr()), "uep_solve_placement")
    out["global_loads"] = gl
    out["status"] = status
    return out


def oracle_params(case):
    from oracle import uep_oracle as O

    return O.SolverParams(case.balance_threshold, case.min_tokens, case.allow_zero, case.locality, case.eps)


def plan_to_device(plan, dev="cuda"):
    return {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in plan.fields().items()}


def cuda_dense_reroute(routing_map, probs, l2p, lcnts, rqp, P, interleave=True, quota_mode=True):
    L_ = capi.lib()
    T, L = routing_map.shape
    D = l2p.shape[1]
    dev = routing_map.device
    out_map = torch.full((T, P), 3, dtype=torch.uint8, device=dev)
    out_probs = torch.full((T, P), float("nan"), dtype=torch.float32, device=dev)
    scratch = torch.empty(int(L_.uep_reroute_scratch_elems(T, 0, L)), dtype=torch.int32, device=dev)
    capi.check(L_.uep_dense_reroute_forward(
        routing_map.data_ptr(), probs.data_ptr(), l2p.data_ptr(), lcnts.data_ptr(), rqp.data_ptr(),
        out_map.data_ptr(), out_probs.data_ptr(), scratch.data_ptr(), T, L, P, D, int(quota_mode), int(interleave),
        stream_ptr()), "uep_dense_reroute_forward")
    return out_probs, out_map.view(torch.bool)


def cuda_dense_reroute_backward(grad_expanded, routing_map, expanded_map, l2p, lcnts):
    L_ = capi.lib()
    T, L = routing_map.shape
    P = grad_expanded.shape[1]
    out = torch.full((T, L), float("nan"), dtype=torch.float32, device=routing_map.device)
    capi.check(L_.uep_dense_reroute_backward(
        grad_expanded.data_ptr(), routing_map.data_ptr(), expanded_map.data_ptr(), l2p.data_ptr(), lcnts.data_ptr(),
        out.data_ptr(), T, L, P, l2p.shape[1], stream_ptr()), "uep_dense_reroute_backward")
    return out


def cuda_sparse_reroute(ids, l2p, lcnts, rqp, interleave=True, inplace=False):
    L_ = capi.lib()
    T, K = ids.shape
    L, D = l2p.shape
    out = ids if inplace else torch.full_like(ids, -5)
    scratch = torch.empty(int(L_.uep_reroute_scratch_elems(T, max(K, 1), L)), dtype=torch.int32, device=ids.device)
    fn = L_.uep_sparse_reroute_i64 if ids.dtype == torch.int64 else L_.uep_sparse_reroute_i32
    capi.check(fn(ids.data_ptr(), out.data_ptr(), T, K, L, l2p.data_ptr(), lcnts.data_ptr(), rqp.data_ptr(), D,
                  int(interleave), scratch.data_ptr(), stream_ptr()), "uep_sparse_reroute")
    return out


def cuda_histogram(x, L, kind):
    L_ = capi.lib()
    loads = torch.full((L,), -1, dtype=torch.int32, device=x.device)
    if kind == "map":
        capi.check(L_.uep_histogram_map(x.data_ptr(), x.shape[0], L, loads.data_ptr(), stream_ptr()))
    elif kind == "ids32":
        capi.check(L_.uep_histogram_ids32(x.data_ptr(), x.numel(), L, loads.data_ptr(), stream_ptr()))
    else:
        capi.check(L_.uep_histogram_ids64(x.data_ptr(), x.numel(), L, loads.data_ptr(), stream_ptr()))
    return loads


def cuda_dispatch_positions(phys, P):
    L_ = capi.lib()
    n = phys.numel()
    pos = torch.full((n,), -1, dtype=torch.int32, device=phys.device)
    offsets = torch.full((P + 1,), -1, dtype=torch.int32, device=phys.device)
    scratch = torch.empty(int(L_.uep_dispatch_scratch_elems(n, P)), dtype=torch.int32, device=phys.device)
    capi.check(L_.uep_dispatch_positions(phys.data_ptr(), n, P, pos.data_ptr(), offsets.data_ptr(),
                                         scratch.data_ptr(), stream_ptr()), "uep_dispatch_positions")
    return pos, offsets


def cuda_gather_rows(rows, pos):
    L_ = capi.lib()
    out = torch.empty((pos.numel(), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    status = torch.zeros(2, dtype=torch.int32, device=rows.device)
    capi.check(L_.uep_gather_rows(rows.data_ptr(), pos.data_ptr(), out.data_ptr(), pos.numel(), rows.shape[0],
                                  rows.shape[1] * rows.element_size(), status.data_ptr(), stream_ptr()),
               "uep_gather_rows")
    return out, status
