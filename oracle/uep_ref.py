"""ctypes front end of oracle/_ref/libuep_ref.so: the reference's own CUDA kernels, built
unmodified from the reference checkout by `make -C oracle ref` (see oracle/ref_shim.cu).

TEST INFRASTRUCTURE ONLY. Needs a GPU. Used to pin the CPU oracle and the new kernels
against the real reference and to time the reference's sm_100 build.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(_HERE, "_ref", "libuep_ref.so")

_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float
_lib = None


def available() -> bool:
    return os.path.exists(SO)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        L = C.CDLL(SO)
        L.uep_ref_last_error.restype = C.c_char_p
        L.uep_ref_solve_placement.argtypes = [_vp] * 9 + [_i] * 6 + [_f, C.c_int32, _i, _i, _f, _i, _i]
        L.uep_ref_rmap_local_sum.argtypes = [_i, _i, _vp, _vp, _vp]
        L.uep_ref_topk_local_sum.argtypes = [_vp, _i, _i, _i, _vp, _vp]
        L.uep_ref_reduce_per_rank_loads.argtypes = [_vp, _vp, _i, _i, _vp]
        L.uep_ref_dense_reroute_forward_quota.argtypes = [_vp] * 8 + [_i] * 5 + [_vp]
        L.uep_ref_dense_reroute_backward.argtypes = [_vp] * 6 + [_i] * 4 + [_vp]
        L.uep_ref_sparse_reroute_quota.argtypes = [_vp] * 5 + [_i] * 4 + [_vp]
        L.uep_ref_workspace_create.restype = _vp
        L.uep_ref_workspace_create.argtypes = [_i, _i, _i, _i, _i64, _i64, _i, _i, _i64, _i64, _i, _i,
                                               C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp)]
        L.uep_ref_workspace_destroy.argtypes = [_vp]
        L.uep_ref_weight_sync.argtypes = [_vp] * 11
        L.uep_ref_grad_reduce.argtypes = [_vp] * 6 + [_i, _i, _vp]
        _lib = L
    return _lib


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference {what} failed: {lib().uep_ref_last_error().decode(errors='replace')}")


def solve_placement(loads_per_rank, M, R, nvl=None, my_rank=0, balance_threshold=1.0, min_tokens=1024,
                    allow_zero=False, locality=True, eps=0.01, kernel_stage=1, global_loads=None):
    """torch int32 cuda [N, L] -> dict of torch tensors, via the reference's solve_placement."""
    import torch

    lpr = loads_per_rank.contiguous()
    N, L = lpr.shape
    nvl = nvl or N
    D = N
    P = N * (M + R)
    dev = lpr.device
    gl = lpr.sum(0, dtype=torch.int32).contiguous() if global_loads is None else global_loads.contiguous()
    out = {
        "p2l": torch.empty(P, dtype=torch.int32, device=dev),
        "l2p": torch.empty(L, D, dtype=torch.int32, device=dev),
        "lcnts": torch.empty(L, dtype=torch.int32, device=dev),
        "quota": torch.empty(L, D, dtype=torch.int32, device=dev),
        "quota_prefix": torch.empty(L, D, dtype=torch.int32, device=dev),
        "rank_quota_prefix": torch.empty(L, D, dtype=torch.int32, device=dev),
    }
    stream = torch.cuda.current_stream().cuda_stream
    _check(lib().uep_ref_solve_placement(
        gl.data_ptr(), lpr.data_ptr(), out["p2l"].data_ptr(), out["l2p"].data_ptr(), out["lcnts"].data_ptr(),
        out["quota"].data_ptr(), out["quota_prefix"].data_ptr(), out["rank_quota_prefix"].data_ptr(), stream,
        L, N, M, R, nvl, D, balance_threshold, min_tokens, int(allow_zero), int(locality), eps, kernel_stage,
        my_rank), "solve_placement")
    return out


def dense_reroute_forward(routing_map, probs, l2p, lcnts, rqp, P, interleave=True):
    import torch

    T, L = routing_map.shape
    D = l2p.shape[1]
    dev = routing_map.device
    out_map = torch.zeros(T, P, dtype=torch.bool, device=dev)
    out_probs = torch.zeros(T, P, dtype=torch.float32, device=dev)
    tiles = (T + 127) // 128
    scratch = torch.empty(max(1, L * tiles), dtype=torch.int32, device=dev)
    _check(lib().uep_ref_dense_reroute_forward_quota(
        routing_map.data_ptr(), probs.data_ptr(), l2p.data_ptr(), lcnts.data_ptr(), rqp.data_ptr(),
        out_map.data_ptr(), out_probs.data_ptr(), scratch.data_ptr(), T, L, P, D, int(interleave),
        torch.cuda.current_stream().cuda_stream), "dense_reroute_forward")
    return out_probs, out_map


def dense_reroute_backward(grad_expanded, routing_map, expanded_map, l2p, lcnts):
    import torch

    T, L = routing_map.shape
    P = grad_expanded.shape[1]
    out = torch.zeros(T, L, dtype=torch.float32, device=routing_map.device)
    _check(lib().uep_ref_dense_reroute_backward(
        grad_expanded.data_ptr(), routing_map.data_ptr(), expanded_map.data_ptr(), l2p.data_ptr(), lcnts.data_ptr(),
        out.data_ptr(), T, L, P, l2p.shape[1], torch.cuda.current_stream().cuda_stream), "dense_reroute_backward")
    return out


def histogram_map(routing_map):
    import torch

    T, L = routing_map.shape
    loads = torch.empty(L, dtype=torch.int32, device=routing_map.device)
    _check(lib().uep_ref_rmap_local_sum(T, L, routing_map.data_ptr(), loads.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream), "rmap_local_sum")
    return loads


def histogram_ids64(ids, L):
    import torch

    T, K = ids.shape
    loads = torch.empty(L, dtype=torch.int32, device=ids.device)
    _check(lib().uep_ref_topk_local_sum(ids.data_ptr(), T, K, L, loads.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream), "topk_local_sum")
    return loads


def sparse_reroute_quota(ids64, l2p, lcnts, rqp):
    """In place on a copy; ordinals come from an atomic counter, so only counts are defined."""
    import torch

    out = ids64.clone()
    T, K = out.shape
    L = lcnts.shape[0]
    counters = torch.empty(L, dtype=torch.int32, device=out.device)
    _check(lib().uep_ref_sparse_reroute_quota(out.data_ptr(), l2p.data_ptr(), lcnts.data_ptr(), rqp.data_ptr(),
                                              counters.data_ptr(), T, K, L, l2p.shape[1],
                                              torch.cuda.current_stream().cuda_stream), "sparse_reroute_quota")
    return out


class Workspace:
    """One rank's scratch for the reference's weight_sync / grad_reduce launch pairs."""

    def __init__(self, rank, nvl, M, R, fc1_numel, fc2_numel, weight_elem_bytes, scale_elem_bytes, fc1_scale_numel,
                 fc2_scale_numel, D, remote_weight, remote_scale, remote_grad):
        def table(ptrs):
            if ptrs is None:
                return None
            return (C.c_void_p * len(ptrs))(*ptrs)

        self._tables = (table(remote_weight), table(remote_scale), table(remote_grad))
        self.handle = lib().uep_ref_workspace_create(rank, nvl, M, R, fc1_numel, fc2_numel, weight_elem_bytes,
                                                     scale_elem_bytes, fc1_scale_numel, fc2_scale_numel, D, 0,
                                                     *self._tables)
        if not self.handle:
            raise RuntimeError(f"reference workspace: {lib().uep_ref_last_error().decode(errors='replace')}")

    def weight_sync(self, p2l, l2p, lcnts, fc1_ptrs, fc2_ptrs, fc1_scale_ptrs, fc2_scale_ptrs, replica_weight,
                    replica_scale, stream):
        _check(lib().uep_ref_weight_sync(
            self.handle, p2l.data_ptr(), l2p.data_ptr(), lcnts.data_ptr(), fc1_ptrs.data_ptr(), fc2_ptrs.data_ptr(),
            fc1_scale_ptrs.data_ptr() if fc1_scale_ptrs is not None else 0,
            fc2_scale_ptrs.data_ptr() if fc2_scale_ptrs is not None else 0,
            replica_weight.data_ptr(), replica_scale.data_ptr() if replica_scale is not None else 0, stream),
            "weight_sync")

    def grad_reduce(self, p2l, l2p, lcnts, fc1_grad_ptrs, fc2_grad_ptrs, num_sms, deterministic, stream):
        _check(lib().uep_ref_grad_reduce(self.handle, p2l.data_ptr(), l2p.data_ptr(), lcnts.data_ptr(),
                                         fc1_grad_ptrs.data_ptr(), fc2_grad_ptrs.data_ptr(), num_sms,
                                         int(deterministic), stream), "grad_reduce")

    def close(self):
        if self.handle:
            lib().uep_ref_workspace_destroy(self.handle)
            self.handle = None


# ---- the reference's legacy host-side solver (no GPU needed) ---------------------------------
LEGACY_SO = os.path.join(_HERE, "_ref", "libuep_ref_legacy.so")
_legacy = None


def legacy_available() -> bool:
    return os.path.exists(LEGACY_SO)


def legacy_solve_host(global_loads, num_ranks: int, M: int, R: int, nvl_ranks: int, balance_threshold: float = 1.0,
                      D: int | None = None):
    """(p2l, l2p, lcnts) as csrc/kernels/legacy/placement_cpu.cpp computes them, on host arrays."""
    import numpy as np

    global _legacy
    if _legacy is None:
        _legacy = C.CDLL(LEGACY_SO)
        _legacy.uep_ref_legacy_solve_host.argtypes = [_vp] * 4 + [_i] * 6 + [_f]
    loads = np.ascontiguousarray(global_loads, dtype=np.int32)
    L, P = num_ranks * M, num_ranks * (M + R)
    D = D or num_ranks
    p2l = np.zeros(P, np.int32)
    l2p = np.zeros((L, D), np.int32)
    lcnts = np.zeros(L, np.int32)
    _legacy.uep_ref_legacy_solve_host(loads.ctypes.data, p2l.ctypes.data, l2p.ctypes.data, lcnts.ctypes.data, L, num_ranks,
                                      M, R, nvl_ranks, D, balance_threshold)
    return p2l, l2p, lcnts
