"""ctypes/numpy front end of the CPU oracle (oracle/uep_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests, by the smoke check and by the CPU-baseline
leg of the benchmark; never by the product package.
"""

from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libuep_oracle.so")

_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def build(force: bool = False) -> str:
    """Compile the oracle with g++ if the shared object is missing or stale."""
    src = os.path.join(_HERE, "uep_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_SO):
        build()
    L = C.CDLL(_SO)
    L.uep_oracle_histogram_ids32.argtypes = [_i32p, C.c_int64, C.c_int, _i32p]
    L.uep_oracle_histogram_ids64.argtypes = [_i64p, C.c_int64, C.c_int, _i32p]
    L.uep_oracle_histogram_map.argtypes = [_u8p, C.c_int, C.c_int, _i32p]
    L.uep_oracle_reduce_loads.argtypes = [_i32p, C.c_int, C.c_int, _i32p]
    L.uep_oracle_init_master_placement.argtypes = [_i32p] * 6 + [C.c_int] * 4
    L.uep_oracle_solve_placement.argtypes = (
        [_i32p] * 8
        + [C.c_int] * 5
        + [C.c_float, C.c_int32, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_void_p]
    )
    L.uep_oracle_solve_placement.restype = C.c_int
    L.uep_oracle_legacy_solve_placement.argtypes = [_i32p] * 4 + [C.c_int] * 5 + [C.c_float]
    L.uep_oracle_dense_reroute_forward.argtypes = [_u8p, _f32p, _i32p, _i32p, _i32p, _u8p, _f32p] + [C.c_int] * 5
    L.uep_oracle_dense_reroute_forward_rr.argtypes = [_u8p, _f32p, _i32p, _i32p, _u8p, _f32p] + [C.c_int] * 4
    L.uep_oracle_sparse_reroute32.argtypes = [_i32p, _i32p, C.c_int64, C.c_int, _i32p, _i32p, _i32p, C.c_int, C.c_int]
    L.uep_oracle_sparse_reroute64.argtypes = [_i64p, _i64p, C.c_int64, C.c_int, _i32p, _i32p, _i32p, C.c_int, C.c_int]
    L.uep_oracle_dense_reroute_backward.argtypes = [_f32p, _u8p, _u8p, _i32p, _i32p, _f32p] + [C.c_int] * 4
    L.uep_oracle_dispatch_positions.argtypes = [_i32p, C.c_int64, C.c_int, _i32p, C.c_void_p]
    L.uep_oracle_gather_rows16.argtypes = [_u16p, _i32p, _u16p, C.c_int64, C.c_int]
    L.uep_oracle_weight_sync_recv.argtypes = [
        C.c_int, C.c_int, C.c_int, _i32p, _i32p, C.c_int, C.POINTER(C.c_void_p), C.c_int64, C.c_void_p,
        C.c_int64, C.c_int64,
    ]
    L.uep_oracle_grad_reduce_shard.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int64]
    L.uep_oracle_time_forward_layer.argtypes = [
        _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int32, C.c_int, C.c_int, C.c_float,
        C.c_int, C.POINTER(C.c_void_p), C.c_int64, C.POINTER(C.c_void_p), _i32p, _i32p, C.c_int, C.c_int,
        C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double),
    ]
    L.uep_oracle_time_forward_layer.restype = C.c_double
    L.uep_oracle_hardware_threads.restype = C.c_int
    _lib = L
    return L


@dataclass
class SolverParams:
    """Solver tunables at the reference's defaults (ultra_ep/config.py:54-71 of the reference)."""

    balance_threshold: float = 1.0
    min_tokens_per_replica: int = 1024
    allow_zero_master_quota: bool = False
    locality_aware: bool = True
    oracle_eps: float = 0.01
    interleave: bool = True


@dataclass
class Plan:
    p2l: np.ndarray  # [P]
    l2p: np.ndarray  # [L, D]
    lcnts: np.ndarray  # [L]
    quota: np.ndarray  # [L, D]
    quota_prefix: np.ndarray  # [L, D]
    rank_quota_prefix: np.ndarray  # [L, D]   (specific to `my_rank`)
    threshold: np.ndarray | None = None  # [num_domains]
    path: np.ndarray | None = None  # [num_domains] 0 none, 1 fast, 2 precheck, 3 search

    def fields(self):
        return {
            "p2l": self.p2l, "l2p": self.l2p, "lcnts": self.lcnts, "quota": self.quota,
            "quota_prefix": self.quota_prefix, "rank_quota_prefix": self.rank_quota_prefix,
        }


def histogram_ids(ids: np.ndarray, L: int) -> np.ndarray:
    ids = np.ascontiguousarray(ids).reshape(-1)
    out = np.empty(L, np.int32)
    if ids.dtype == np.int64:
        lib().uep_oracle_histogram_ids64(ids, ids.size, L, out)
    else:
        lib().uep_oracle_histogram_ids32(ids.astype(np.int32, copy=False), ids.size, L, out)
    return out


def histogram_map(routing_map: np.ndarray) -> np.ndarray:
    m = np.ascontiguousarray(routing_map).view(np.uint8)
    T, L = m.shape
    out = np.empty(L, np.int32)
    lib().uep_oracle_histogram_map(m, T, L, out)
    return out


def init_master_placement(num_ranks: int, M: int, R: int, D: int | None = None) -> Plan:
    D = D or num_ranks
    L, P = num_ranks * M, num_ranks * (M + R)
    p = Plan(*(np.empty(s, np.int32) for s in [(P,), (L, D), (L,), (L, D), (L, D), (L, D)]))
    lib().uep_oracle_init_master_placement(p.p2l, p.l2p, p.lcnts, p.quota, p.quota_prefix, p.rank_quota_prefix,
                                           num_ranks, M, R, D)
    return p


def legacy_solve_placement(global_loads: np.ndarray, num_ranks: int, M: int, R: int, nvl_ranks: int | None = None,
                           balance_threshold: float = 1.0, D: int | None = None) -> Plan:
    """The plan of legacy_placement=True (host-side solver of the reference): p2l, l2p, lcnts; quotas stay zero."""
    loads = np.ascontiguousarray(global_loads, dtype=np.int32)
    L, P = num_ranks * M, num_ranks * (M + R)
    assert loads.shape == (L,)
    D = D or num_ranks
    p = Plan(*(np.zeros(s, np.int32) for s in [(P,), (L, D), (L,), (L, D), (L, D), (L, D)]))
    lib().uep_oracle_legacy_solve_placement(loads, p.p2l, p.l2p, p.lcnts, num_ranks, M, R, nvl_ranks or num_ranks, D,
                                            balance_threshold)
    return p


def solve_placement(loads_per_rank: np.ndarray, M: int, R: int, nvl_ranks: int | None = None, my_rank: int = 0,
                    params: SolverParams | None = None, D: int | None = None,
                    global_loads: np.ndarray | None = None) -> Plan:
    """loads_per_rank: int32 [N, L]. Returns the plan as rank `my_rank` computes it."""
    params = params or SolverParams()
    lpr = np.ascontiguousarray(loads_per_rank, dtype=np.int32)
    N, L = lpr.shape
    assert L == N * M
    nvl = nvl_ranks or N
    D = D or N
    P = N * (M + R)
    if global_loads is None:
        global_loads = np.empty(L, np.int32)
        lib().uep_oracle_reduce_loads(lpr, N, L, global_loads)
    global_loads = np.ascontiguousarray(global_loads, dtype=np.int32)
    p = Plan(*(np.empty(s, np.int32) for s in [(P,), (L, D), (L,), (L, D), (L, D), (L, D)]))
    p.threshold = np.zeros(N // nvl, np.int32)
    p.path = np.zeros(N // nvl, np.int32)
    rc = lib().uep_oracle_solve_placement(
        global_loads, lpr, p.p2l, p.l2p, p.lcnts, p.quota, p.quota_prefix, p.rank_quota_prefix,
        N, nvl, M, R, D, params.balance_threshold, params.min_tokens_per_replica,
        int(params.allow_zero_master_quota), int(params.locality_aware), params.oracle_eps, my_rank,
        p.threshold.ctypes.data, p.path.ctypes.data)
    if rc != 0:
        raise RuntimeError(f"oracle solve_placement failed with code {rc}")
    return p


def dense_reroute_forward(routing_map: np.ndarray, probs: np.ndarray, plan: Plan, P: int, interleave: bool = True,
                          quota: bool = True):
    m = np.ascontiguousarray(routing_map).view(np.uint8)
    pr = np.ascontiguousarray(probs, dtype=np.float32)
    T, L = m.shape
    D = plan.l2p.shape[1]
    out_map = np.empty((T, P), np.uint8)
    out_probs = np.empty((T, P), np.float32)
    if quota:
        lib().uep_oracle_dense_reroute_forward(m, pr, plan.l2p, plan.lcnts, plan.rank_quota_prefix, out_map,
                                               out_probs, T, L, P, D, int(interleave))
    else:
        lib().uep_oracle_dense_reroute_forward_rr(m, pr, plan.l2p, plan.lcnts, out_map, out_probs, T, L, P, D)
    return out_probs, out_map.view(np.bool_)


def sparse_reroute(ids: np.ndarray, plan: Plan, interleave: bool = True) -> np.ndarray:
    a = np.ascontiguousarray(ids)
    L, D = plan.l2p.shape
    out = np.empty_like(a)
    if a.dtype == np.int64:
        lib().uep_oracle_sparse_reroute64(a.reshape(-1), out.reshape(-1), a.size, L, plan.l2p, plan.lcnts,
                                          plan.rank_quota_prefix, D, int(interleave))
    else:
        assert a.dtype == np.int32
        lib().uep_oracle_sparse_reroute32(a.reshape(-1), out.reshape(-1), a.size, L, plan.l2p, plan.lcnts,
                                          plan.rank_quota_prefix, D, int(interleave))
    return out


def dense_reroute_backward(grad_expanded: np.ndarray, routing_map: np.ndarray, expanded_map: np.ndarray,
                           plan: Plan) -> np.ndarray:
    g = np.ascontiguousarray(grad_expanded, dtype=np.float32)
    m = np.ascontiguousarray(routing_map).view(np.uint8)
    em = np.ascontiguousarray(expanded_map).view(np.uint8)
    T, L = m.shape
    P = g.shape[1]
    out = np.empty((T, L), np.float32)
    lib().uep_oracle_dense_reroute_backward(g, m, em, plan.l2p, plan.lcnts, out, T, L, P, plan.l2p.shape[1])
    return out


def physical_loads_from_plan(plan: Plan, P: int) -> np.ndarray:
    """Tokens per physical slot under a plan: quota[l, j] scattered to l2p[l, j] (ultra_ep/manager.py:345-357
    of the reference, the scatter_add form of its profiling kernel)."""
    out = np.zeros(P, np.int32)
    l2p = np.asarray(plan.l2p).reshape(-1)
    quota = np.asarray(plan.quota).reshape(-1)
    valid = l2p >= 0
    np.add.at(out, l2p[valid], quota[valid])
    return out


def dispatch_positions(phys_ids: np.ndarray, P: int):
    a = np.ascontiguousarray(phys_ids, dtype=np.int32).reshape(-1)
    pos = np.empty(a.size, np.int32)
    offsets = np.empty(P + 1, np.int32)
    lib().uep_oracle_dispatch_positions(a, a.size, P, pos, offsets.ctypes.data)
    return pos, offsets


def gather_rows16(rows: np.ndarray, pos: np.ndarray) -> np.ndarray:
    r = np.ascontiguousarray(rows).view(np.uint16)
    out = np.empty_like(r)
    lib().uep_oracle_gather_rows16(r, np.ascontiguousarray(pos, dtype=np.int32), out, r.shape[0], r.shape[1])
    return out


def weight_sync_expected(rank: int, M: int, R: int, plan: Plan, master_shards: list, replica_before: np.ndarray,
                         shard_offset: int, shard_bytes: int) -> np.ndarray:
    """Expected contents of rank's replica buffer ([R, slot_stride] uint8) after weight_sync of one shard.

    master_shards[r*M+m] is a contiguous uint8 array holding that shard of master m on rank r."""
    out = np.ascontiguousarray(replica_before).copy()
    ptrs = (C.c_void_p * len(master_shards))(*[s.ctypes.data for s in master_shards])
    lib().uep_oracle_weight_sync_recv(rank, M, R, plan.p2l, plan.l2p, plan.l2p.shape[1], ptrs, shard_bytes,
                                      out.ctypes.data, out.shape[1], shard_offset)
    return out


def grad_reduce_shard(master: np.ndarray, replicas: list) -> None:
    """In place: master += replicas in order (fp32, fixed order); replicas zeroed."""
    assert master.dtype == np.float32 and master.flags.c_contiguous
    ptrs = (C.c_void_p * max(1, len(replicas)))(*[r.ctypes.data for r in replicas])
    lib().uep_oracle_grad_reduce_shard(master.ctypes.data, ptrs, len(replicas), master.size)


# ----------------------------------------------------------------------------------------
# Invariants the reference's own tests assert (tests/test_solving.py:56-99, 140-160 of the
# reference), restated on numpy arrays.
# ----------------------------------------------------------------------------------------
def assert_plan_legal(plan: Plan, num_ranks: int, M: int, R: int, nvl: int) -> None:
    Lp = M + R
    L = num_ranks * M
    l2p, lcnts, p2l = plan.l2p, plan.lcnts, plan.p2l
    logical = np.arange(L)
    master_rank = logical // M
    valid = l2p >= 0
    phys = np.maximum(l2p, 0)
    phys_rank = phys // Lp
    phys_local = phys % Lp
    expected_master = master_rank * Lp + logical % M
    assert np.array_equal(l2p[:, 0], expected_master), "master not at slot 0 / home id"
    assert np.array_equal(lcnts, valid.sum(1).astype(np.int32)), "lcnts != number of valid slots"
    same_domain = (phys_rank // nvl) == (master_rank[:, None] // nvl)
    assert (same_domain | ~valid).all(), "replica crosses NVL domain"
    for r in range(num_ranks):
        copies = ((phys_rank == r) & valid).sum(1)
        assert (copies <= 1).all(), "duplicate logical expert on a rank"
    redundant = phys_local >= M
    assert ((redundant | ~valid) | (l2p == expected_master[:, None])).all()
    used = (p2l.reshape(num_ranks, Lp)[:, M:] >= 0).sum()
    assert used <= num_ranks * R
    # p2l / l2p consistency
    for l in range(L):
        for j in range(lcnts[l]):
            assert p2l[l2p[l, j]] == l
    assert (plan.quota[valid] >= 0).all()
    assert np.array_equal(plan.quota_prefix[np.arange(L), lcnts - 1], (plan.quota * valid).sum(1))


def assert_rank_quota_complete(rank_quota_prefix: np.ndarray, lcnts: np.ndarray, my_loads: np.ndarray) -> None:
    L = lcnts.shape[0]
    last = rank_quota_prefix[np.arange(L), np.maximum(lcnts - 1, 0)]
    assert np.array_equal(last, my_loads), "rank quota prefixes do not match source loads"
