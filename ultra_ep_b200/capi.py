"""ctypes binding of the C ABI declared in include/uep_b200.h.

The library must have been built (python -m ultra_ep_b200.build); a missing library is an
error, never a reason to fall back to another implementation.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libuep_b200.so")

UEP_OK = 0
IPC_HANDLE_BYTES = 64

# uep_buffer_id
(BUF_P2L, BUF_L2P, BUF_LCNTS, BUF_QUOTA, BUF_QUOTA_PREFIX, BUF_RANK_QUOTA_PREFIX, BUF_GLOBAL_LOADS,
 BUF_LOADS_PER_RANK, BUF_REPLICA_WEIGHT, BUF_REPLICA_FC1_WEIGHT, BUF_REPLICA_FC2_WEIGHT, BUF_REPLICA_SCALE,
 BUF_REPLICA_FC1_SCALE, BUF_REPLICA_FC2_SCALE, BUF_REPLICA_GRAD, BUF_REPLICA_FC1_GRAD, BUF_REPLICA_FC2_GRAD,
 BUF_PHYSICAL_LOADS) = range(18)

DEV_STATUS_NAMES = {
    0: "ok", 1: "timeout waiting for a peer's load row", 2: "timeout waiting for a peer's weight_sync flag",
    3: "timeout waiting for an async bulk copy", 4: "solver: final plan infeasible", 5: "plan entry outside its table",
}


class SolverParams(C.Structure):
    _fields_ = [
        ("balance_threshold", C.c_float),
        ("locality_aware", C.c_int32),
        ("min_tokens_per_replica", C.c_int32),
        ("allow_zero_master_quota", C.c_int32),
        ("oracle_eps", C.c_float),
        ("reroute_interleave", C.c_int32),
    ]

    @classmethod
    def defaults(cls, **kw):
        p = cls(1.0, 1, 1024, 0, 0.01, 1)
        for k, v in kw.items():
            setattr(p, k, v)
        return p


class Config(C.Structure):
    _fields_ = [
        ("num_ranks", C.c_int32), ("nvl_ranks", C.c_int32), ("rank", C.c_int32), ("sim_ranks", C.c_int32),
        ("num_layers", C.c_int32), ("num_local_master_experts", C.c_int32),
        ("num_local_redundant_experts", C.c_int32),
        ("expert_fc1_numel", C.c_int64), ("expert_fc2_numel", C.c_int64),
        ("weight_data_element_bytes", C.c_int32), ("weight_scale_element_bytes", C.c_int32),
        ("expert_fc1_weight_scale_numel", C.c_int64), ("expert_fc2_weight_scale_numel", C.c_int64),
        ("grad_element_bytes", C.c_int32), ("is_train", C.c_int32), ("legacy_placement", C.c_int32),
        ("solver", SolverParams),
        ("quota_kernel_stage", C.c_int32), ("grad_reduce_num_sms", C.c_int32),
        ("grad_reduce_deterministic", C.c_int32), ("weight_sync_plan_mode", C.c_int32),
        ("weight_sync_relay_min_replicas", C.c_int32), ("weight_sync_relay_max_relays", C.c_int32),
        ("weight_sync_relay_min_fanout_gain", C.c_int32), ("weight_sync_num_sms", C.c_int32),
        ("wait_timeout_ms", C.c_int32), ("reroute_max_tokens", C.c_int32), ("reroute_max_topk", C.c_int32),
    ]


_vp, _i, _i64 = C.c_void_p, C.c_int, C.c_int64

# name -> (restype, argtypes): every symbol include/uep_b200.h declares
SIGNATURES = {
    "uep_last_error": (C.c_char_p, []),
    "uep_version": (C.c_char_p, []),
    "uep_histogram_ids32": (_i, [_vp, _i64, _i, _vp, _vp]),
    "uep_histogram_ids64": (_i, [_vp, _i64, _i, _vp, _vp]),
    "uep_histogram_map": (_i, [_vp, _i, _i, _vp, _vp]),
    "uep_solve_placement": (_i, [_vp] * 8 + [_i] * 5 + [C.POINTER(SolverParams), _i, _vp, _vp]),
    "uep_legacy_solve_placement": (_i, [_vp] * 7 + [_i] * 5 + [C.c_float, _vp, _vp]),
    "uep_init_master_placement": (_i, [_vp] * 6 + [_i] * 4 + [_vp]),
    "uep_reroute_scratch_elems": (_i64, [_i64, _i, _i]),
    "uep_dense_reroute_forward": (_i, [_vp] * 8 + [_i] * 6 + [_vp]),
    "uep_dense_reroute_backward": (_i, [_vp] * 6 + [_i] * 4 + [_vp]),
    "uep_sparse_reroute_i32": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "uep_sparse_reroute_i64": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "uep_sparse_reroute_i32_static": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "uep_dispatch_positions": (_i, [_vp, _i64, _i, _vp, _vp, _vp, _vp]),
    "uep_dispatch_scratch_elems": (_i64, [_i64, _i]),
    "uep_gather_rows": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "uep_manager_create": (_i, [C.POINTER(Config), C.POINTER(_vp)]),
    "uep_manager_export_handle": (_i, [_vp, _vp]),
    "uep_manager_connect": (_i, [_vp, _vp]),
    "uep_manager_destroy": (_i, [_vp]),
    "uep_manager_num_local": (_i, [_vp]),
    "uep_manager_num_sms": (_i, [_vp]),
    "uep_manager_buffer": (_i, [_vp, _i, _i, C.POINTER(_vp), C.POINTER(_i), C.POINTER(_i64), C.POINTER(_i64)]),
    "uep_manager_peer_buffer": (_i, [_vp, _i, _i, _i, C.POINTER(_vp)]),
    "uep_debug_link_probe": (_i, [_vp, _i, _i64, _i, _i, C.POINTER(C.c_float)]),
    "uep_update_placement": (_i, [_vp, _i, _i, C.POINTER(_vp), C.POINTER(_i), _i, _vp]),
    "uep_weight_sync": (_i, [_vp, _i] + [C.POINTER(_vp)] * 4 + [_vp, _i, _vp, C.POINTER(_vp)]),
    "uep_grad_reduce": (_i, [_vp, _i] + [C.POINTER(_vp)] * 2 + [_vp, _i, _vp, C.POINTER(_vp)]),
    "uep_reroute_dense_forward": (_i, [_vp, _i] + [C.POINTER(_vp)] * 4 + [C.POINTER(_i), _vp]),
    "uep_reroute_dense_backward": (_i, [_vp, _i] + [C.POINTER(_vp)] * 4 + [C.POINTER(_i), _i, _vp]),
    "uep_reroute_sparse": (_i, [_vp, _i, _i, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i), _i, _vp]),
    "uep_set_weight_sync_plan_mode": (_i, [_vp, _i]),
    "uep_set_grad_reduce_deterministic": (_i, [_vp, _i, _i]),
    "uep_manager_comm_stream": (_vp, [_vp]),
    "uep_event_record": (_i, [_vp, C.POINTER(_vp)]),
    "uep_event_stream_wait": (_i, [_vp, _vp]),
    "uep_event_synchronize": (_i, [_vp]),
    "uep_event_destroy": (None, [_vp]),
    "uep_poll_status": (_i, [_vp, _i, C.POINTER(_i), C.POINTER(_i)]),
    "uep_clear_status": (_i, [_vp]),
    "uep_debug_withhold_rank": (_i, [_vp, _i]),
    "uep_debug_sync_trace": (_i, [_vp, _vp, _i]),
    "uep_launch_count": (_i64, []),
    "uep_reset_launch_count": (None, []),
}

_lib = None
MISSING: list = []  # declared symbols the loaded library does not export (must stay empty)


class UepError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Load the native library and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise UepError(
            f"{LIB_PATH} is missing: build it with `python -m ultra_ep_b200.build` "
            "(there is no non-CUDA fallback for this library)")
    L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    MISSING.clear()
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(L, name)
        except AttributeError:  # the header and the library disagree; the symbol test reports it
            MISSING.append(name)
            continue
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def check(rc: int, what: str = "") -> None:
    if rc != UEP_OK:
        msg = lib().uep_last_error().decode(errors="replace")
        raise UepError(f"{what or 'uep call'} failed ({rc}): {msg}")


def ptr(t) -> int:
    """Device (or host) address of a torch tensor / numpy array, 0 for None."""
    if t is None:
        return 0
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def ptr_array(values):
    arr = (C.c_void_p * max(1, len(values)))()
    for i, v in enumerate(values):
        arr[i] = v if isinstance(v, int) else ptr(v)
    return arr


def int_array(values):
    return (C.c_int * max(1, len(values)))(*values)
