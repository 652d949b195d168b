"""The allocation-free sparse reroute entry point (uep_sparse_reroute_i32_static).

It exists for hosts that cannot call cudaMalloc where routing happens (a serving process whose
own pool owns the device memory, or a region in which the allocator is frozen): its scratch is a
fixed array inside the library. Checked here through the C ABI against the regular entry point,
bit for bit, on two calls in a row with different inputs (the array is reused, so the second call
runs over the first call's leftovers), and for its size limit. Collected last on purpose."""

import numpy as np
import pytest
import torch

import gpu_util as G
from oracle import uep_oracle as O
from ultra_ep_b200 import capi
from ultra_ep_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _static_reroute(lib, ids, plan_dev, interleave=True):
    T, K = ids.shape
    L, D = plan_dev["l2p"].shape
    out = torch.full_like(ids, -7)
    rc = lib.uep_sparse_reroute_i32_static(ids.data_ptr(), out.data_ptr(), T, K, L, plan_dev["l2p"].data_ptr(),
                                           plan_dev["lcnts"].data_ptr(), plan_dev["rank_quota_prefix"].data_ptr(), D,
                                           int(interleave), G.stream_ptr())
    return rc, out


def test_static_scratch_entry_matches_regular_entry(native_lib, cuda_device):
    lib = capi.lib()
    first = None
    for call, (name, rank, interleave) in enumerate([("cfg3_qwen3_235b_fp8", 6, True), ("cfg1_plan_reroute", 2, False)]):
        cfg = W.CONFIGS[name]
        lpr = W.loads_per_rank(cfg)
        plan = O.solve_placement(lpr, cfg.masters, cfg.redundant, cfg.ep, rank)
        pd = G.plan_to_device(plan, cuda_device)
        ids = torch.from_numpy(W.routing_ids(cfg, rank)).to(cuda_device)
        expected = G.cuda_sparse_reroute(ids, pd["l2p"], pd["lcnts"], pd["rank_quota_prefix"], interleave)
        rc, got = _static_reroute(lib, ids, pd, interleave)
        capi.check(rc, "uep_sparse_reroute_i32_static")
        torch.cuda.synchronize()
        assert torch.equal(got, expected), f"call {call}: static-scratch result differs from the regular entry point"
        assert np.array_equal(got.cpu().numpy(), O.sparse_reroute(ids.cpu().numpy(), plan, interleave))
        if first is None:
            first = got.clone()
    assert first is not None


def test_static_scratch_entry_rejects_oversize(native_lib, cuda_device):
    lib = capi.lib()
    L, D = 512, 8
    dummy = torch.zeros(8, dtype=torch.int32, device=cuda_device)
    # 2^20 entries with 512 experts need 512 * 512 + 4 int32: four more than the array holds
    rc = lib.uep_sparse_reroute_i32_static(dummy.data_ptr(), dummy.data_ptr(), 1 << 17, 8, L, dummy.data_ptr(),
                                           dummy.data_ptr(), dummy.data_ptr(), D, 1, G.stream_ptr())
    assert rc == -1
    msg = lib.uep_last_error()
    assert b"built-in array holds 262144" in msg and b"uep_sparse_reroute_i32" in msg
    # empty input is fine and launches nothing
    assert lib.uep_sparse_reroute_i32_static(None, None, 0, 8, L, None, None, None, D, 1, G.stream_ptr()) == 0
