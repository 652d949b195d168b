"""Parity at the benchmark's FULL sizes on the simulated group (all eight ranks on one device): plans and
routing against the CPU oracle, every replica slot against its master's bytes (19 MB, 9.4 MB and 44 MB experts:
hundreds to thousands of tiles per expert, the atomic hand-out under real contention, all plan modes), and the
fp32 Wgrad reduce of 75.5 MB replicas against the fixed-order sum, bit for bit. The checks are the ones the
benchmark runs on itself (bench.py), driven here through the same C ABI."""

import argparse

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(native_lib, cuda_device):
    import bench

    return bench.Env()


def _args(plan_mode):
    return argparse.Namespace(plan_mode_resolved=plan_mode, relay_min_replicas=4, sync_sms=0, reduce_sms=42)


@pytest.mark.parametrize("name,plan_mode", [
    ("cfg2_qwen3_30b_bf16", 0), ("cfg3_qwen3_235b_fp8", 0), ("cfg3_qwen3_235b_fp8", 1), ("cfg3_qwen3_235b_fp8", 2),
    ("cfg5_dsv3_stress", 0), ("cfg5_dsv3_stress", 2),
])
def test_forward_full_size(env, name, plan_mode):
    import bench
    from ultra_ep_b200 import workloads as W

    env.failures.clear()
    fw = bench.Forward(env, W.CONFIGS[name], _args(plan_mode), num_layers=2, pool=2)
    try:
        par = fw.parity([0, 1], f"{name} plan mode {plan_mode}")
        assert all(par.values()) and not env.failures, (par, env.failures[:5])
    finally:
        fw.close()


def test_grad_reduce_full_size(env):
    import bench
    from ultra_ep_b200 import workloads as W

    env.failures.clear()
    cfg = W.CONFIGS["cfg4_qwen3_235b_bwd"]
    group, ranks = bench.make_group(env, cfg, 1, True, _args(0))
    try:
        ids = [torch.from_numpy(W.routing_ids(cfg, r)).to(env.dev) for r in ranks]
        group.update_placement(0, ids)
        torch.cuda.synchronize()
        plan = bench.oracle_plans(cfg, [x.cpu().numpy() for x in ids], ranks)[0]
        bw = bench.Backward(env, cfg, group, ranks)
        for launch in range(2):  # the second launch finds the slots the first one cleared, refilled with new values
            bw.fill_replicas(plan, salt=11 + launch)
            b1, b2 = bw.snapshot(plan)
            torch.cuda.synchronize()
            group.grad_reduce(0, bw.t1, bw.t2)
            torch.cuda.synchronize()
            group.check_status()
            assert bw.check_reduce(plan, 11 + launch, b1, b2, f"launch {launch}") and not env.failures, env.failures[:5]
    finally:
        group.destroy()
        torch.cuda.empty_cache()
