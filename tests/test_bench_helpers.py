"""Host-side helpers of the benchmark that need no GPU: the restated workload generator of the reference's own
tests, the relay rule restated from the kernel, and the link-volume accounting the roofline figures rest on."""

import numpy as np
import pytest


@pytest.mark.parametrize("target", [1.5, 2.0, 3.0])
def test_reference_style_loads_reach_the_requested_imbalance(target):
    from ultra_ep_b200 import workloads as W

    loads, ids0 = W.reference_style_loads(num_ranks=16, masters=4, topk=8, tokens_per_rank=2048, imbalance_ratio=target)
    assert loads.shape == (16, 64) and ids0.shape == (2048, 8)
    assert loads.sum() == 16 * 2048 * 8
    # every token routes to eight DIFFERENT experts
    assert all(len(set(row)) == 8 for row in ids0[:64])
    per_rank = loads.sum(axis=0).reshape(16, 4).sum(axis=1)  # tokens that land on each rank's masters
    imbalance = per_rank.max() / per_rank.mean()
    assert abs(imbalance - target) / target < 0.08, imbalance


def _plans(name, ep, microbatches):
    import bench
    from ultra_ep_b200 import workloads as W

    cfg = W.CONFIGS[name].with_ep(ep) if ep != W.CONFIGS[name].ep else W.CONFIGS[name]
    ranks = list(range(cfg.ep))
    for mb in microbatches:
        ids = [W.routing_ids(cfg, r, microbatch=mb) for r in ranks]
        yield cfg, ranks, bench.oracle_plans(cfg, ids, ranks)[0]


def test_relay_rule_and_link_volumes():
    import bench

    seen_relay = False
    for ep in (4, 8):
        for cfg, ranks, plan in _plans("cfg3_qwen3_235b_fp8", ep, range(4)):
            M, R, N = cfg.masters, cfg.redundant, cfg.ep
            reps = (plan.lcnts - 1).clip(min=0)
            assert bench.relay_selection(cfg, plan, 0, 4) is None
            forced = bench.relay_selection(cfg, plan, 2, 4)
            assert [bool(x) for x in forced] == [bool(2 <= r <= 16) for r in reps]
            adaptive = bench.relay_selection(cfg, plan, 1, 4)
            p2l = plan.p2l.reshape(N, M + R)
            floor_in = max(1, max(int((p2l[r, M:] >= 0).sum()) for r in range(N)))
            for r in range(N):
                mine = range(r * M, (r + 1) * M)
                out = sum(1 if adaptive[l] else int(reps[l]) for l in mine if reps[l] > 0)
                left = [l for l in mine if not adaptive[l] and reps[l] >= 2]
                assert out <= floor_in or not left, (ep, r, out, floor_in)
            seen_relay |= any(adaptive)
            for rel in (None, forced, adaptive):
                vol = bench.link_volumes(cfg, plan, ranks, rel)
                # what leaves the ranks arrives somewhere: relaying moves volume between senders, it adds none
                assert abs(sum(v["egress"] for v in vol) - sum(v["ingress"] for v in vol)) < 1e-9
                assert sum(v["writes"] for v in vol) == int(reps.sum())
    assert seen_relay
    # two ranks: nothing can be relayed, whatever the mode
    for cfg, ranks, plan in _plans("cfg3_qwen3_235b_fp8", 2, range(2)):
        assert bench.relay_selection(cfg, plan, 1, 4) is None and bench.relay_selection(cfg, plan, 2, 4) is None
