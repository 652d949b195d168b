"""Capture of one layer's forward balancing step (update_placement -> weight_sync on the
communication stream, overlapped with reroute) into a CUDA graph, and replay on new routing.

The exchange epochs of the plan and sync kernels are counted on the device, so a replayed
graph opens a new epoch every time; nothing in the step allocates or synchronises once the
scratch has its size (the first, eager call). Results of every replay are checked against the
CPU oracle: plan, physical ids and replica bytes, bit for bit."""

import numpy as np
import pytest
import torch

from oracle import uep_oracle as O
from ultra_ep_b200 import capi, sim
from ultra_ep_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _expected_replicas(cfg, plans, masters, r, nbytes):
    """Bytes of rank r's replica slots after weight_sync (unused slots keep their old content)."""
    Lp = cfg.masters + cfg.redundant
    out = {}
    p2l = plans[r].p2l.reshape(cfg.ep, Lp)
    for slot in range(cfg.redundant):
        l = int(p2l[r, cfg.masters + slot])
        if l >= 0:
            out[slot] = masters[l // cfg.masters][l % cfg.masters]
    return out


@pytest.mark.parametrize("ids_dtype", [torch.int32, torch.int64])
def test_forward_step_graph_capture_and_replay(native_lib, cuda_device, ids_dtype):
    cfg = W.CONFIGS["cfg1_plan_reroute"]
    fc1, fc2 = 2 * 64 * 128, 64 * 128
    group = sim.SimGroup(sim.make_config(cfg.ep, cfg.masters, cfg.redundant, 2, fc1_numel=fc1, fc2_numel=fc2,
                                         weight_elem_bytes=1, is_train=False, sim=True))
    gen = torch.Generator(device="cpu").manual_seed(11)
    host_masters = [[torch.randint(0, 256, (fc1 + fc2,), dtype=torch.uint8, generator=gen) for _ in range(cfg.masters)]
                    for _ in range(cfg.ep)]
    dev_masters = [[t.to(cuda_device) for t in per] for per in host_masters]
    t1 = group.pointer_tables([[t[:fc1] for t in per] for per in dev_masters])
    t2 = group.pointer_tables([[t[fc1:] for t in per] for per in dev_masters])

    def ids_of(mb):
        return [W.routing_ids(cfg, r, microbatch=mb) for r in range(cfg.ep)]

    static_ids = [torch.from_numpy(x).to(cuda_device).to(ids_dtype) for x in ids_of(0)]
    static_out = [torch.empty_like(x) for x in static_ids]

    def step():
        group.update_placement(0, static_ids)
        ev = group.weight_sync(0, t1, t2, async_finish=True)
        group.reroute_sparse(0, static_ids, static_out)
        group.wait_event(ev)

    # eager warm-up on a side stream (sizes the scratch; graphs are captured on a side stream too)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    group.check_status()

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    torch.cuda.synchronize()

    for mb in (3, 1, 2, 5):
        ids = ids_of(mb)
        for dst, src in zip(static_ids, ids):
            dst.copy_(torch.from_numpy(src).to(ids_dtype))
        for r in range(cfg.ep):  # poison the outputs of the previous replay
            static_out[r].fill_(-7)
            group.buffer(r, capi.BUF_REPLICA_WEIGHT).fill_(0xEE)
        graph.replay()
        torch.cuda.synchronize()
        group.check_status()
        lpr = np.stack([np.bincount(x.reshape(-1), minlength=cfg.num_experts) for x in ids]).astype(np.int32)
        plans = [O.solve_placement(lpr, cfg.masters, cfg.redundant, cfg.ep, r) for r in range(cfg.ep)]
        for r in range(cfg.ep):
            got = group.plan(r, 0)
            for f in ("p2l", "l2p", "lcnts", "quota", "quota_prefix", "rank_quota_prefix"):
                assert np.array_equal(got[f].cpu().numpy(), getattr(plans[r], f)), f"mb {mb} rank {r} field {f}"
            assert np.array_equal(static_out[r].cpu().numpy().astype(np.int64),
                                  O.sparse_reroute(ids[r], plans[r], True).astype(np.int64)), f"mb {mb} rank {r} ids"
            rep = group.buffer(r, capi.BUF_REPLICA_WEIGHT).cpu()
            expected = _expected_replicas(cfg, plans, host_masters, r, fc1 + fc2)
            for slot in range(cfg.redundant):
                if slot in expected:
                    assert torch.equal(rep[slot, :fc1 + fc2], expected[slot]), f"mb {mb} rank {r} slot {slot}"
                else:
                    assert bool((rep[slot] == 0xEE).all()), f"mb {mb} rank {r}: unused slot {slot} was touched"
    group.destroy()
