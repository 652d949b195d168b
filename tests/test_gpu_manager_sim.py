"""The manager (C ABI) hosting a whole EP group on one device: plan, reroute, weight_sync and
Wgrad reduce against the CPU oracle and, where oracle/_ref is present, against the
reference's own kernels. Integer and byte results are bit-exact; the fp32 reduce is bit-exact
because the accumulation order is fixed (master, then replicas in plan slot order)."""

import ctypes as C

import numpy as np
import pytest
import torch

import gpu_util as G
from oracle import uep_oracle as O
from oracle import uep_ref
from ultra_ep_b200 import capi, sim
from ultra_ep_b200 import workloads as W

pytestmark = pytest.mark.gpu

PLAN_FIELDS = G.PLAN_FIELDS


def small_cfg(name="cfg1_plan_reroute", **over):
    import dataclasses

    return dataclasses.replace(W.CONFIGS[name], **over)


def make_group(cfg, num_layers=2, fc1=0, fc2=0, elem=2, s1=0, s2=0, train=True, **kw):
    return sim.SimGroup(sim.make_config(cfg.ep, cfg.masters, cfg.redundant, num_layers, fc1_numel=fc1, fc2_numel=fc2,
                                        weight_elem_bytes=elem, scale_elem_bytes=1, fc1_scale_numel=s1,
                                        fc2_scale_numel=s2, is_train=train, sim=True, **kw))


def oracle_plans(lpr, cfg, params=None):
    return [O.solve_placement(lpr, cfg.masters, cfg.redundant, cfg.ep, r, params) for r in range(cfg.ep)]


def assert_plans_equal(group, layer, plans):
    for r, plan in enumerate(plans):
        got = group.plan(r, layer)
        for f in PLAN_FIELDS:
            assert np.array_equal(got[f].cpu().numpy(), getattr(plan, f)), f"rank {r} field {f}"


@pytest.mark.parametrize("name", ["cfg1_plan_reroute", "cfg3_qwen3_235b_fp8", "cfg5_dsv3_stress"])
def test_update_placement_all_input_kinds(native_lib, cuda_device, name):
    cfg = W.CONFIGS[name]
    group = make_group(cfg, num_layers=3)
    ids = [W.routing_ids(cfg, r) for r in range(cfg.ep)]
    lpr = np.stack([np.bincount(x.reshape(-1), minlength=cfg.num_experts) for x in ids]).astype(np.int32)
    plans = oracle_plans(lpr, cfg)
    d_ids32 = [torch.from_numpy(x).to(cuda_device) for x in ids]
    d_ids64 = [x.long() for x in d_ids32]
    d_maps = [torch.from_numpy(W.ids_to_map(x, cfg.num_experts)).to(cuda_device) for x in ids]
    # masters-only plan before the first update (what the constructor writes)
    init = O.init_master_placement(cfg.ep, cfg.masters, cfg.redundant)
    for f in PLAN_FIELDS:
        assert np.array_equal(group.plan(0, 1)[f].cpu().numpy(), getattr(init, f))
    group.update_placement(0, d_ids32)
    group.update_placement(1, d_ids64)
    group.update_placement(2, d_maps)
    torch.cuda.synchronize()
    group.check_status()
    for layer in range(3):
        assert_plans_equal(group, layer, plans)
    for r in range(cfg.ep):
        assert np.array_equal(group.buffer(r, capi.BUF_GLOBAL_LOADS).cpu().numpy(), lpr.sum(0))
        assert np.array_equal(group.buffer(r, capi.BUF_LOADS_PER_RANK).cpu().numpy(), lpr)
        # per-slot loads written by the plan kernel = the reference's profiling formula over the plan
        expected = O.physical_loads_from_plan(plans[r], group.P)
        assert int(expected.sum()) == int(lpr.sum())
        for layer in range(3):
            assert np.array_equal(group.buffer(r, capi.BUF_PHYSICAL_LOADS)[layer].cpu().numpy(), expected)
    group.destroy()


def test_update_placement_repeated_and_ragged(native_lib, cuda_device):
    """Many calls in a row (both parities of the exchange buffers), different token counts per
    rank, an empty rank, and a different routing per call."""
    cfg = small_cfg(tokens_per_rank=1500)
    group = make_group(cfg, num_layers=4)
    for call in range(7):
        tokens = [0 if (r == 3 and call % 2) else 200 + 173 * ((r + call) % 5) for r in range(cfg.ep)]
        ids = [W.routing_ids(cfg, r, microbatch=call, tokens=tokens[r]) for r in range(cfg.ep)]
        lpr = np.stack([np.bincount(x.reshape(-1), minlength=cfg.num_experts) for x in ids]).astype(np.int32)
        group.update_placement(call % 4, [torch.from_numpy(x).to(cuda_device) for x in ids])
        torch.cuda.synchronize()
        group.check_status()
        assert_plans_equal(group, call % 4, oracle_plans(lpr, cfg))
    group.destroy()


def test_reroute_through_manager(native_lib, cuda_device):
    cfg = W.CONFIGS["cfg1_plan_reroute"]
    group = make_group(cfg)
    ids = [W.routing_ids(cfg, r) for r in range(cfg.ep)]
    lpr = np.stack([np.bincount(x.reshape(-1), minlength=cfg.num_experts) for x in ids]).astype(np.int32)
    plans = oracle_plans(lpr, cfg)
    d_ids = [torch.from_numpy(x).to(cuda_device) for x in ids]
    group.update_placement(1, d_ids)
    # sparse, on another stream than the plan: the manager must order it after the plan
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        phys = group.reroute_sparse(1, d_ids)
    side.synchronize()
    maps = [W.ids_to_map(x, cfg.num_experts) for x in ids]
    probs = [W.probs_for_map(m, 100 + r) for r, m in enumerate(maps)]
    d_maps = [torch.from_numpy(m).to(cuda_device) for m in maps]
    d_probs = [torch.from_numpy(p).to(cuda_device) for p in probs]
    out_probs, out_maps = group.reroute_dense(1, d_maps, d_probs)
    grads = [torch.randn(m.shape[0], group.P, device=cuda_device) for m in maps]
    back = group.reroute_dense_backward(1, grads, d_maps, out_maps)
    torch.cuda.synchronize()
    group.check_status()
    for r in range(cfg.ep):
        assert np.array_equal(phys[r].cpu().numpy(), O.sparse_reroute(ids[r], plans[r], True))
        exp_probs, exp_map = O.dense_reroute_forward(maps[r], probs[r], plans[r], group.P, True)
        assert np.array_equal(out_maps[r].cpu().numpy(), exp_map)
        assert np.array_equal(out_probs[r].cpu().numpy().view(np.uint32), exp_probs.view(np.uint32))
        exp_back = O.dense_reroute_backward(grads[r].cpu().numpy(), maps[r], exp_map, plans[r])
        assert np.array_equal(back[r].cpu().numpy().view(np.uint32), exp_back.view(np.uint32))
    # post-balance rank loads: no rank above the solver's threshold bound by more than rounding
    counts = sum(torch.bincount(p.flatten().long(), minlength=group.P) for p in phys)
    rank_loads = counts.view(cfg.ep, -1).sum(1).float()
    assert float(rank_loads.max() / rank_loads.mean()) < 1.03
    group.destroy()


def _master_tensors(cfg, group, nbytes_per_shard, misalign=0):
    """Random master shards per rank: list over shard of list over rank of list over master."""
    shards = []
    gen = torch.Generator(device="cpu").manual_seed(5)
    for s, nbytes in enumerate(nbytes_per_shard):
        per_rank = []
        for r in range(cfg.ep):
            per_rank.append([
                torch.randint(0, 256, (nbytes + misalign,), dtype=torch.uint8, generator=gen).to(group.device)[misalign:]
                for _ in range(cfg.masters)])
        shards.append(per_rank)
    return shards


@pytest.mark.parametrize("fc1,fc2,s1,s2,elem,misalign", [
    (2 * 96 * 128, 96 * 128, 0, 0, 2, 0),          # bf16, no scales
    (2 * 128 * 160, 128 * 160, 320, 160, 1, 0),     # fp8 + scales, all multiples of 16
    (40000, 20000 - 16, 313, 157, 1, 0),            # scale bytes not multiples of 16 (tail bytes)
    (2 * 96 * 128, 96 * 128, 100, 50, 1, 8),        # masters not 16-byte aligned: plain copy path
    (33 * 1024 * 16, 16, 0, 0, 1, 0),               # several tiles per shard and a one-vector shard
])
@pytest.mark.parametrize("plan_mode", [0, 2, 1])  # direct; every expert with >= 2 replicas relayed; adaptive (>= 3 here)
def test_weight_sync_bitwise(native_lib, cuda_device, fc1, fc2, s1, s2, elem, misalign, plan_mode):
    # cfg 3's routing of microbatch 1 gives experts with one, two and three replicas
    cfg = small_cfg("cfg3_qwen3_235b_fp8")
    group = make_group(cfg, fc1=fc1, fc2=fc2, elem=elem, s1=s1, s2=s2, relay_min_replicas=3)
    capi.check(group.lib.uep_set_weight_sync_plan_mode(group.handle, plan_mode))
    ids = [torch.from_numpy(W.routing_ids(cfg, r, microbatch=1)).to(cuda_device) for r in range(cfg.ep)]
    group.update_placement(0, ids)
    nbytes = [fc1 * elem, fc2 * elem] + ([s1, s2] if s1 + s2 else [])
    shards = _master_tensors(cfg, group, nbytes, misalign)
    tables = [group.pointer_tables(sh) for sh in shards] + [None] * (4 - len(shards))
    for rep in range(3):  # several epochs; the slots are re-randomised so that every epoch has to deliver
        w_before, s_before = [], []
        for r in range(cfg.ep):
            w = group.buffer(r, capi.BUF_REPLICA_WEIGHT)
            w.random_(0, 256)
            w_before.append(w.clone())
            sbuf = group.buffer(r, capi.BUF_REPLICA_SCALE)
            if sbuf.numel():
                sbuf.random_(0, 256)
            s_before.append(sbuf.clone())
        ev = group.weight_sync(0, *tables, async_finish=bool(rep))
        if ev is not None:
            group.wait_event(ev)
        torch.cuda.synchronize()
        group.check_status()
    plan = O.Plan(**{f: group.plan(0, 0)[f].cpu().numpy() for f in PLAN_FIELDS})
    assert int((plan.lcnts > 1).sum()) > 0, "the case must replicate something"
    if plan_mode:
        assert int((plan.lcnts > 3).sum()) > 0 and int((plan.lcnts == 3).sum()) > 0 and int((plan.lcnts == 2).sum()) > 0
    for r in range(cfg.ep):
        exp_w = w_before[r].cpu().numpy()
        offs = [0, fc1 * elem]
        for s in range(2):
            masters = [shards[s][q][m].cpu().numpy() for q in range(cfg.ep) for m in range(cfg.masters)]
            exp_w = O.weight_sync_expected(r, cfg.masters, cfg.redundant, plan, masters, exp_w, offs[s], nbytes[s])
        assert np.array_equal(group.buffer(r, capi.BUF_REPLICA_WEIGHT).cpu().numpy(), exp_w), f"rank {r} weights"
        if s1 + s2:
            exp_s = s_before[r].cpu().numpy()
            soffs = [0, (s1 + 15) // 16 * 16]
            for s in range(2):
                masters = [shards[2 + s][q][m].cpu().numpy() for q in range(cfg.ep) for m in range(cfg.masters)]
                exp_s = O.weight_sync_expected(r, cfg.masters, cfg.redundant, plan, masters, exp_s, soffs[s], nbytes[2 + s])
            assert np.array_equal(group.buffer(r, capi.BUF_REPLICA_SCALE).cpu().numpy(), exp_s), f"rank {r} scales"
            # the strided fc1 / fc2 scale views alias the full buffer
            full = group.buffer(r, capi.BUF_REPLICA_SCALE)
            assert torch.equal(group.buffer(r, capi.BUF_REPLICA_FC1_SCALE), full[:, :s1])
            assert torch.equal(group.buffer(r, capi.BUF_REPLICA_FC2_SCALE), full[:, soffs[1]:soffs[1] + s2])
        full = group.buffer(r, capi.BUF_REPLICA_WEIGHT)
        assert torch.equal(group.buffer(r, capi.BUF_REPLICA_FC1_WEIGHT), full[:, :fc1 * elem])
        assert torch.equal(group.buffer(r, capi.BUF_REPLICA_FC2_WEIGHT), full[:, fc1 * elem:])
    group.destroy()


@pytest.mark.skipif(not uep_ref.available(), reason="oracle/_ref/libuep_ref.so not built")
def test_weight_sync_matches_reference_kernels(native_lib, cuda_device):
    """Same plan, same masters: the reference's task build + copy kernel fill replica buffers
    with exactly the bytes ours does."""
    cfg = W.CONFIGS["cfg1_plan_reroute"]
    fc1, fc2, s1, s2, elem = 2 * 128 * 160, 128 * 160, 320, 160, 1
    group = make_group(cfg, fc1=fc1, fc2=fc2, elem=elem, s1=s1, s2=s2)
    ids = [torch.from_numpy(W.routing_ids(cfg, r)).to(cuda_device) for r in range(cfg.ep)]
    group.update_placement(0, ids)
    shards = _master_tensors(cfg, group, [fc1, fc2, s1, s2])
    tables = [group.pointer_tables(sh) for sh in shards]
    group.weight_sync(0, *tables)
    torch.cuda.synchronize()
    ours_w = [group.buffer(r, capi.BUF_REPLICA_WEIGHT).clone() for r in range(cfg.ep)]
    ours_s = [group.buffer(r, capi.BUF_REPLICA_SCALE).clone() for r in range(cfg.ep)]
    ref_w = [torch.zeros_like(t) for t in ours_w]
    ref_s = [torch.zeros_like(t) for t in ours_s]
    stream = torch.cuda.current_stream().cuda_stream
    spaces = []
    for r in range(cfg.ep):
        ws = uep_ref.Workspace(r, cfg.ep, cfg.masters, cfg.redundant, fc1, fc2, elem, 1, s1, s2, cfg.ep,
                               [t.data_ptr() for t in ref_w], [t.data_ptr() for t in ref_s], None)
        p = group.plan(r, 0)
        ws.weight_sync(p["p2l"], p["l2p"], p["lcnts"], tables[0][r], tables[1][r], tables[2][r], tables[3][r],
                       ref_w[r], ref_s[r], stream)
        spaces.append(ws)
    torch.cuda.synchronize()
    plan = group.plan(0, 0)
    used = (plan["p2l"].view(cfg.ep, -1)[:, cfg.masters:] >= 0).cpu()
    for r in range(cfg.ep):
        for s in range(cfg.redundant):
            if used[r, s]:
                assert torch.equal(ours_w[r][s], ref_w[r][s]) and torch.equal(ours_s[r][s], ref_s[r][s])
    for ws in spaces:
        ws.close()
    group.destroy()


@pytest.mark.parametrize("fc1,fc2,misalign", [(2 * 96 * 128, 96 * 128, 0), (5000, 2048 * 3 + 4, 0), (1001, 37, 0),
                                             (4096, 4096, 1)])
def test_grad_reduce_bitwise(native_lib, cuda_device, fc1, fc2, misalign):
    cfg = W.CONFIGS["cfg1_plan_reroute"]
    # 16-byte weight elements make any numel a legal shard size; only the fp32 gradients matter here
    group = make_group(cfg, fc1=fc1, fc2=fc2, elem=16)
    ids = [torch.from_numpy(W.routing_ids(cfg, r)).to(cuda_device) for r in range(cfg.ep)]
    group.update_placement(1, ids)
    torch.cuda.synchronize()
    plan = O.Plan(**{f: group.plan(0, 1)[f].cpu().numpy() for f in PLAN_FIELDS})
    N, M, R, Lp = cfg.ep, cfg.masters, cfg.redundant, cfg.masters + cfg.redundant
    gen = torch.Generator(device="cpu").manual_seed(9)

    def rnd(n, std):  # values that do NOT add exactly, so the order matters
        return (torch.randn(n + misalign, generator=gen) * std).to(cuda_device)[misalign:]

    fc1_g = [[rnd(fc1, 1e-4) for _ in range(M)] for _ in range(N)]
    fc2_g = [[rnd(fc2, 1e-4) for _ in range(M)] for _ in range(N)]
    replica = [group.buffer(r, capi.BUF_REPLICA_GRAD) for r in range(N)]
    for r in range(N):
        replica[r].copy_(torch.randn(replica[r].shape, generator=gen) * 1e-4)
    rep_before = [t.clone() for t in replica]
    exp_fc1 = [[t.cpu().numpy().copy() for t in row] for row in fc1_g]
    exp_fc2 = [[t.cpu().numpy().copy() for t in row] for row in fc2_g]
    exp_rep = [t.cpu().numpy().copy() for t in rep_before]
    for l in range(N * M):
        reps1, reps2 = [], []
        for j in range(1, plan.lcnts[l]):
            phys = plan.l2p[l, j]
            rr, slot = phys // Lp, phys % Lp - M
            reps1.append(exp_rep[rr][slot, :fc1])
            reps2.append(exp_rep[rr][slot, fc1:])
        if reps1:
            # views into exp_rep rows are not contiguous as a whole, but each slice is
            r1 = [np.ascontiguousarray(x) for x in reps1]
            r2 = [np.ascontiguousarray(x) for x in reps2]
            O.grad_reduce_shard(exp_fc1[l // M][l % M], r1)
            O.grad_reduce_shard(exp_fc2[l // M][l % M], r2)
            for x, y in zip(reps1, r1):
                x[...] = y
            for x, y in zip(reps2, r2):
                x[...] = y
    t1 = group.pointer_tables(fc1_g)
    t2 = group.pointer_tables(fc2_g)
    ev = group.grad_reduce(1, t1, t2, async_finish=True)
    group.wait_event(ev)
    torch.cuda.synchronize()
    group.check_status()
    for r in range(N):
        for m_ in range(M):
            assert np.array_equal(fc1_g[r][m_].cpu().numpy().view(np.uint32), exp_fc1[r][m_].view(np.uint32)), (r, m_)
            assert np.array_equal(fc2_g[r][m_].cpu().numpy().view(np.uint32), exp_fc2[r][m_].view(np.uint32)), (r, m_)
        assert np.array_equal(replica[r].cpu().numpy().view(np.uint32), exp_rep[r].view(np.uint32)), f"replica {r}"
        full = group.buffer(r, capi.BUF_REPLICA_GRAD)
        assert torch.equal(group.buffer(r, capi.BUF_REPLICA_FC1_GRAD), full[:, :fc1])
        assert torch.equal(group.buffer(r, capi.BUF_REPLICA_FC2_GRAD), full[:, fc1:])
    used = (plan.p2l.reshape(N, Lp)[:, M:] >= 0)
    assert used.any()
    for r in range(N):
        for s in range(R):
            if used[r, s]:
                assert not replica[r][s].any(), "consumed replica regions must be zero"
            else:
                assert torch.equal(replica[r][s], rep_before[r][s]), "unused slots must be untouched"
    group.destroy()


@pytest.mark.skipif(not uep_ref.available(), reason="oracle/_ref/libuep_ref.so not built")
def test_grad_reduce_matches_reference_kernel(native_lib, cuda_device):
    cfg = W.CONFIGS["cfg1_plan_reroute"]
    fc1, fc2 = 2 * 96 * 128, 96 * 128 + 8
    group = make_group(cfg, fc1=fc1, fc2=fc2)
    ids = [torch.from_numpy(W.routing_ids(cfg, r)).to(cuda_device) for r in range(cfg.ep)]
    group.update_placement(0, ids)
    N, M = cfg.ep, cfg.masters
    fc1_g = [[torch.randn(fc1, device=cuda_device) * 1e-4 for _ in range(M)] for _ in range(N)]
    fc2_g = [[torch.randn(fc2, device=cuda_device) * 1e-4 for _ in range(M)] for _ in range(N)]
    replica = [group.buffer(r, capi.BUF_REPLICA_GRAD) for r in range(N)]
    for t in replica:
        t.normal_(0, 1e-4)
    ref_fc1 = [[t.clone() for t in row] for row in fc1_g]
    ref_fc2 = [[t.clone() for t in row] for row in fc2_g]
    ref_rep = [t.clone() for t in replica]
    group.grad_reduce(0, group.pointer_tables(fc1_g), group.pointer_tables(fc2_g))
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    rt1, rt2 = group.pointer_tables(ref_fc1), group.pointer_tables(ref_fc2)
    spaces = []
    for r in range(N):
        ws = uep_ref.Workspace(r, N, M, cfg.redundant, fc1, fc2, 2, 1, 0, 0, N, None, None,
                               [t.data_ptr() for t in ref_rep])
        p = group.plan(r, 0)
        ws.grad_reduce(p["p2l"], p["l2p"], p["lcnts"], rt1[r], rt2[r], 42, True, stream)
        spaces.append(ws)
    torch.cuda.synchronize()
    for r in range(N):
        for m_ in range(M):
            assert torch.equal(fc1_g[r][m_], ref_fc1[r][m_]) and torch.equal(fc2_g[r][m_], ref_fc2[r][m_])
        assert torch.equal(replica[r], ref_rep[r])
    for ws in spaces:
        ws.close()
    group.destroy()


def test_wait_timeout_is_reported_not_fatal(native_lib, cuda_device):
    """Failure detection without a device fault: one hosted rank withholds its flags (a host-side
    switch); the ranks that wait for it give up after the time limit, report a status code, the
    context stays usable, and the next call succeeds."""
    cfg = W.CONFIGS["cfg1_plan_reroute"]
    group = make_group(cfg, fc1=4096, fc2=2048, wait_timeout_ms=150)
    ids = [torch.from_numpy(W.routing_ids(cfg, r)).to(cuda_device) for r in range(cfg.ep)]
    lpr = np.stack([np.bincount(x.cpu().numpy().reshape(-1), minlength=cfg.num_experts) for x in ids]).astype(np.int32)
    group.update_placement(0, ids)
    torch.cuda.synchronize()
    group.check_status()
    capi.check(group.lib.uep_debug_withhold_rank(group.handle, 5))
    group.update_placement(1, ids)
    torch.cuda.synchronize()
    for r in range(cfg.ep):
        assert group.status(r) == (capi_code("gather"), 5)
    with pytest.raises(capi.UepError):
        group.check_status()
    # layer 1 still holds the masters-only plan
    init = O.init_master_placement(cfg.ep, cfg.masters, cfg.redundant)
    assert np.array_equal(group.plan(2, 1)["lcnts"].cpu().numpy(), init.lcnts)
    # weight_sync with the withheld rank: its receivers time out
    shards = _master_tensors(cfg, group, [4096 * 2, 2048 * 2])
    tables = [group.pointer_tables(sh) for sh in shards]
    capi.check(group.lib.uep_clear_status(group.handle))
    plan = O.solve_placement(lpr, cfg.masters, cfg.redundant, cfg.ep, 0)
    Lp = cfg.masters + cfg.redundant
    senders = {int(plan.l2p[l, 0]) // Lp for l in range(cfg.num_experts) if plan.lcnts[l] > 1}
    victim = sorted(senders)[0]
    capi.check(group.lib.uep_debug_withhold_rank(group.handle, victim))
    group.weight_sync(0, tables[0], tables[1])
    torch.cuda.synchronize()
    codes = [group.status(r) for r in range(cfg.ep)]
    assert any(c == (capi_code("sync"), victim) for c in codes) and all(c[0] in (0, capi_code("sync")) for c in codes)
    # recovery
    capi.check(group.lib.uep_debug_withhold_rank(group.handle, -1))
    capi.check(group.lib.uep_clear_status(group.handle))
    group.update_placement(1, ids)
    group.weight_sync(1, tables[0], tables[1])
    torch.cuda.synchronize()
    group.check_status()
    assert_plans_equal(group, 1, oracle_plans(lpr, cfg))
    group.destroy()


def capi_code(kind):
    return {"gather": 1, "sync": 2}[kind]


def test_manager_argument_errors(native_lib, cuda_device):
    lib = capi.lib()
    h = C.c_void_p()
    bad = sim.make_config(8, 8, 2, sim=True)
    bad.grad_element_bytes = 2
    assert lib.uep_manager_create(C.byref(bad), C.byref(h)) == -1 and b"fp32 gradients" in lib.uep_last_error()
    bad = sim.make_config(8, 8, 2, sim=True, grad_reduce_num_sms=41)
    assert lib.uep_manager_create(C.byref(bad), C.byref(h)) == -1 and b"even" in lib.uep_last_error()
    bad = sim.make_config(8, 8, 2, sim=True, fc1_numel=7, weight_elem_bytes=2)
    assert lib.uep_manager_create(C.byref(bad), C.byref(h)) == -1 and b"multiples of 16" in lib.uep_last_error()
    bad = sim.make_config(8, 8, 2, sim=True)
    bad.nvl_ranks = 4  # a group that spans two NVLink domains: the load exchange needs peer memory
    assert lib.uep_manager_create(C.byref(bad), C.byref(h)) == -4
    group = sim.SimGroup(sim.make_config(4, 2, 1, 2, sim=True, is_train=False))
    p, nd = C.c_void_p(), C.c_int()
    shape, stride = (C.c_int64 * 3)(), (C.c_int64 * 3)()
    assert lib.uep_manager_buffer(group.handle, 0, capi.BUF_REPLICA_GRAD, C.byref(p), C.byref(nd), shape, stride) == -3
    assert b"inference mode" in lib.uep_last_error()
    ids = [torch.zeros(4, 2, dtype=torch.int32, device=cuda_device) for _ in range(4)]
    with pytest.raises(capi.UepError):
        group.update_placement(5, ids)
    group.destroy()


def test_peer_buffer_addresses_and_scratch_presizing(native_lib, cuda_device):
    """uep_manager_peer_buffer hands out the address under which a hosted rank reaches a peer's replica buffers
    (on one device: the peer's own buffer); the link probe refuses a simulated group; with reroute_max_tokens the
    reroute scratch has its size from the start."""
    lib = capi.lib()
    mcfg = sim.make_config(4, 2, 2, 1, fc1_numel=1024, fc2_numel=512, weight_elem_bytes=2, fc1_scale_numel=16,
                           fc2_scale_numel=8, sim=True, is_train=True)
    mcfg.reroute_max_tokens = 4096
    mcfg.reroute_max_topk = 4
    group = sim.SimGroup(mcfg)
    for buf in (capi.BUF_REPLICA_WEIGHT, capi.BUF_REPLICA_SCALE, capi.BUF_REPLICA_GRAD):
        for local in range(4):
            for peer in range(4):
                out = C.c_void_p()
                capi.check(lib.uep_manager_peer_buffer(group.handle, local, peer, buf, C.byref(out)))
                assert out.value == group.buffer(peer, buf).data_ptr()
    out = C.c_void_p()
    assert lib.uep_manager_peer_buffer(group.handle, 0, 9, capi.BUF_REPLICA_WEIGHT, C.byref(out)) == -1
    assert lib.uep_manager_peer_buffer(group.handle, 0, 1, capi.BUF_P2L, C.byref(out)) == -1
    ms = C.c_float()
    assert lib.uep_debug_link_probe(group.handle, 1, 1024, 1, 0, C.byref(ms)) == -3  # needs real peers
    # reroutes up to the stated bound work right away (and larger ones still grow the buffer)
    ids = [torch.randint(0, 8, (4096, 4), dtype=torch.int32, device=cuda_device) for _ in range(4)]
    group.update_placement(0, ids)
    phys = group.reroute_sparse(0, ids)
    torch.cuda.synchronize()
    group.check_status()
    assert all(int(p.min()) >= 0 and int(p.max()) < 16 for p in phys)
    group.destroy()


def test_legacy_placement_mode(native_lib, cuda_device):
    """legacy_placement=True through the manager: the counts-only greedy plan from the gathered loads, round-robin
    reroute (dense and sparse) over an expert's instances, weights synced to every instance."""
    cfg = W.CONFIGS["cfg1_plan_reroute"]
    fc1, fc2 = 2 * 64 * 128, 64 * 128
    mcfg = sim.make_config(cfg.ep, cfg.masters, cfg.redundant, 2, fc1_numel=fc1, fc2_numel=fc2, weight_elem_bytes=1,
                           is_train=False, sim=True)
    mcfg.legacy_placement = 1
    group = sim.SimGroup(mcfg)
    ids = [W.routing_ids(cfg, r) for r in range(cfg.ep)]
    lpr = np.stack([np.bincount(x.reshape(-1), minlength=cfg.num_experts) for x in ids]).astype(np.int32)
    plan = O.legacy_solve_placement(lpr.sum(0), cfg.ep, cfg.masters, cfg.redundant, cfg.ep, 1.0)
    assert int((plan.lcnts > 1).sum()) > 0
    d_ids = [torch.from_numpy(x).to(cuda_device) for x in ids]
    group.update_placement(1, d_ids)
    phys = group.reroute_sparse(1, d_ids)
    maps = [W.ids_to_map(x, cfg.num_experts) for x in ids]
    probs = [W.probs_for_map(m, 7 + r) for r, m in enumerate(maps)]
    out_probs, out_maps = group.reroute_dense(1, [torch.from_numpy(m).to(cuda_device) for m in maps],
                                              [torch.from_numpy(p).to(cuda_device) for p in probs])
    shards = _master_tensors(cfg, group, [fc1, fc2])
    tables = [group.pointer_tables(sh) for sh in shards]
    for r in range(cfg.ep):
        group.buffer(r, capi.BUF_REPLICA_WEIGHT).fill_(0xEE)
    group.weight_sync(1, tables[0], tables[1])
    torch.cuda.synchronize()
    group.check_status()
    D = cfg.ep
    for r in range(cfg.ep):
        got = group.plan(r, 1)
        for f in ("p2l", "l2p", "lcnts"):
            assert np.array_equal(got[f].cpu().numpy(), getattr(plan, f)), f"rank {r} field {f}"
        assert not got["quota"].any() and not got["rank_quota_prefix"].any()
        # round-robin: the n-th token (row-major) of expert e on this rank goes to instance n mod C
        flat = ids[r].reshape(-1)
        expect = np.empty_like(flat)
        seen = np.zeros(cfg.num_experts, np.int64)
        for i, e in enumerate(flat):
            expect[i] = plan.l2p.reshape(-1, D)[e, seen[e] % plan.lcnts[e]]
            seen[e] += 1
        assert np.array_equal(phys[r].cpu().numpy().reshape(-1), expect), f"rank {r} sparse round-robin"
        exp_map = np.zeros((ids[r].shape[0], group.P), bool)
        exp_map[np.repeat(np.arange(ids[r].shape[0]), ids[r].shape[1]), expect] = True
        assert np.array_equal(out_maps[r].cpu().numpy(), exp_map), f"rank {r} dense round-robin"
        # every instance holds its expert's bytes
        rep = group.buffer(r, capi.BUF_REPLICA_WEIGHT).cpu()
        Lp = cfg.masters + cfg.redundant
        for slot in range(cfg.redundant):
            l = int(plan.p2l[r * Lp + cfg.masters + slot])
            if l >= 0:
                src = torch.cat([shards[0][l // cfg.masters][l % cfg.masters], shards[1][l // cfg.masters][l % cfg.masters]]).cpu()
                assert torch.equal(rep[slot, :fc1 + fc2], src), f"rank {r} slot {slot}"
            else:
                assert bool((rep[slot] == 0xEE).all())
    group.destroy()
