"""Multi-GPU end-to-end check of the drop-in Manager (one process per GPU, NCCL for bootstrap
only). Launch with torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 tests/dist_worker.py

Mirrors what the reference's distributed test asserts (tests/test_e2e.py of the reference): gathered
loads equal an all-reduce, every token keeps top-k physical experts, weight_sync is bitwise with
untouched unused slots, the Wgrad reduce is bitwise and zeroes the used replica slots. On top of
that every rank's plan and routing are compared bit for bit with the CPU oracle, and the gradients
are random (not exactly summable), so the accumulation order is pinned too.
"""

import os
import shutil
import tempfile
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import uep_oracle as O  # noqa: E402
from ultra_ep_b200 import Manager  # noqa: E402
from ultra_ep_b200 import workloads as W  # noqa: E402

FIELDS = ("p2l", "l2p", "lcnts", "quota", "quota_prefix", "rank_quota_prefix")


def seeded(key, n, dtype, dev, std=1.0):
    g = torch.Generator(device="cpu").manual_seed(int(key))
    if dtype == torch.uint8:
        return torch.randint(0, 256, (n,), dtype=torch.uint8, generator=g).to(dev)
    return (torch.randn(n, generator=g) * std).to(dtype).to(dev)


def main():
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    base = W.CONFIGS[os.environ.get("UEP_TEST_CONFIG", "cfg1_plan_reroute")]
    cfg = base.with_ep(world)
    N, M, R = world, cfg.masters, cfg.redundant
    L, Lp, P = cfg.num_experts, M + R, world * (M + R)
    hidden, ffn = 256, 96
    fc1, fc2 = 2 * hidden * ffn, hidden * ffn
    s1, s2 = fc1 // 128, fc2 // 128 + 3  # fc2 scale bytes not a multiple of 16
    layers = 3
    # expert-load trace: switched on through the reference's environment variables, checked at the end
    trace_dir = tempfile.mkdtemp(prefix="uep_trace_") if rank == 0 else ""
    if rank == 0:
        os.environ["ULTRA_EP_LOAD_PROFILING"] = "1"
        os.environ["ULTRA_EP_LOAD_PROFILE_DIR"] = trace_dir
    trace_expect = []  # (virtual layer, global logical loads, physical loads) in call order
    mgr = Manager(dist.group.WORLD, layers, M, R, fc1, fc2, is_train=True, explicitly_destroy=True, max_microbatches=2,
                  weight_data_dtype=torch.uint8, weight_scale_dtype=torch.uint8, expert_fc1_weight_scale_numel=s1,
                  expert_fc2_weight_scale_numel=s2)
    assert mgr.nvl_domain_size == world

    # masters: bytes seeded by global physical id, so every rank can rebuild any master locally
    def master(shard, phys, n):
        return seeded(1000003 * shard + phys, n, torch.uint8, dev)

    sizes = [fc1, fc2, s1, s2]
    mine = [[master(s, rank * Lp + m, sizes[s]) for m in range(M)] for s in range(4)]
    fc1_g = [seeded(7000003 + rank * Lp + m, fc1, torch.float32, dev, 1e-4) for m in range(M)]
    fc2_g = [seeded(9000011 + rank * Lp + m, fc2, torch.float32, dev, 1e-4) for m in range(M)]
    for real_layer in range(1, layers + 1):
        mgr.construct_local_master_ptr_pool(real_layer, mine[0], mine[1], fc1_g, fc2_g, mine[2], mine[3])

    for it in range(6):
        if it == 3:  # the second half runs with every multi-replica expert relayed (scatter + forward)
            mgr.set_weight_sync_plan_mode("force_relay")
        real_layer = 1 + it % layers
        vid = mgr.allocate_microbatch_slot(real_layer)
        ids_all = [W.routing_ids(cfg, r, microbatch=it) for r in range(N)]
        lpr = np.stack([np.bincount(x.reshape(-1), minlength=L) for x in ids_all]).astype(np.int32)
        plan = O.solve_placement(lpr, M, R, N, rank)
        ids = ids_all[rank]
        rmap_np = W.ids_to_map(ids, L)
        probs_np = W.probs_for_map(rmap_np, 100 * it + rank)
        rmap = torch.from_numpy(rmap_np).to(dev)
        probs = torch.from_numpy(probs_np).to(dev).requires_grad_(True)

        # randomise the replica slots so that "untouched" is observable
        mgr.local_replica_weight_buffer.random_(0, 256)
        mgr.local_replica_weight_scale_buffer_raw.random_(0, 256)
        before_w = mgr.local_replica_weight_buffer.clone()
        before_s = mgr.local_replica_weight_scale_buffer_raw.clone()
        torch.cuda.synchronize()
        dist.barrier()

        if it % 2 == 0:
            mgr.update_placement(vid, rmap, verify_reduced_loads=True)
        else:
            mgr.update_placement_sparse(vid, torch.from_numpy(ids).to(dev).long())
        ev = mgr.weight_sync(vid, async_finish=True)
        exp_probs_t, exp_map_t = mgr.reroute(vid, probs, rmap)
        ev.current_stream_wait()
        torch.cuda.synchronize()
        mgr.check_status()
        dist.barrier()

        if rank == 0:
            trace_expect.append((vid, mgr.runtime.get_global_logical_expert_loads_tensor().cpu().numpy().copy(),
                                 mgr._profile_physical_loads_from_quota(vid).cpu().numpy().copy()))
        got = {"p2l": mgr.physical_to_logical_map[vid], "l2p": mgr.logical_to_physical_map[vid],
               "lcnts": mgr.logical_replica_counts[vid], "quota": mgr.logical_instance_quota[vid],
               "quota_prefix": mgr.logical_instance_quota_prefix[vid], "rank_quota_prefix": mgr.rank_quota_prefix[vid]}
        for f in FIELDS:
            assert np.array_equal(got[f].cpu().numpy(), getattr(plan, f)), f"iter {it} rank {rank}: plan field {f}"
        o_probs, o_map = O.dense_reroute_forward(rmap_np, probs_np, plan, P, True)
        assert np.array_equal(exp_map_t.cpu().numpy(), o_map), f"iter {it} rank {rank}: expanded map"
        assert np.array_equal(exp_probs_t.detach().cpu().numpy().view(np.uint32), o_probs.view(np.uint32))
        assert bool((exp_map_t.sum(1) == cfg.topk).all())
        upstream = torch.randn_like(exp_probs_t)
        exp_probs_t.backward(upstream)
        o_back = O.dense_reroute_backward(upstream.cpu().numpy(), rmap_np, o_map, plan)
        assert np.array_equal(probs.grad.cpu().numpy().view(np.uint32), o_back.view(np.uint32)), "reroute backward"
        sparse = torch.from_numpy(ids).to(dev).long()
        mgr.reroute_sparse(vid, sparse)
        assert np.array_equal(sparse.cpu().numpy(), O.sparse_reroute(ids.astype(np.int64), plan, True)), "sparse reroute"

        # weight_sync: used slots hold the master's bytes, unused slots are untouched
        w_now = mgr.local_replica_weight_buffer
        s_now = mgr.local_replica_weight_scale_buffer_raw
        s2_off = (s1 + 15) // 16 * 16
        for slot in range(R):
            l = int(plan.p2l[rank * Lp + M + slot])
            if l < 0:
                assert torch.equal(w_now[slot], before_w[slot]) and torch.equal(s_now[slot], before_s[slot])
                continue
            mphys = int(plan.l2p[l, 0])
            assert torch.equal(w_now[slot, :fc1], master(0, mphys, fc1)), f"iter {it} rank {rank} slot {slot}: fc1"
            assert torch.equal(w_now[slot, fc1:], master(1, mphys, fc2)), "fc2"
            assert torch.equal(s_now[slot, :s1], master(2, mphys, s1)), "fc1 scales"
            assert torch.equal(s_now[slot, s2_off:s2_off + s2], master(3, mphys, s2)), "fc2 scales"
            assert torch.equal(mgr.local_replica_fc1_weight_scale_buffer[slot], master(2, mphys, s1))
            assert torch.equal(mgr.local_replica_fc2_weight_scale_buffer[slot], master(3, mphys, s2))

        # backward: replicas hold a gradient seeded by (iteration, physical id)
        rep = mgr.local_replica_grad_buffer
        for slot in range(R):
            phys = rank * Lp + M + slot
            rep[slot].copy_(seeded(31 * it + 500000 + phys, fc1 + fc2, torch.float32, dev, 1e-4))
        rep_before = rep.clone()
        base1 = [g.clone() for g in fc1_g]
        base2 = [g.clone() for g in fc2_g]
        torch.cuda.synchronize()
        dist.barrier()
        mgr.weight_sync(vid, async_finish=False)  # the backward re-pushes the layer's weights first
        gev = mgr.grad_reduce(vid, async_finish=True)
        gev.current_stream_wait()
        torch.cuda.synchronize()
        mgr.check_status()
        dist.barrier()
        for m in range(M):
            l = rank * M + m
            e1, e2 = base1[m].cpu().numpy().copy(), base2[m].cpu().numpy().copy()
            r1, r2 = [], []
            for j in range(1, int(plan.lcnts[l])):
                phys = int(plan.l2p[l, j])
                g = seeded(31 * it + 500000 + phys, fc1 + fc2, torch.float32, "cpu", 1e-4).numpy()
                r1.append(np.ascontiguousarray(g[:fc1]))
                r2.append(np.ascontiguousarray(g[fc1:]))
            if r1:
                O.grad_reduce_shard(e1, r1)
                O.grad_reduce_shard(e2, r2)
            assert np.array_equal(fc1_g[m].cpu().numpy().view(np.uint32), e1.view(np.uint32)), f"iter {it}: fc1 grad {m}"
            assert np.array_equal(fc2_g[m].cpu().numpy().view(np.uint32), e2.view(np.uint32)), f"iter {it}: fc2 grad {m}"
        for slot in range(R):
            if int(plan.p2l[rank * Lp + M + slot]) >= 0:
                assert not rep[slot].any(), "used replica gradient slot must be zeroed by its master's rank"
            else:
                assert torch.equal(rep[slot], rep_before[slot]), "unused replica gradient slot must be untouched"
        assert torch.equal(mgr.local_replica_fc1_grad_buffer, rep[:, :fc1])
        assert torch.equal(mgr.local_replica_fc2_grad_buffer, rep[:, fc1:])

    # a short timing of the forward step, maximum over ranks
    rmap = torch.from_numpy(W.ids_to_map(W.routing_ids(cfg, rank), L)).to(dev)
    probs = torch.rand(rmap.shape, device=dev)
    times = []
    for it in range(12):
        vid = mgr.allocate_microbatch_slot(1)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        mgr.update_placement(vid, rmap)
        ev = mgr.weight_sync(vid, async_finish=True)
        mgr.reroute(vid, probs, rmap)
        ev.current_stream_wait()
        e1.record()
        torch.cuda.synchronize()
        if it >= 2:
            times.append(e0.elapsed_time(e1))
    t = torch.tensor([sum(times) / len(times)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    mgr.check_status()
    if rank == 0:
        print(f"[dist_worker] EP{world}: all checks passed; forward step {t.item() * 1e3:.1f} us (max over ranks, small layer)",
              flush=True)
    mgr.destroy()
    if rank == 0:  # the trace holds every update_placement of this run; the checked ones come first
        import glob
        import json

        manifest = json.load(open(glob.glob(os.path.join(trace_dir, "*.manifest.json"))[0]))
        assert manifest["schema"] == "ultra_ep_trace_v1" and manifest["dropped_records"] == 0, manifest
        rows = []
        for path in sorted(glob.glob(os.path.join(trace_dir, "*.npz"))):
            z = np.load(path)
            rows += list(zip(z["virtual_layers"], z["pre_logical_loads"], z["post_physical_loads"]))
        assert len(rows) >= len(trace_expect) > 0
        for (vid_got, pre, post), (vid, exp_pre, exp_post) in zip(rows, trace_expect):
            assert int(vid_got) == vid and np.array_equal(pre, exp_pre) and np.array_equal(post, exp_post)
            assert int(post.sum()) == int(pre.sum())
        shutil.rmtree(trace_dir, ignore_errors=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
