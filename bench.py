#!/usr/bin/env python
"""Benchmark of the per-layer balancing hot path: plan + weight_sync + reroute.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

One "step" is one MoE layer's forward balancing path on one synthetic microbatch:
update_placement (histogram, load all-gather, solve) -> weight_sync (asynchronous, on the
library's communication stream) overlapped with reroute -> join. The workload is the
Qwen3-235B-A22B-shaped FP8 layer (128 experts, top-8, 8192 tokens per rank, R=4 redundant
slots per rank, fp8 weights with UE8M0 scales).

  --gpus 1   EP8 is SIMULATED: all eight ranks live on one device and every kernel serves the
             eight ranks in one launch; peers are buffers of the same device, so weight_sync is
             bounded by HBM, not by NVLink. A step is the whole eight-rank layer.
  --gpus N   (torchrun, one process per GPU) EP = N over cudaIpc-mapped peer memory; a step is
             one rank's layer, the reported time is the maximum over ranks.

Prints ONE JSON line (rank 0). `value` is microseconds per layer with inputs resident on the
device; `e2e` is the same step driven from pinned host buffers (routing ids copied in,
physical ids copied out, every step). `roofline` describes the weight_sync kernel;
`cpu_baseline` is the CPU oracle timed on a bounded sample of the same workload.

--impl reference times the reference's logic for this path on the host cores (the CPU
restatement under oracle/: the reference itself has no CPU implementation of this path) and,
when a GPU and oracle/_ref are present, also reports the reference's own sm_100 kernels on the
same simulated workload under "ref_sm100".
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "us_per_layer_plan_sync_reroute"
UNIT = "us/layer"
FLUSH_BYTES = 256 << 20


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", 6650.0)), "measured (MEASURED_PEAKS.json: hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


NVLINK_PEER_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool (nominal 900)
# DRAM bytes moved inside a full-size weight_sync launch / its algorithmic bytes, from the one-pass ncu capture
# summarised in profiles/weight_sync_kernel_cfg3_dram_traffic.md (reads match; part of the writes is still dirty
# in L2 when the kernel ends)
NCU_SYNC_TRAFFIC_RATIO = 0.72


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# workload
# ------------------------------------------------------------------------------------------
class ForwardWorkload:
    """Device-resident state of the forward step for the ranks this process hosts."""

    def __init__(self, cfg, group, ranks, num_microbatches, num_layers):
        import torch

        from ultra_ep_b200 import workloads as W

        self.torch = torch
        self.cfg, self.group, self.ranks = cfg, group, ranks
        self.num_layers = num_layers
        dev = group.device
        M = cfg.masters
        sizes = [cfg.fc1_numel * cfg.weight_elem_bytes, cfg.fc2_numel * cfg.weight_elem_bytes,
                 cfg.fc1_scale_numel, cfg.fc2_scale_numel]
        self.shard_bytes = sizes
        # master weights: only the bytes matter to the copy path; random bytes on the device
        self.masters = []  # [shard][local rank] -> uint8 [M, bytes]
        g = torch.Generator(device=dev).manual_seed(cfg.seed)
        for nbytes in sizes:
            self.masters.append([torch.randint(0, 256, (M, max(nbytes, 1)), dtype=torch.uint8, device=dev, generator=g)
                                 for _ in ranks])
        self.tables = [group.pointer_tables([[t[m] for m in range(M)] for t in per_rank]) if sizes[s] else None
                       for s, per_rank in enumerate(self.masters)]
        # routing ids: a pool of microbatches, on the device and in pinned host memory. The
        # ranks hosted here share one contiguous buffer per direction, so a step's input is one
        # host->device copy and its result one device->host copy.
        self.ids_host, self.ids_dev, self.ids_all_dev = [], [], []
        for mb in range(num_microbatches):
            host = torch.from_numpy(np.stack([W.routing_ids(cfg, r, microbatch=mb) for r in ranks])).pin_memory()
            self.ids_host.append(host)
            dev_all = host.to(dev)
            self.ids_all_dev.append(dev_all)
            self.ids_dev.append([dev_all[i] for i in range(len(ranks))])
        self.stage_all = torch.empty_like(self.ids_host[0], device=dev)
        self.ids_stage = [self.stage_all[i] for i in range(len(ranks))]
        self.phys_all = torch.empty_like(self.stage_all)
        self.phys_dev = [self.phys_all[i] for i in range(len(ranks))]
        self.phys_host = torch.empty_like(self.ids_host[0]).pin_memory()
        self.flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
        self.flush_read = torch.zeros(FLUSH_BYTES // 4, dtype=torch.int32, device=dev)
        self.h2d_bytes = self.ids_host[0].numel() * 4
        self.d2h_bytes = self.h2d_bytes

    def flush_l2(self):
        """Write a buffer twice the size of L2, then read another one: the step starts with a cold
        L2 that holds no dirty lines of the flush (their write-back would otherwise land inside the
        timed step and be charged to it)."""
        self.flush.zero_()
        self.flush_read.sum()

    def step(self, i, ids=None, result_to_host=False):
        g = self.group
        layer = i % self.num_layers
        ids = self.ids_dev[i % len(self.ids_dev)] if ids is None else ids
        g.update_placement(layer, ids)
        ev = g.weight_sync(layer, self.tables[0], self.tables[1], self.tables[2], self.tables[3], async_finish=True)
        g.reroute_sparse(layer, ids, self.phys_dev)
        if result_to_host:  # the physical ids leave while the weights are still in flight
            self.phys_host.copy_(self.phys_all, non_blocking=True)
        g.wait_event(ev)

    def step_e2e(self, i):
        self.stage_all.copy_(self.ids_host[i % len(self.ids_host)], non_blocking=True)
        self.step(i, self.ids_stage, result_to_host=True)

    def sync_bytes(self, layer, relay_min=0):
        """Algorithmic bytes of one weight_sync launch of the hosted ranks: every replicated
        master is read once and written once per replica. egress / ingress: the largest per-rank
        NVLink volume in each direction; with relaying (experts with >= relay_min replicas) a master's
        rank sends such an expert once and each of its r replicas forwards (r-1)/r of it."""
        cfg = self.cfg
        total_read = total_write = 0
        egress = ingress = 0
        Lp = cfg.masters + cfg.redundant
        for li, r in enumerate(self.ranks):
            lc = self.group.buffer(li, 2)[layer].cpu().numpy()  # BUF_LCNTS
            p2l = self.group.buffer(li, 0)[layer].cpu().numpy()  # BUF_P2L
            reps_of = (lc - 1).clip(min=0)
            relayed = (reps_of >= max(relay_min, 2)) if relay_min > 0 else np.zeros_like(reps_of, bool)
            mine = np.arange(r * cfg.masters, (r + 1) * cfg.masters)
            total_read += int((reps_of[mine] > 0).sum()) * cfg.expert_bytes
            total_write += int(reps_of[mine].sum()) * cfg.expert_bytes
            out = float(np.where(relayed[mine], np.minimum(reps_of[mine], 1), reps_of[mine]).sum())
            hosted = p2l.reshape(cfg.ep, Lp)[r, cfg.masters:]
            hosted = hosted[hosted >= 0]
            out += float(sum((reps_of[l] - 1) / reps_of[l] for l in hosted if relayed[l]))
            if relay_min > 0:  # a forwarded tile is read again from the slot it landed in (its writes are counted above)
                total_read += int(sum(cfg.expert_bytes * (reps_of[l] - 1) / reps_of[l] for l in hosted if relayed[l]))
            egress = max(egress, out * cfg.expert_bytes)
            ingress = max(ingress, len(hosted) * cfg.expert_bytes)
        return total_read, total_write, egress, ingress


def event_ms(torch, fn, stream=None):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    fn()
    e1.record(stream)
    return e0, e1


def run_ours(args):
    import torch
    import torch.distributed as dist

    from ultra_ep_b200 import capi, sim
    from ultra_ep_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    base = W.CONFIGS[args.config]
    num_layers = 8
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        cfg = base.with_ep(world)
        mcfg = sim.make_config(world, cfg.masters, cfg.redundant, num_layers, fc1_numel=cfg.fc1_numel,
                               fc2_numel=cfg.fc2_numel, weight_elem_bytes=cfg.weight_elem_bytes,
                               fc1_scale_numel=cfg.fc1_scale_numel, fc2_scale_numel=cfg.fc2_scale_numel, is_train=False,
                               rank=rank, sim=False, weight_sync_num_sms=args.sync_sms, plan_mode=args.plan_mode,
                               relay_min_replicas=args.relay_min_replicas)
        group = sim.IpcGroup(mcfg, dist.group.WORLD)
        ranks = [rank]
    else:
        cfg = base
        mcfg = sim.make_config(cfg.ep, cfg.masters, cfg.redundant, num_layers, fc1_numel=cfg.fc1_numel,
                               fc2_numel=cfg.fc2_numel, weight_elem_bytes=cfg.weight_elem_bytes,
                               fc1_scale_numel=cfg.fc1_scale_numel, fc2_scale_numel=cfg.fc2_scale_numel, is_train=False,
                               sim=True, weight_sync_num_sms=args.sync_sms, plan_mode=args.plan_mode,
                               relay_min_replicas=args.relay_min_replicas)
        group = sim.SimGroup(mcfg)
        ranks = list(range(cfg.ep))
    wl = ForwardWorkload(cfg, group, ranks, num_microbatches=8, num_layers=num_layers)
    lib = capi.lib()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    # ---- warm-up ---------------------------------------------------------------------------
    for i in range(max(args.warmup, 3)):
        wl.flush_l2()
        wl.step(i)
    barrier()
    group.check_status()

    # ---- timed: K steps, device-resident inputs, L2 flushed between steps ------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    lib.uep_reset_launch_count()
    events = []
    barrier()
    t_wall0 = time.perf_counter()
    for i in range(args.steps):
        wl.flush_l2()  # on the stream: no host synchronisation inside the timed region
        events.append(event_ms(torch, lambda: wl.step(i)))
    barrier()
    t_wall = time.perf_counter() - t_wall0
    launches = int(lib.uep_launch_count())
    step_ms = [a.elapsed_time(b) for a, b in events]
    mean_ms = sum(step_ms) / len(step_ms)

    # ---- e2e: host buffers in, host buffers out, every step ---------------------------------
    for i in range(3):
        wl.step_e2e(i)
    barrier()
    e2e_events = []
    for i in range(args.steps):
        wl.flush_l2()
        e2e_events.append(event_ms(torch, lambda: wl.step_e2e(i)))
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    e2e_ms = sum(a.elapsed_time(b) for a, b in e2e_events) / len(e2e_events)
    group.check_status()

    # ---- the same step captured once into a CUDA graph and replayed (device-resident inputs) ---
    graph_ms = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            wl.step(0, wl.ids_stage)  # sizes are final: nothing allocates during the capture
        torch.cuda.current_stream().wait_stream(side)
        barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            wl.step(0, wl.ids_stage)
        barrier()
        graph_events = []
        for i in range(args.steps):
            wl.stage_all.copy_(wl.ids_all_dev[i % len(wl.ids_all_dev)], non_blocking=True)
            wl.flush_l2()
            graph_events.append(event_ms(torch, graph.replay))
        barrier()
        graph_ms = sum(a.elapsed_time(b) for a, b in graph_events) / len(graph_events)
        group.check_status()

    # ---- per-operation breakdown and the roofline of the weight_sync kernel -----------------
    comm = group.comm_stream()
    plan_ms, sync_ms, reroute_ms = [], [], []
    rd = wr = 0
    link_bytes = []  # per launch: the larger of this GPU's outbound and inbound bytes
    nb = min(args.steps, 16)
    # Each operation is queued right behind the L2 flush (no host synchronisation in between), so
    # its events bracket the kernels, not the latency of a launch into an idle GPU.
    for i in range(nb):
        layer = i % num_layers
        ids = wl.ids_dev[i % len(wl.ids_dev)]
        barrier()
        wl.flush_l2()
        a, b = event_ms(torch, lambda: group.update_placement(layer, ids))
        barrier()
        plan_ms.append(a.elapsed_time(b))
        # weight_sync is timed right behind a plan issued on the same (communication) stream: the
        # plan's load exchange has just lined the ranks up, and there is no cross-stream hand-over
        with torch.cuda.stream(comm):
            wl.flush_l2()
            group.update_placement(layer, ids)
            a, b = event_ms(torch, lambda: group.weight_sync(layer, wl.tables[0], wl.tables[1], wl.tables[2], wl.tables[3]),
                            stream=comm)
        barrier()
        sync_ms.append(a.elapsed_time(b))
        relay_min = 0 if args.plan_mode == 0 else (2 if args.plan_mode == 2 else max(2, args.relay_min_replicas))
        r_, w_, eg, ig = wl.sync_bytes(layer, relay_min)
        rd, wr = rd + r_, wr + w_
        link_bytes.append(float(max(eg, ig)))
        wl.flush_l2()
        a, b = event_ms(torch, lambda: group.reroute_sparse(layer, ids, wl.phys_dev))
        barrier()
        reroute_ms.append(a.elapsed_time(b))
    group.check_status()

    # ---- reduce over ranks -------------------------------------------------------------------
    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def max_over_ranks_each(xs):
        if world == 1:
            return list(xs)
        t = torch.tensor(list(xs), dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    mean_ms = max_over_ranks(mean_ms)
    e2e_ms = max_over_ranks(e2e_ms)
    if graph_ms is not None:
        graph_ms = max_over_ranks(graph_ms)
    sync_each_ms = max_over_ranks_each(sync_ms)  # per launch: the slowest rank
    sync_total_ms = sum(sync_each_ms)
    plan_mean = max_over_ranks(sum(plan_ms) / nb)
    reroute_mean = max_over_ranks(sum(reroute_ms) / nb)
    sync_mean = sync_total_ms / nb
    peak_hbm, peak_src = load_peaks()
    if world == 1:
        alg_bytes = (rd + wr) / nb
        achieved = (rd + wr) / 1e9 / (sync_total_ms / 1e3)
        roofline = {"kernel": "weight_sync_kernel", "bound": "hbm", "achieved": round(achieved, 1), "peak": peak_hbm,
                    "unit": "GB/s", "frac": round(achieved / peak_hbm, 4),
                    "traffic": int(alg_bytes * NCU_SYNC_TRAFFIC_RATIO) if base.name == "cfg3_qwen3_235b_fp8" else None,
                    "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of a full-size launch, as a "
                                      "ratio of its algorithmic bytes (profiles/weight_sync_kernel_cfg3_dram_traffic.md)",
                    "algorithmic_bytes_per_launch": int(alg_bytes), "peak_source": peak_src + "; of measured",
                    "note": "simulated EP: peers are same-device buffers, bytes = reads + writes through HBM"}
    else:
        busiest = sum(max_over_ranks_each(link_bytes))  # per launch: the busiest GPU's link bytes
        achieved = busiest / 1e9 / (sync_total_ms / 1e3)
        roofline = {"kernel": "weight_sync_kernel", "bound": "nvlink", "achieved": round(achieved, 1),
                    "peak": NVLINK_PEER_GBS, "unit": "GB/s", "frac": round(achieved / NVLINK_PEER_GBS, 4),
                    "traffic": None, "algorithmic_bytes_per_launch": int(busiest / nb),
                    "peak_source": "measured peer copy on this pool, per direction (nominal 900); of measured",
                    "note": "per launch: bytes = max(egress, ingress) of the busiest GPU, time = slowest rank; summed over launches"}

    out = None
    if rank == 0:
        cpu = cpu_baseline(cfg if world == 1 else base, args) if (world == 1 and not args.no_cpu_baseline) else None
        ref = ref_sm100(base, args, dev) if (world == 1 and not args.no_ref) else None
        out = {
            "metric": METRIC, "value": round(mean_ms * 1e3, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(mean_ms, 5), "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {
                "workload": f"{cfg.name}: forward update_placement + weight_sync + reroute, "
                            + ("EP8 simulated on one GPU (8 ranks per launch)" if world == 1 else f"EP{world}, one rank per GPU"),
                "experts": cfg.num_experts, "topk": cfg.topk, "tokens_per_rank": cfg.tokens_per_rank,
                "redundant_per_rank": cfg.redundant, "expert_bytes": cfg.expert_bytes, "zipf_s": cfg.zipf_s,
                "weight_sync_plan_mode": args.plan_mode,
                "l2": "between timed steps a 256 MiB buffer is written, then a second 256 MiB buffer is read", "microbatch_pool": 8,
            },
            "clocks": clocks,
            "e2e": {"value": round(e2e_ms * 1e3, 2), "unit": UNIT, "h2d_bytes_per_step": wl.h2d_bytes,
                    "d2h_bytes_per_step": wl.d2h_bytes},
            "gpu_launches": launches,
            "roofline": roofline,
            "breakdown_us": {"plan": round(plan_mean * 1e3, 2), "weight_sync": round(sync_mean * 1e3, 2),
                             "reroute": round(reroute_mean * 1e3, 2),
                             "step_min": round(min(step_ms) * 1e3, 2), "step_max": round(max(step_ms) * 1e3, 2)},
            "wall_s_timed_region": round(t_wall, 3),
        }
        if graph_ms is not None:
            out["graph_replay"] = {"value": round(graph_ms * 1e3, 2), "unit": UNIT,
                                   "note": "the same step (same three calls) captured once into a CUDA graph and replayed; "
                                           "a step always works on layer slot 0 of the plan storage"}
        if cpu is not None:
            out["cpu_baseline"] = cpu
        if ref is not None:
            out["ref_sm100"] = ref
    group.destroy()
    del wl
    torch.cuda.empty_cache()
    if not args.no_backward:
        backward = run_backward(args, world, rank, dev, peak_hbm, max_over_ranks_each)
        if out is not None:
            out["backward"] = backward
    if world > 1:
        dist.destroy_process_group()
    if out is not None:
        print(json.dumps(out))


# ------------------------------------------------------------------------------------------
# backward path (secondary figures)
# ------------------------------------------------------------------------------------------
def run_backward(args, world, rank, dev, peak_hbm, max_over_ranks_each):
    """Backward balancing path of the same layer shape: dense reroute backward (probability
    gradients [T,P] -> [T,L]), the token-gradient row gather ([T*K, hidden] bf16, physical-expert
    order back to (token,k) order) and the fp32 Wgrad reduce of the replicas into their masters.
    Returns per-operation times and the rooflines of the gather and of the reduce."""
    import torch
    import torch.distributed as dist

    from ultra_ep_b200 import capi, sim
    from ultra_ep_b200 import workloads as W

    lib = capi.lib()
    base = W.CONFIGS["cfg4_qwen3_235b_bwd"]
    cfg = base.with_ep(world) if world > 1 else base
    N, M, R, L = cfg.ep, cfg.masters, cfg.redundant, cfg.num_experts
    P = N * (M + R)
    mcfg = sim.make_config(N, M, R, 1, fc1_numel=cfg.fc1_numel, fc2_numel=cfg.fc2_numel,
                           weight_elem_bytes=cfg.weight_elem_bytes, fc1_scale_numel=cfg.fc1_scale_numel,
                           fc2_scale_numel=cfg.fc2_scale_numel, is_train=True, rank=rank, sim=(world == 1),
                           grad_reduce_num_sms=args.reduce_sms)
    group = sim.SimGroup(mcfg) if world == 1 else sim.IpcGroup(mcfg, dist.group.WORLD)
    ranks = list(range(N)) if world == 1 else [rank]
    flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
    flush_read = torch.zeros(FLUSH_BYTES // 4, dtype=torch.int32, device=dev)

    def flush_l2():
        flush.zero_()
        flush_read.sum()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    ids = [torch.from_numpy(W.routing_ids(cfg, r)).to(dev) for r in ranks]
    group.update_placement(0, ids)
    phys = group.reroute_sparse(0, ids)
    barrier()
    reps = 6
    out = {"workload": f"{cfg.name}: backward of the same layer, " + ("EP8 simulated on one GPU" if world == 1 else f"EP{world}")}

    # -- Wgrad reduce ------------------------------------------------------------------------
    numel = cfg.fc1_numel + cfg.fc2_numel
    g1 = [torch.full((M, cfg.fc1_numel), 1e-4, dtype=torch.float32, device=dev) for _ in ranks]
    g2 = [torch.full((M, cfg.fc2_numel), 1e-4, dtype=torch.float32, device=dev) for _ in ranks]
    t1 = group.pointer_tables([[g[m] for m in range(M)] for g in g1])
    t2 = group.pointer_tables([[g[m] for m in range(M)] for g in g2])
    for li in range(len(ranks)):
        group.buffer(li, capi.BUF_REPLICA_GRAD).fill_(1e-4)
    hbm_bytes = 0
    link = 0
    for li, r in enumerate(ranks):
        lc = group.buffer(li, capi.BUF_LCNTS)[0].cpu().numpy()
        p2l = group.buffer(li, capi.BUF_P2L)[0].cpu().numpy().reshape(N, M + R)
        mine = lc[r * M:(r + 1) * M]
        n_rep = int((mine - 1).clip(min=0).sum())
        hbm_bytes += int((mine > 1).sum()) * 8 * numel + n_rep * 8 * numel  # masters read+written; replicas read+zeroed
        used = int((p2l[r, M:] >= 0).sum())
        link = max(link, n_rep * 4 * numel, used * 4 * numel)
    comm = group.comm_stream()
    red = []
    for it in range(3 + reps):
        barrier()
        with torch.cuda.stream(comm):
            flush_l2()
            a, b = event_ms(torch, lambda: group.grad_reduce(0, t1, t2), stream=comm)
        barrier()
        if it >= 3:
            red.append(a.elapsed_time(b))
    group.check_status()
    red = max_over_ranks_each(red)
    red_ms = sum(red) / len(red)
    out["grad_reduce_us"] = round(red_ms * 1e3, 1)
    if world == 1:
        ach = hbm_bytes / 1e9 / (red_ms / 1e3)
        out["grad_reduce_roofline"] = {"bound": "hbm", "achieved": round(ach, 1), "peak": peak_hbm, "unit": "GB/s",
                                       "frac": round(ach / peak_hbm, 4), "algorithmic_bytes_per_launch": hbm_bytes,
                                       "ctas": args.reduce_sms,
                                       "note": "simulated EP: masters read+written, replicas read+zeroed, all through HBM"}
    else:
        busiest = max(max_over_ranks_each([float(link)]))
        ach = busiest / 1e9 / (red_ms / 1e3)
        out["grad_reduce_roofline"] = {"bound": "nvlink", "achieved": round(ach, 1), "peak": NVLINK_PEER_GBS, "unit": "GB/s",
                                       "frac": round(ach / NVLINK_PEER_GBS, 4), "algorithmic_bytes_per_launch": int(busiest),
                                       "ctas": args.reduce_sms,
                                       "note": "bytes = replica gradients the busiest GPU pulls in (it pushes as many zeros)"}
    del g1, g2, t1, t2

    # -- token-gradient gather (one rank's rows per launch) ------------------------------------
    H = cfg.hidden
    rows = cfg.tokens_per_rank * cfg.topk
    src = torch.empty((rows, H), dtype=torch.bfloat16, device=dev).normal_(0, 1e-3)
    dst = torch.empty_like(src)
    pos = torch.empty(rows, dtype=torch.int32, device=dev)
    offs = torch.empty(P + 1, dtype=torch.int32, device=dev)
    scratch = torch.empty(int(lib.uep_dispatch_scratch_elems(rows, P)), dtype=torch.int32, device=dev)
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    pos_t, gat_t = [], []
    for it in range(3 + reps):
        barrier()
        flush_l2()
        a, b = event_ms(torch, lambda: capi.check(lib.uep_dispatch_positions(
            phys[0].data_ptr(), rows, P, pos.data_ptr(), offs.data_ptr(), scratch.data_ptr(), st), "uep_dispatch_positions"))
        c, d = event_ms(torch, lambda: capi.check(lib.uep_gather_rows(
            src.data_ptr(), pos.data_ptr(), dst.data_ptr(), rows, rows, H * 2, status.data_ptr(), st), "uep_gather_rows"))
        barrier()
        if it >= 3:
            pos_t.append(a.elapsed_time(b))
            gat_t.append(c.elapsed_time(d))
    if int(status[0].item()) != 0:
        raise RuntimeError("uep_gather_rows reported an out-of-range row index")
    gat = max_over_ranks_each(gat_t)
    gat_ms = sum(gat) / len(gat)
    gbytes = 2 * rows * H * 2
    ach = gbytes / 1e9 / (gat_ms / 1e3)
    out["dispatch_positions_us"] = round(sum(pos_t) / len(pos_t) * 1e3, 1)
    out["gather_rows_us"] = round(gat_ms * 1e3, 1)
    out["gather_rows_roofline"] = {"bound": "hbm", "achieved": round(ach, 1), "peak": peak_hbm, "unit": "GB/s",
                                   "frac": round(ach / peak_hbm, 4), "algorithmic_bytes_per_launch": gbytes,
                                   "note": f"[{rows},{H}] bf16 rows read once and written once, one rank per launch"}
    del src, dst

    # -- dense reroute backward (probability gradients) ---------------------------------------
    maps = [torch.from_numpy(W.ids_to_map(x.cpu().numpy(), L)).to(dev) for x in ids]
    probs = [torch.rand(m.shape, dtype=torch.float32, device=dev) * m for m in maps]
    ex_probs, ex_maps = group.reroute_dense(0, maps, probs)
    fwd = []
    for it in range(3 + reps):
        barrier()
        flush_l2()
        a, b = event_ms(torch, lambda: group.reroute_dense(0, maps, probs, out=(ex_probs, ex_maps)))
        barrier()
        if it >= 3:
            fwd.append(a.elapsed_time(b))
    fwd = max_over_ranks_each(fwd)
    fwd_ms = sum(fwd) / len(fwd)
    T_ = cfg.tokens_per_rank
    fwd_bytes = len(ranks) * T_ * (L * 5 + P * 5)  # bool map + fp32 probs in, bool map + fp32 probs out (written once)
    out["dense_reroute_forward_us"] = round(fwd_ms * 1e3, 1)
    out["dense_reroute_forward_roofline"] = {"bound": "hbm", "achieved": round(fwd_bytes / 1e9 / (fwd_ms / 1e3), 1),
                                             "peak": peak_hbm, "unit": "GB/s",
                                             "frac": round(fwd_bytes / 1e9 / (fwd_ms / 1e3) / peak_hbm, 4),
                                             "algorithmic_bytes_per_launch": fwd_bytes,
                                             "note": "two launches (tile counts, scatter) into preallocated outputs"}
    grads = [torch.rand_like(p_) for p_ in ex_probs]
    bwd = []
    for it in range(3 + reps):
        barrier()
        flush_l2()
        a, b = event_ms(torch, lambda: group.reroute_dense_backward(0, grads, maps, ex_maps))
        barrier()
        if it >= 3:
            bwd.append(a.elapsed_time(b))
    bwd = max_over_ranks_each(bwd)
    out["dense_reroute_backward_us"] = round(sum(bwd) / len(bwd) * 1e3, 1)
    group.check_status()
    group.destroy()
    return out


# ------------------------------------------------------------------------------------------
# baselines
# ------------------------------------------------------------------------------------------
def cpu_forward_layer(cfg, iters_cap=200, budget_s=10.0, threads=None):
    """The oracle's whole-group forward layer on host threads (plan + reroute + weight copy)."""
    import ctypes as C

    from oracle import uep_oracle as O
    from ultra_ep_b200 import workloads as W

    lib = O.lib()
    N, M, R = cfg.ep, cfg.masters, cfg.redundant
    threads = threads or min(N, lib.uep_oracle_hardware_threads() or 1)
    ids = np.ascontiguousarray(np.stack([W.routing_ids(cfg, r).reshape(-1) for r in range(N)]))
    expert_bytes = cfg.expert_bytes
    masters = np.empty((N * M, expert_bytes), np.uint8)
    masters[:] = 7
    replicas = np.zeros((N, R, expert_bytes), np.uint8)
    mptr = (C.c_void_p * (N * M))(*[masters[i].ctypes.data for i in range(N * M)])
    rptr = (C.c_void_p * N)(*[replicas[r].ctypes.data for r in range(N)])
    p2l = np.empty(N * (M + R), np.int32)
    phys = np.empty_like(ids)
    parts = [C.c_double(), C.c_double(), C.c_double()]

    def run(iters):
        return lib.uep_oracle_time_forward_layer(
            ids, cfg.tokens_per_rank, cfg.topk, N, M, R, 1.0, 1024, 0, 1, 0.01, 1, mptr, expert_bytes, rptr, p2l, phys,
            iters, threads, C.byref(parts[0]), C.byref(parts[1]), C.byref(parts[2]))

    t1 = run(1)
    iters = int(max(3, min(iters_cap, budget_s / max(t1, 1e-6))))
    total = run(iters)
    return {"us_per_layer": total / iters * 1e6, "iters": iters, "threads": threads,
            "plan_us": parts[0].value / iters * 1e6, "reroute_us": parts[1].value / iters * 1e6,
            "sync_us": parts[2].value / iters * 1e6, "cores_online": lib.uep_oracle_hardware_threads()}


def cpu_baseline(cfg, args):
    r = cpu_forward_layer(cfg, budget_s=args.cpu_budget_s)
    return {"value": round(r["us_per_layer"], 1), "unit": UNIT, "cores": r["threads"], "kind": "port",
            "sample": f"{r['iters']} layers of the same 8-rank workload (all ranks on host threads; "
                      f"plan {r['plan_us']:.0f} us, reroute {r['reroute_us']:.0f} us, weight copy {r['sync_us']:.0f} us)",
            "host_threads_online": r["cores_online"]}


def ref_sm100(cfg, args, dev):
    """The reference's own kernels (built unmodified for sm_100 into oracle/_ref) on the same
    simulated eight-rank layer: histogram + reduce + solve, task build + copy kernel, sparse
    quota reroute, rank after rank on one stream, as the reference issues them."""
    try:
        import torch

        from oracle import uep_ref
        from ultra_ep_b200 import workloads as W

        if not uep_ref.available():
            return {"unavailable": "oracle/_ref/libuep_ref.so not present"}
        N, M, R, L = cfg.ep, cfg.masters, cfg.redundant, cfg.num_experts
        lib = uep_ref.lib()
        ids = [torch.from_numpy(W.routing_ids(cfg, r)).to(dev).long() for r in range(N)]
        sizes = [cfg.fc1_numel * cfg.weight_elem_bytes, cfg.fc2_numel * cfg.weight_elem_bytes, cfg.fc1_scale_numel,
                 cfg.fc2_scale_numel]
        masters = [[torch.randint(0, 256, (M, max(n, 1)), dtype=torch.uint8, device=dev) for _ in range(N)] for n in sizes]
        tables = [[torch.tensor([t[m].data_ptr() for m in range(M)], dtype=torch.int64, device=dev) for t in per]
                  for per in masters]
        scale_stride = (((sizes[2] + 15) // 16 * 16) + sizes[3] + 15) // 16 * 16
        rep_w = [torch.zeros(R, sizes[0] + sizes[1], dtype=torch.uint8, device=dev) for _ in range(N)]
        rep_s = [torch.zeros(R, max(scale_stride, 1), dtype=torch.uint8, device=dev) for _ in range(N)]
        spaces = [uep_ref.Workspace(r, N, M, R, cfg.fc1_numel, cfg.fc2_numel, cfg.weight_elem_bytes, 1, cfg.fc1_scale_numel,
                                    cfg.fc2_scale_numel, N, [t.data_ptr() for t in rep_w], [t.data_ptr() for t in rep_s], None)
                  for r in range(N)]
        per_rank = torch.zeros(N, L, dtype=torch.int32, device=dev)
        gl = torch.zeros(L, dtype=torch.int32, device=dev)
        local = torch.zeros(L, dtype=torch.int32, device=dev)
        P, D = N * (M + R), N
        plans = [{k: torch.empty(s, dtype=torch.int32, device=dev) for k, s in
                  [("p2l", (P,)), ("l2p", (L, D)), ("lcnts", (L,)), ("quota", (L, D)), ("qp", (L, D)), ("rqp", (L, D))]}
                 for _ in range(N)]
        counters = torch.zeros(L, dtype=torch.int32, device=dev)
        flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
        flush_read = torch.zeros(FLUSH_BYTES // 4, dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        work = [t.clone() for t in ids]

        def plan_all():
            for r in range(N):  # histogram of each rank, written into the gathered matrix
                lib.uep_ref_topk_local_sum(ids[r].data_ptr(), cfg.tokens_per_rank, cfg.topk, L, per_rank[r].data_ptr(), stream)
            for r in range(N):
                lib.uep_ref_reduce_per_rank_loads(per_rank.data_ptr(), gl.data_ptr(), N, L, stream)
                p = plans[r]
                lib.uep_ref_solve_placement(gl.data_ptr(), per_rank.data_ptr(), p["p2l"].data_ptr(), p["l2p"].data_ptr(),
                                            p["lcnts"].data_ptr(), p["quota"].data_ptr(), p["qp"].data_ptr(),
                                            p["rqp"].data_ptr(), stream, L, N, M, R, N, D, 1.0, 1024, 0, 1, 0.01, 1, r)

        def sync_all():
            for r in range(N):
                p = plans[r]
                spaces[r].weight_sync(p["p2l"], p["l2p"], p["lcnts"], tables[0][r], tables[1][r], tables[2][r],
                                      tables[3][r], rep_w[r], rep_s[r], stream)

        def reroute_all():
            for r in range(N):
                p = plans[r]
                lib.uep_ref_sparse_reroute_quota(work[r].data_ptr(), p["l2p"].data_ptr(), p["lcnts"].data_ptr(),
                                                 p["rqp"].data_ptr(), counters.data_ptr(), cfg.tokens_per_rank, cfg.topk,
                                                 L, D, stream)

        res = {}
        for name, fn in (("plan", plan_all), ("weight_sync", sync_all), ("reroute", reroute_all)):
            times = []
            for it in range(3 + min(args.steps, 16)):
                if name == "reroute":
                    for w_, s_ in zip(work, ids):
                        w_.copy_(s_)
                flush.zero_()
                flush_read.sum()
                torch.cuda.synchronize()
                a, b = event_ms(torch, fn)
                torch.cuda.synchronize()
                if it >= 3:
                    times.append(a.elapsed_time(b))
            res[name] = round(sum(times) / len(times) * 1e3, 2)
        for ws in spaces:
            ws.close()
        res["serial_total"] = round(res["plan"] + res["weight_sync"] + res["reroute"], 2)
        res["exposed_total"] = round(res["plan"] + max(res["weight_sync"], res["reroute"]), 2)
        res["unit"] = UNIT
        res["note"] = ("reference kernels compiled from its sources for sm_100, eight simulated ranks issued one after "
                       "another on one stream; weight_sync runs its thread-copy kernel (NVLink domain <= 8)")
        return res
    except Exception as e:  # the reference build is optional evidence, never a reason to fail the bench
        return {"unavailable": f"{type(e).__name__}: {e}"}


def run_reference(args):
    """Reference arm: the reference's logic for this path on host cores (bounded sample)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from ultra_ep_b200 import workloads as W

    cfg = W.CONFIGS[args.config]
    steps = max(1, args.steps)
    per_step = []
    r = None
    for _ in range(min(args.warmup, 1)):
        cpu_forward_layer(cfg, iters_cap=2, budget_s=1.0)
    budget = min(args.cpu_budget_s, 60.0 / steps)
    for _ in range(min(steps, 5)):
        r = cpu_forward_layer(cfg, iters_cap=50, budget_s=budget)
        per_step.append(r["us_per_layer"])
    value = sum(per_step) / len(per_step)
    out = {
        "impl": "reference", "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(value / 1e3, 4), "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": f"{cfg.name}: forward update_placement + weight_sync + reroute, EP8, all ranks on host threads",
                   "experts": cfg.num_experts, "topk": cfg.topk, "tokens_per_rank": cfg.tokens_per_rank,
                   "redundant_per_rank": cfg.redundant, "expert_bytes": cfg.expert_bytes},
        "cpu_baseline": {"value": round(value, 1), "unit": UNIT, "cores": r["threads"], "kind": "port",
                         "sample": f"{len(per_step)} samples of {r['iters']} layers each; the reference has no CPU "
                                   "implementation of this path, the CPU restatement under oracle/ is timed",
                         "host_threads_online": r["cores_online"]},
        "e2e": {"value": round(value, 1), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    try:
        import torch

        if torch.cuda.is_available() and not args.no_ref:
            torch.cuda.set_device(0)
            out["ref_sm100"] = ref_sm100(cfg, args, torch.device("cuda", 0))
    except Exception as e:
        out["ref_sm100"] = {"unavailable": f"{type(e).__name__}: {e}"}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg3_qwen3_235b_fp8")
    ap.add_argument("--sync-sms", type=int, default=0, help="CTAs per rank of the weight_sync kernel (0 = default)")
    ap.add_argument("--plan-mode", type=int, default=0, choices=[0, 1, 2],
                    help="weight_sync: 0 direct fan-out, 1 relay experts with >= --relay-min-replicas replicas, 2 relay all with >= 2")
    ap.add_argument("--relay-min-replicas", type=int, default=4)
    ap.add_argument("--cpu-budget-s", type=float, default=10.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="skip the CUDA-graph replay figure")
    ap.add_argument("--no-backward", action="store_true", help="skip the backward-path figures (cfg4)")
    ap.add_argument("--reduce-sms", type=int, default=42, help="CTAs of the Wgrad reduce kernel (reference default 42)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
