#!/usr/bin/env python
"""Benchmark of the per-layer balancing hot path: plan + weight_sync + reroute.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

One "step" is one MoE layer's forward balancing path on one synthetic microbatch:
update_placement (histogram, load all-gather, solve) -> weight_sync (asynchronous, on the
library's communication stream) overlapped with reroute -> join. The headline workload is the
Qwen3-235B-A22B-shaped FP8 layer (128 experts, top-8, 8192 tokens per rank, R=4 redundant
slots per rank, fp8 weights with UE8M0 scales).

  --gpus 1   EP8 is SIMULATED: all eight ranks live on one device and every kernel serves the
             eight ranks in one launch; peers are buffers of the same device, so weight_sync is
             bounded by HBM, not by NVLink. A step is the whole eight-rank layer.
  --gpus N   (torchrun, one process per GPU) EP = N over cudaIpc-mapped peer memory; a step is
             one rank's layer, the reported time is the maximum over ranks.

Prints ONE JSON line (rank 0):
  value         microseconds per layer, inputs resident on the device, C-ABI calls (mean over the timed
                steps of the per-step maximum over ranks; `step_stats_us` adds median and percentiles,
                `value_statistic` the largest of the ranks' own means). At N > 1 the ranks are lined up on the
                device (a one-word all-reduce on the stream) in front of every L2 flush, outside the timed events
  e2e           the same step driven from pinned host buffers (routing ids copied in, physical ids
                copied out, every step): through the drop-in `Manager` (pybind module `_C`) at N > 1,
                through the C ABI on the simulated group at N = 1 (the Manager hosts one rank per process)
  parity        every check of this run against the CPU oracle / the fixed-order sums: plans, routing,
                synced bytes, reduced gradients, at the benchmark's full sizes; a false entry makes the
                process exit non-zero
  roofline      the weight_sync kernel (HBM at N = 1, NVLink at N > 1 with the link measured in the run)
  ref_sm100     the reference's own kernels (oracle/_ref) on the same plans, masters and peer memory
  manager_api   the drop-in Manager timed at full size (N > 1)
  backward      cfg 4: Wgrad reduce, token-gradient gather, dense reroute forward/backward
  configs       cfg 1, cfg 2 and cfg 5 (forward + backward with four microbatch slots in flight)
  cpu_baseline  the CPU oracle timed on a bounded sample of the same workload (N = 1)

--profile-case NAME runs a few launches of one kernel family and exits (for profiler captures); NAME = trace prints
the kernels' own time stamps of plan and weight_sync at full size, at any N.

--impl reference times the reference's logic for this path on the host cores (the CPU
restatement under oracle/: the reference itself has no CPU implementation of this path).
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
NVLINK_NOMINAL_GBS = 900.0  # per direction per GPU, the figure the target of this path is stated against
# DRAM bytes moved inside a full-size weight_sync launch of the simulated group / its algorithmic bytes, from a
# one-pass ncu capture of dram__bytes_read.sum + dram__bytes_write.sum (reads match the algorithmic reads; part
# of the writes is still dirty in L2 when the kernel ends). Recorded, not measured in this run.
NCU_SYNC_TRAFFIC_RATIO = 0.72


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", 6650.0)), "measured (MEASURED_PEAKS.json: hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


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


def stats_us(ms_values):
    """mean / median / 10th / 90th percentile (microseconds) of a list of milliseconds."""
    v = sorted(float(x) * 1e3 for x in ms_values)
    if not v:
        return None
    q = lambda f: v[min(len(v) - 1, max(0, int(round(f * (len(v) - 1)))))]
    return {"mean": round(sum(v) / len(v), 2), "median": round(q(0.5), 2), "p10": round(q(0.1), 2),
            "p90": round(q(0.9), 2), "min": round(v[0], 2), "max": round(v[-1], 2), "n": len(v)}


def pool_size(steps: int) -> int:
    """Microbatch pool: a divisor of the step count (so that every microbatch runs equally often), 4..10."""
    for n in (8, 10, 6, 5, 4, 9, 7):
        if steps % n == 0:
            return n
    return 8


# ------------------------------------------------------------------------------------------
# process-wide helpers
# ------------------------------------------------------------------------------------------
class Env:
    def __init__(self):
        import torch

        self.torch = torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=self.dev)
        self.flush_read = torch.zeros(FLUSH_BYTES // 4, dtype=torch.int32, device=self.dev)
        self._align_word = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.failures = []  # parity failures (messages)

    def flush_l2(self):
        """Write a buffer twice the size of L2, then read another one: the step starts with a cold
        L2 that holds no dirty lines of the flush (their write-back would otherwise land inside the
        timed step and be charged to it)."""
        self.align()
        self.flush.zero_()
        self.flush_read.sum()

    def align(self):
        """Line the ranks up ON THE DEVICE (a one-word all-reduce queued on the stream; the host does not wait):
        the ranks enter every timed step together, as they enter a layer behind the dispatch of the layer
        before. Without it a rank that had little to copy in one step starts the next step early, waits in the
        load exchange for the others, and that wait is charged to the next step's slowest-rank time."""
        if self.world > 1:
            self.dist.all_reduce(self._align_word)

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()

    def max_each(self, xs):
        xs = list(xs)
        if self.world == 1 or not xs:
            return xs
        t = self.torch.tensor(xs, dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def all_true(self, ok: bool) -> bool:
        if self.world == 1:
            return bool(ok)
        t = self.torch.tensor([0 if ok else 1], dtype=self.torch.int32, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return int(t.item()) == 0

    def check(self, what: str, ok: bool) -> bool:
        if not ok:
            self.failures.append(f"rank {self.rank}: {what}")
            print(f"[bench] PARITY FAILURE rank {self.rank}: {what}", file=sys.stderr, flush=True)
        return bool(ok)

    def gather_ids(self, ids_local):
        """int32 [T,K] tensors of the hosted ranks -> numpy arrays of all ranks of the group."""
        if self.world == 1:
            return [x.cpu().numpy() for x in ids_local]
        parts = [self.torch.empty_like(ids_local[0]) for _ in range(self.world)]
        self.dist.all_gather(parts, ids_local[0].contiguous())
        return [p.cpu().numpy() for p in parts]


def timed(torch, fn, stream=None):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    fn()
    e1.record(stream)
    return e0, e1


def seeded_bytes(torch, dev, key: int, n: int):
    g = torch.Generator(device=dev).manual_seed(int(key))
    return torch.randint(0, 256, (max(n, 1),), dtype=torch.uint8, device=dev, generator=g)


def seeded_normal(torch, dev, key: int, n: int, std: float):
    g = torch.Generator(device=dev).manual_seed(int(key))
    return torch.randn(n, dtype=torch.float32, device=dev, generator=g) * std


def master_key(cfg, expert: int, shard: int) -> int:
    return (cfg.seed * 1000003 + expert) * 4 + shard


def make_group(env, cfg, num_layers, is_train, args, plan_mode=None, reduce_sms=None):
    """The C-ABI group of this process: the simulated one (all ranks hosted here) or one rank of the real one."""
    from ultra_ep_b200 import sim

    pm = args.plan_mode_resolved if plan_mode is None else plan_mode
    mcfg = sim.make_config(cfg.ep, cfg.masters, cfg.redundant, num_layers, fc1_numel=cfg.fc1_numel,
                           fc2_numel=cfg.fc2_numel, weight_elem_bytes=cfg.weight_elem_bytes,
                           fc1_scale_numel=cfg.fc1_scale_numel, fc2_scale_numel=cfg.fc2_scale_numel, is_train=is_train,
                           rank=env.rank if env.world > 1 else 0, sim=(env.world == 1),
                           weight_sync_num_sms=args.sync_sms, plan_mode=pm, relay_min_replicas=args.relay_min_replicas,
                           grad_reduce_num_sms=reduce_sms or args.reduce_sms)
    mcfg.reroute_max_tokens = cfg.tokens_per_rank  # the reroute scratch has its final size from the start
    mcfg.reroute_max_topk = cfg.topk
    if env.world == 1:
        return sim.SimGroup(mcfg), list(range(cfg.ep))
    return sim.IpcGroup(mcfg, env.dist.group.WORLD), [env.rank]


class Masters:
    """Master weights of the hosted ranks: bytes seeded by (global expert, shard), so that any rank can
    rebuild any master on its own device when it checks what landed in its replica slots."""

    def __init__(self, env, cfg, group, ranks):
        torch = env.torch
        self.env, self.cfg, self.ranks = env, cfg, ranks
        M = cfg.masters
        self.sizes = [cfg.fc1_numel * cfg.weight_elem_bytes, cfg.fc2_numel * cfg.weight_elem_bytes,
                      cfg.fc1_scale_numel, cfg.fc2_scale_numel]
        self.data = []  # [shard][local rank] -> uint8 [M, bytes]
        for s, nbytes in enumerate(self.sizes):
            per_rank = []
            for r in ranks:
                t = torch.empty((M, max(nbytes, 1)), dtype=torch.uint8, device=env.dev)
                for m in range(M):
                    t[m].copy_(seeded_bytes(torch, env.dev, master_key(cfg, r * M + m, s), nbytes))
                per_rank.append(t)
            self.data.append(per_rank)
        self.tables = [group.pointer_tables([[t[m] for m in range(M)] for t in per_rank]) if self.sizes[s] else None
                       for s, per_rank in enumerate(self.data)]

    def expected(self, expert: int, shard: int):
        return seeded_bytes(self.env.torch, self.env.dev, master_key(self.cfg, expert, shard), self.sizes[shard])


def oracle_plans(cfg, ids_all, ranks):
    from oracle import uep_oracle as O

    L = cfg.num_experts
    lpr = np.stack([np.bincount(x.reshape(-1), minlength=L) for x in ids_all]).astype(np.int32)
    return {r: O.solve_placement(lpr, cfg.masters, cfg.redundant, cfg.ep, r) for r in ranks}


def check_plan_and_routing(env, cfg, group, ranks, layer, ids_local, phys_local, tag):
    """Plans (all six arrays) and physical ids of the hosted ranks against the CPU oracle, bit for bit."""
    from oracle import uep_oracle as O
    from ultra_ep_b200 import capi

    ids_all = env.gather_ids(ids_local)
    plans = oracle_plans(cfg, ids_all, ranks)
    ok_plan = ok_route = True
    for li, r in enumerate(ranks):
        got = group.plan(li, layer)
        for f, v in plans[r].fields().items():
            ok_plan &= env.check(f"{tag}: plan field {f} of rank {r}", np.array_equal(got[f].cpu().numpy(), v))
        if phys_local is not None:
            exp = O.sparse_reroute(ids_all[r if env.world > 1 else li].astype(np.int32), plans[r], True)
            ok_route &= env.check(f"{tag}: physical ids of rank {r}", np.array_equal(phys_local[li].cpu().numpy(), exp))
        pl = group.buffer(li, capi.BUF_PHYSICAL_LOADS)[layer].cpu().numpy()
        ok_plan &= env.check(f"{tag}: physical loads of rank {r}",
                             np.array_equal(pl, O.physical_loads_from_plan(plans[r], pl.shape[0])))
    return ok_plan, ok_route, plans


def check_replica_bytes(env, cfg, group, ranks, masters, plans, before_w, before_s, tag):
    """Every used replica slot holds its master's bytes (all four shards); unused slots are untouched."""
    from ultra_ep_b200 import capi

    torch = env.torch
    M, R = cfg.masters, cfg.redundant
    Lp = M + R
    s2_off = (masters.sizes[2] + 15) // 16 * 16
    ok = True
    for li, r in enumerate(ranks):
        w = group.buffer(li, capi.BUF_REPLICA_WEIGHT)
        s = group.buffer(li, capi.BUF_REPLICA_SCALE)
        plan = plans[r]
        for slot in range(R):
            l = int(plan.p2l[r * Lp + M + slot])
            if l < 0:
                ok &= env.check(f"{tag}: unused slot {slot} of rank {r} was written",
                                torch.equal(w[slot], before_w[li][slot]) and (s.numel() == 0 or torch.equal(s[slot], before_s[li][slot])))
                continue
            b1, b2 = masters.sizes[0], masters.sizes[1]
            ok &= env.check(f"{tag}: fc1 bytes of expert {l} in slot {slot} of rank {r}", torch.equal(w[slot, :b1], masters.expected(l, 0)))
            ok &= env.check(f"{tag}: fc2 bytes of expert {l} in slot {slot} of rank {r}", torch.equal(w[slot, b1:b1 + b2], masters.expected(l, 1)))
            if masters.sizes[2]:
                ok &= env.check(f"{tag}: fc1 scales of expert {l} in slot {slot} of rank {r}",
                                torch.equal(s[slot, :masters.sizes[2]], masters.expected(l, 2)))
                ok &= env.check(f"{tag}: fc2 scales of expert {l} in slot {slot} of rank {r}",
                                torch.equal(s[slot, s2_off:s2_off + masters.sizes[3]], masters.expected(l, 3)))
    return ok


def randomise_replicas(env, group, ranks):
    """Fill the replica slots with noise and return copies, so that 'untouched' is observable."""
    from ultra_ep_b200 import capi

    bw, bs = [], []
    for li in range(len(ranks)):
        w = group.buffer(li, capi.BUF_REPLICA_WEIGHT)
        s = group.buffer(li, capi.BUF_REPLICA_SCALE)
        w.random_(0, 256)
        if s.numel():
            s.random_(0, 256)
        bw.append(w.clone())
        bs.append(s.clone())
    return bw, bs


def link_volumes(cfg, plan, ranks, relay_of=None):
    """Experts each hosted rank sends / receives under a plan (NVLink volume in units of one expert), and
    the reads / writes of the launch. relay_of[l] > 0: expert l is relayed (its master sends it once, each
    of its r replicas forwards (r-1)/r of it)."""
    M, R, N = cfg.masters, cfg.redundant, cfg.ep
    Lp = M + R
    reps = (plan.lcnts - 1).clip(min=0)
    p2l = plan.p2l.reshape(N, Lp)
    out = []
    for r in ranks:
        mine = range(r * M, (r + 1) * M)
        eg = 0.0
        for l in mine:
            if reps[l] > 0:
                eg += 1.0 if (relay_of is not None and relay_of[l]) else float(reps[l])
        hosted = [int(l) for l in p2l[r, M:] if l >= 0]
        if relay_of is not None:
            eg += sum((reps[l] - 1) / reps[l] for l in hosted if relay_of[l])
        out.append({"egress": eg, "ingress": float(len(hosted)),
                    "reads": int(sum(1 for l in mine if reps[l] > 0)), "writes": int(sum(int(reps[l]) for l in mine))})
    return out


def relay_selection(cfg, plan, plan_mode, relay_min):
    """Which experts weight_sync relays: the rule of the kernel (ultra_ep_b200/csrc/weight_sync.cu), restated."""
    if plan_mode == 0 or cfg.ep <= 2:  # two ranks: the library launches the direct kernel whatever the mode
        return None
    M, R, N = cfg.masters, cfg.redundant, cfg.ep
    Lp = M + R
    reps = (plan.lcnts - 1).clip(min=0)
    thr = 2 if plan_mode == 2 else max(2, relay_min)
    rel = [int(r) if (r >= thr and r <= 16) else 0 for r in reps]
    if plan_mode == 1:
        p2l = plan.p2l.reshape(N, Lp)
        floor_in = max(1, max(int((p2l[r, M:] >= 0).sum()) for r in range(N)))
        for r in range(N):
            out = int(reps[r * M:(r + 1) * M].sum())
            while out > floor_in:
                best, best_reps = -1, 1
                for l in range(r * M, (r + 1) * M):
                    if not rel[l] and reps[l] > best_reps and reps[l] <= 16:
                        best, best_reps = l, int(reps[l])
                if best < 0:
                    break
                rel[best] = best_reps
                out -= best_reps - 1
    return rel


# ------------------------------------------------------------------------------------------
# forward path of one configuration through the C ABI
# ------------------------------------------------------------------------------------------
class Forward:
    def __init__(self, env, cfg, args, num_layers, pool, is_train=False, with_weights=True):
        from ultra_ep_b200 import workloads as W

        torch = env.torch
        self.env, self.cfg, self.args, self.num_layers = env, cfg, args, num_layers
        self.with_weights = with_weights and cfg.expert_bytes > 0
        self.group, self.ranks = make_group(env, cfg, num_layers, is_train, args)
        self.masters = Masters(env, cfg, self.group, self.ranks) if self.with_weights else None
        # routing ids: a pool of microbatches, on the device and in pinned host memory. The ranks hosted
        # here share one contiguous buffer per direction, so a step's input is one host->device copy and
        # its result one device->host copy.
        self.ids_host, self.ids_dev, self.ids_all_dev = [], [], []
        for mb in range(pool):
            host = torch.from_numpy(np.stack([W.routing_ids(cfg, r, microbatch=mb) for r in self.ranks])).pin_memory()
            self.ids_host.append(host)
            dev_all = host.to(env.dev)
            self.ids_all_dev.append(dev_all)
            self.ids_dev.append([dev_all[i] for i in range(len(self.ranks))])
        self.stage_all = torch.empty_like(self.ids_host[0], device=env.dev)
        self.ids_stage = [self.stage_all[i] for i in range(len(self.ranks))]
        self.phys_all = torch.empty_like(self.stage_all)
        self.phys_dev = [self.phys_all[i] for i in range(len(self.ranks))]
        self.phys_host = torch.empty_like(self.ids_host[0]).pin_memory()
        self.h2d_bytes = self.ids_host[0].numel() * 4
        self.d2h_bytes = self.h2d_bytes

    def step(self, i, ids=None, result_to_host=False, layer=None):
        g = self.group
        layer = i % self.num_layers if layer is None else layer
        ids = self.ids_dev[i % len(self.ids_dev)] if ids is None else ids
        g.update_placement(layer, ids)
        ev = None
        if self.with_weights:
            t = self.masters.tables
            ev = g.weight_sync(layer, t[0], t[1], t[2], t[3], async_finish=True)
        g.reroute_sparse(layer, ids, self.phys_dev)
        if result_to_host:  # the physical ids leave while the weights are still in flight
            self.phys_host.copy_(self.phys_all, non_blocking=True)
        if ev is not None:
            g.wait_event(ev)

    def step_e2e(self, i):
        self.stage_all.copy_(self.ids_host[i % len(self.ids_host)], non_blocking=True)
        self.step(i, self.ids_stage, result_to_host=True)

    def run_timed(self, fn, steps, warmup):
        env = self.env
        for i in range(warmup):
            env.flush_l2()
            fn(i)
        env.barrier()
        self.group.check_status()
        events = []
        env.barrier()
        for i in range(steps):
            env.flush_l2()  # on the stream: no host synchronisation inside the timed region
            events.append(timed(env.torch, lambda: fn(i)))
        env.barrier()
        self.group.check_status()
        own = [a.elapsed_time(b) for a, b in events]
        # the other statistic: every rank's own mean step, then the largest of them
        self.rank_mean_max_ms = max(env.max_each([sum(own) / len(own)]))
        return env.max_each(own)  # per step: the slowest rank

    def parity(self, microbatches, tag):
        """One checked step per listed microbatch: plan and routing against the oracle, replica bytes
        against the seeded masters, with the slots randomised first."""
        env = self.env
        ok = {"plan": True, "routing": True, "sync_bytes": True}
        for mb in microbatches:
            env.barrier()
            before = randomise_replicas(env, self.group, self.ranks) if self.with_weights else None
            env.barrier()
            layer = mb % self.num_layers
            self.step(mb, layer=layer)
            env.barrier()
            self.group.check_status()
            p, r, plans = check_plan_and_routing(env, self.cfg, self.group, self.ranks, layer,
                                                 self.ids_dev[mb % len(self.ids_dev)], self.phys_dev, f"{tag} mb{mb}")
            ok["plan"] &= p
            ok["routing"] &= r
            if self.with_weights:
                ok["sync_bytes"] &= check_replica_bytes(env, self.cfg, self.group, self.ranks, self.masters, plans,
                                                        before[0], before[1], f"{tag} mb{mb}")
            self.last_plans = plans
        return {k: env.all_true(v) for k, v in ok.items()}

    def breakdown(self, n):
        """Each operation queued right behind the L2 flush (no host synchronisation in between), so its
        events bracket the kernels, not the latency of a launch into an idle GPU. Per launch: slowest rank."""
        from oracle import uep_oracle as O  # link volumes are computed from the oracle's plan of the same routing

        env, g, torch = self.env, self.group, self.env.torch
        comm = g.comm_stream()
        plan_ms, sync_ms, reroute_ms, vols = [], [], [], []
        for i in range(n):
            layer = i % self.num_layers
            ids = self.ids_dev[i % len(self.ids_dev)]
            env.barrier()
            env.flush_l2()
            a, b = timed(torch, lambda: g.update_placement(layer, ids))
            env.barrier()
            plan_ms.append(a.elapsed_time(b))
            if self.with_weights:
                # weight_sync is timed right behind a plan issued on the same (communication) stream: the
                # plan's load exchange has just lined the ranks up, and there is no cross-stream hand-over
                t = self.masters.tables
                with torch.cuda.stream(comm):
                    env.flush_l2()
                    g.update_placement(layer, ids)
                    a, b = timed(torch, lambda: g.weight_sync(layer, t[0], t[1], t[2], t[3]), stream=comm)
                env.barrier()
                sync_ms.append(a.elapsed_time(b))
                vols.append(self.volumes(layer))
            env.flush_l2()
            a, b = timed(torch, lambda: g.reroute_sparse(layer, ids, self.phys_dev))
            env.barrier()
            reroute_ms.append(a.elapsed_time(b))
        g.check_status()
        return env.max_each(plan_ms), env.max_each(sync_ms), env.max_each(reroute_ms), vols

    def volumes(self, layer):
        """Per hosted rank: experts sent / received by the weight_sync of the plan stored under `layer`."""
        from oracle import uep_oracle as O
        from ultra_ep_b200 import capi

        g = self.group
        plan = O.Plan(*(g.buffer(0, b)[layer].cpu().numpy() for b in
                        (capi.BUF_P2L, capi.BUF_L2P, capi.BUF_LCNTS, capi.BUF_QUOTA, capi.BUF_QUOTA_PREFIX,
                         capi.BUF_RANK_QUOTA_PREFIX)))
        rel = relay_selection(self.cfg, plan, self.args.plan_mode_resolved, self.args.relay_min_replicas)
        return link_volumes(self.cfg, plan, self.ranks, rel)

    def close(self):
        self.group.destroy()
        self.group = None
        self.masters = None
        self.env.torch.cuda.empty_cache()


def sync_roofline(env, fw, sync_ms, vols, peak_hbm, peak_src, link):
    """Roofline of weight_sync_kernel over the timed launches."""
    cfg = fw.cfg
    eb = cfg.expert_bytes
    total_ms = sum(sync_ms)
    n = max(len(sync_ms), 1)
    if env.world == 1:
        rd = sum(sum(v["reads"] for v in launch) for launch in vols) * eb
        wr = sum(sum(v["writes"] for v in launch) for launch in vols) * eb
        ach = (rd + wr) / 1e9 / (total_ms / 1e3) if total_ms else 0.0
        return {"kernel": "weight_sync_kernel", "bound": "hbm", "achieved": round(ach, 1), "peak": peak_hbm, "unit": "GB/s",
                "frac": round(ach / peak_hbm, 4),
                "traffic": int((rd + wr) / n * NCU_SYNC_TRAFFIC_RATIO) if cfg.name == "cfg3_qwen3_235b_fp8" else None,
                "traffic_source": "recorded one-pass ncu capture (dram__bytes_read.sum + dram__bytes_write.sum) of a "
                                  "full-size launch of this kernel, as a fixed ratio of the algorithmic bytes; not "
                                  "measured in this run",
                "algorithmic_bytes_per_launch": int((rd + wr) / n), "peak_source": peak_src + "; of measured",
                "note": "simulated EP: peers are same-device buffers, bytes = reads + writes through HBM"}
    # per launch: the busiest GPU's link bytes (the larger of what it sends and what it receives)
    mine = [max(v[0]["egress"], v[0]["ingress"]) * eb for v in vols]
    busiest = env.max_each(mine)
    ach = sum(busiest) / 1e9 / (total_ms / 1e3) if total_ms else 0.0
    out = {"kernel": "weight_sync_kernel", "bound": "nvlink", "achieved": round(ach, 1), "peak": NVLINK_NOMINAL_GBS,
           "unit": "GB/s", "frac": round(ach / NVLINK_NOMINAL_GBS, 4), "traffic": None,
           "algorithmic_bytes_per_launch": int(sum(busiest) / n),
           "peak_source": "nominal NVLink 5 bandwidth per direction per GPU; the link as measured in this run is in peak_measured",
           "note": "per launch: bytes = max(egress, ingress) of the busiest GPU, time = slowest rank; summed over launches"}
    if link:
        out["peak_measured"] = link
        best = max(link.get("copy_engine_gbs") or 0.0, link.get("kernel_gbs") or 0.0)
        if best > 0:
            out["frac_of_measured"] = round(ach / best, 4)
    return out


def link_probe(env, group, cfg):
    """One-directional peer copy rank 0 -> rank 1 through the arena's replica buffer, others idle."""
    import ctypes as C

    from ultra_ep_b200 import capi

    region = cfg.redundant * (cfg.fc1_numel + cfg.fc2_numel) * cfg.weight_elem_bytes
    nbytes = min(region, 256 << 20) // 16 * 16
    res = {"bytes": int(nbytes), "pair": "rank 0 -> rank 1, one direction, other ranks idle"}
    for key, use_kernel in (("copy_engine_gbs", 0), ("kernel_gbs", 1)):
        env.barrier()
        val = None
        if env.rank == 0:
            ms = C.c_float(0)
            capi.check(group.lib.uep_debug_link_probe(group.handle, 1, nbytes, 10, use_kernel, C.byref(ms)), "uep_debug_link_probe")
            val = round(nbytes / 1e9 / (ms.value / 1e3), 1)
        env.barrier()
        res[key] = val
    res["how"] = ("10 back-to-back copies after one warm-up, CUDA events on the communication stream: cudaMemcpyAsync "
                  "to the cudaIpc-mapped peer buffer (copy engine) and a plain 16-byte load/store kernel")
    return res


# ------------------------------------------------------------------------------------------
# the reference's own sm_100 kernels on the same plans, masters and peer memory
# ------------------------------------------------------------------------------------------
def ref_sm100(env, fw, args):
    """Reference kernels (built unmodified into oracle/_ref), per rank, on the plans the new kernels just
    made: histogram + reduce + solve (without its NVSHMEM all-gather, which this build has not), task build
    + thread-copy kernel (the path the reference takes when the NVLink domain has at most 8 ranks) writing
    into the same replica slots over the same peer mappings, sparse and dense reroute. At N = 1 the hosted
    ranks run one after another and the figures are per rank (largest and mean over the ranks)."""
    import ctypes as C

    try:
        from oracle import uep_ref
        from ultra_ep_b200 import capi
        from ultra_ep_b200 import workloads as W

        torch = env.torch
        if not uep_ref.available():
            return {"unavailable": "oracle/_ref/libuep_ref.so not present"}
        cfg, g, ranks = fw.cfg, fw.group, fw.ranks
        N, M, R, L = cfg.ep, cfg.masters, cfg.redundant, cfg.num_experts
        P, D = N * (M + R), N
        lib = uep_ref.lib()
        dev = env.dev

        def peer_ptr(li, p, buf):
            out = C.c_void_p()
            capi.check(g.lib.uep_manager_peer_buffer(g.handle, li, p, buf, C.byref(out)), "uep_manager_peer_buffer")
            return out.value or 0

        spaces = [uep_ref.Workspace(r, N, M, R, cfg.fc1_numel, cfg.fc2_numel, cfg.weight_elem_bytes, 1,
                                    cfg.fc1_scale_numel, cfg.fc2_scale_numel, N,
                                    [peer_ptr(li, p, capi.BUF_REPLICA_WEIGHT) for p in range(N)],
                                    [peer_ptr(li, p, capi.BUF_REPLICA_SCALE) for p in range(N)], None)
                  for li, r in enumerate(ranks)]
        rep_w = [g.buffer(li, capi.BUF_REPLICA_WEIGHT) for li in range(len(ranks))]
        rep_s = [g.buffer(li, capi.BUF_REPLICA_SCALE) for li in range(len(ranks))]
        empty = torch.empty(0, dtype=torch.int64, device=dev)
        tabs = fw.masters.tables
        stream = torch.cuda.current_stream().cuda_stream
        n = min(args.steps, 8)
        res = {k: [] for k in ("plan", "weight_sync", "reroute_sparse", "reroute_dense")}
        ok_bytes = True
        for i in range(3 + n):
            mb = i % len(fw.ids_dev)
            layer = mb % fw.num_layers
            ids32 = fw.ids_dev[mb]
            ids64 = [x.long() for x in ids32]
            g.update_placement(layer, ids32)  # our plan storage has the reference's layout: its kernels read it
            env.barrier()
            plans = [g.plan(li, layer) for li in range(len(ranks))]
            per = {k: [] for k in res}
            for li, r in enumerate(ranks):
                # plan: histogram, reduce, solve (the all-gathered matrix is taken from our exchange)
                lpr = g.buffer(li, capi.BUF_LOADS_PER_RANK).clone()
                gl = torch.zeros(L, dtype=torch.int32, device=dev)
                out = {k: torch.empty_like(v) for k, v in plans[li].items()}
                env.flush_l2()

                def plan_fn():
                    lib.uep_ref_topk_local_sum(ids64[li].data_ptr(), cfg.tokens_per_rank, cfg.topk, L, lpr[r].data_ptr(), stream)
                    lib.uep_ref_reduce_per_rank_loads(lpr.data_ptr(), gl.data_ptr(), N, L, stream)
                    lib.uep_ref_solve_placement(gl.data_ptr(), lpr.data_ptr(), out["p2l"].data_ptr(), out["l2p"].data_ptr(),
                                                out["lcnts"].data_ptr(), out["quota"].data_ptr(), out["quota_prefix"].data_ptr(),
                                                out["rank_quota_prefix"].data_ptr(), stream, L, N, M, R, N, D, 1.0, 1024, 0, 1,
                                                0.01, 1, r)
                a, b = timed(torch, plan_fn)
                torch.cuda.synchronize()
                per["plan"].append(a.elapsed_time(b))
                # sparse reroute (in place, atomic ordinals) and dense reroute (zero-fill + two kernels)
                work = ids64[li].clone()
                counters = torch.zeros(L, dtype=torch.int32, device=dev)
                env.flush_l2()
                a, b = timed(torch, lambda: lib.uep_ref_sparse_reroute_quota(
                    work.data_ptr(), plans[li]["l2p"].data_ptr(), plans[li]["lcnts"].data_ptr(),
                    plans[li]["rank_quota_prefix"].data_ptr(), counters.data_ptr(), cfg.tokens_per_rank, cfg.topk, L, D, stream))
                torch.cuda.synchronize()
                per["reroute_sparse"].append(a.elapsed_time(b))
                rmap = torch.zeros((cfg.tokens_per_rank, L), dtype=torch.bool, device=dev)
                rmap.scatter_(1, ids64[li], True)
                probs = torch.rand(rmap.shape, dtype=torch.float32, device=dev) * rmap
                env.flush_l2()
                a, b = timed(torch, lambda: uep_ref.dense_reroute_forward(
                    rmap, probs, plans[li]["l2p"], plans[li]["lcnts"], plans[li]["rank_quota_prefix"], P, True))
                torch.cuda.synchronize()
                per["reroute_dense"].append(a.elapsed_time(b))
            # weight_sync: every rank's launch pair, then a host barrier (the kernel has no completion wait)
            before = randomise_replicas(env, g, ranks) if i == 3 + n - 1 else None
            env.barrier()
            for li, r in enumerate(ranks):
                env.flush_l2()
                a, b = timed(torch, lambda: spaces[li].weight_sync(
                    plans[li]["p2l"], plans[li]["l2p"], plans[li]["lcnts"], tabs[0][li], tabs[1][li],
                    tabs[2][li] if tabs[2] is not None else empty, tabs[3][li] if tabs[3] is not None else empty,
                    rep_w[li], rep_s[li], stream))
                torch.cuda.synchronize()
                per["weight_sync"].append(a.elapsed_time(b))
            env.barrier()
            if before is not None:  # the bytes the reference's kernel delivered, checked like ours
                ids_all = env.gather_ids(ids32)
                oplans = oracle_plans(cfg, ids_all, ranks)
                ok_bytes = check_replica_bytes(env, cfg, g, ranks, fw.masters, oplans, before[0], before[1], "ref_sm100 weight_sync")
            if i >= 3:
                for k in res:
                    res[k].append(per[k])
        for ws in spaces:
            ws.close()
        out = {"unit": "us", "launches": n}
        for k, rows in res.items():
            worst = env.max_each([max(row) for row in rows])  # per launch: the slowest rank
            out[k] = round(sum(worst) / len(worst) * 1e3, 2)
            if env.world == 1:
                out[k + "_mean_over_ranks"] = round(sum(sum(row) / len(row) for row in rows) / len(rows) * 1e3, 2)
        out["weight_sync_bytes_ok"] = env.all_true(ok_bytes)
        out["exposed_total"] = round(out["plan"] + max(out["weight_sync"], out["reroute_sparse"]), 2)
        out["note"] = ("reference kernels compiled from its sources for sm_100, one rank per launch, per-rank figures "
                       "(largest over the ranks); plan = histogram + reduce + solve without its all-gather; weight_sync = "
                       "task build + thread-copy kernel" + (" into peer memory over NVLink" if env.world > 1 else
                                                            " between buffers of one device (HBM)")
                       + "; reroute_dense includes the zero-fill of its outputs, as its host code does per call")
        return out
    except Exception as e:  # the reference build is optional evidence, never a reason to fail the bench
        return {"unavailable": f"{type(e).__name__}: {e}"}


# ------------------------------------------------------------------------------------------
# the drop-in Manager (pybind `_C` + Python surface) at full size, N > 1
# ------------------------------------------------------------------------------------------
def manager_section(env, cfg, args, pool):
    from oracle import uep_oracle as O
    from ultra_ep_b200 import Manager
    from ultra_ep_b200 import workloads as W

    torch, dist, dev = env.torch, env.dist, env.dev
    N, M, R, L = cfg.ep, cfg.masters, cfg.redundant, cfg.num_experts
    P = N * (M + R)
    os.environ["ULTRA_EP_WEIGHT_SYNC_PLAN_MODE"] = {0: "direct", 1: "adaptive", 2: "force_relay"}[args.plan_mode_resolved]
    mgr = Manager(dist.group.WORLD, 1, M, R, cfg.fc1_numel, cfg.fc2_numel, is_train=False, explicitly_destroy=True,
                  weight_data_dtype=torch.uint8 if cfg.weight_elem_bytes == 1 else torch.bfloat16,
                  weight_scale_dtype=torch.uint8, expert_fc1_weight_scale_numel=cfg.fc1_scale_numel,
                  expert_fc2_weight_scale_numel=cfg.fc2_scale_numel)
    r = env.rank
    wdt = torch.uint8 if cfg.weight_elem_bytes == 1 else torch.bfloat16
    sizes = [cfg.fc1_numel * cfg.weight_elem_bytes, cfg.fc2_numel * cfg.weight_elem_bytes, cfg.fc1_scale_numel, cfg.fc2_scale_numel]
    mine = [[seeded_bytes(torch, dev, master_key(cfg, r * M + m, s), sizes[s]) for m in range(M)] for s in range(4)]
    as_w = lambda t: t.view(wdt)
    mgr.construct_local_master_ptr_pool(1, [as_w(t) for t in mine[0]], [as_w(t) for t in mine[1]], None, None,
                                        mine[2] if sizes[2] else None, mine[3] if sizes[3] else None)
    T, K = cfg.tokens_per_rank, cfg.topk
    ids_host = [torch.from_numpy(W.routing_ids(cfg, r, microbatch=mb).astype(np.int64)).pin_memory() for mb in range(pool)]
    ids_dev = [h.to(dev) for h in ids_host]
    maps = [torch.zeros((T, L), dtype=torch.bool, device=dev).scatter_(1, x, True) for x in ids_dev]
    probs = [torch.rand((T, L), dtype=torch.float32, device=dev) * m for m in maps]
    maps_host = [m.cpu().pin_memory() for m in maps]
    probs_host = [p.cpu().pin_memory() for p in probs]
    stage_ids = torch.empty_like(ids_dev[0])
    out_ids_host = torch.empty_like(ids_host[0]).pin_memory()
    stage_map, stage_probs = torch.empty_like(maps[0]), torch.empty_like(probs[0])
    out_map_host = torch.empty((T, P), dtype=torch.bool).pin_memory()
    out_probs_host = torch.empty((T, P), dtype=torch.float32).pin_memory()

    def sparse_e2e(i):
        stage_ids.copy_(ids_host[i % pool], non_blocking=True)
        vid = mgr.allocate_microbatch_slot(1)
        mgr.update_placement_sparse(vid, stage_ids)
        ev = mgr.weight_sync(vid, async_finish=True)
        mgr.reroute_sparse(vid, stage_ids)  # in place; waits for the plan made on the communication stream
        out_ids_host.copy_(stage_ids, non_blocking=True)
        ev.current_stream_wait()

    def dense_step(i, rmap=None, pr=None):
        rmap = maps[i % pool] if rmap is None else rmap
        pr = probs[i % pool] if pr is None else pr
        vid = mgr.allocate_microbatch_slot(1)
        mgr.update_placement(vid, rmap)
        ev = mgr.weight_sync(vid, async_finish=True)
        out = mgr.reroute(vid, pr, rmap)
        ev.current_stream_wait()
        return out

    def dense_e2e(i):
        stage_map.copy_(maps_host[i % pool], non_blocking=True)
        stage_probs.copy_(probs_host[i % pool], non_blocking=True)
        ep, em = dense_step(i, stage_map, stage_probs)
        out_probs_host.copy_(ep, non_blocking=True)
        out_map_host.copy_(em, non_blocking=True)

    def run(fn, steps):
        for i in range(3):
            env.flush_l2()
            fn(i)
        env.barrier()
        mgr.check_status()
        evs = []
        for i in range(steps):
            env.flush_l2()
            evs.append(timed(torch, lambda: fn(i)))
        env.barrier()
        mgr.check_status()
        return env.max_each([a.elapsed_time(b) for a, b in evs])

    res = {"api": "ultra_ep_b200.Manager over the pybind module _C (the reference's Manager surface)"}
    sparse = run(sparse_e2e, args.steps)
    res["sparse_e2e"] = stats_us(sparse)
    res["sparse_e2e"]["h2d_bytes_per_step"] = ids_host[0].numel() * 8
    res["sparse_e2e"]["d2h_bytes_per_step"] = ids_host[0].numel() * 8
    res["dense_step_device_resident"] = stats_us(run(dense_step, args.steps))
    dense = run(dense_e2e, min(args.steps, 16))
    res["dense_e2e"] = stats_us(dense)
    res["dense_e2e"]["h2d_bytes_per_step"] = T * L * 5
    res["dense_e2e"]["d2h_bytes_per_step"] = T * P * 5
    # parity of one dense step through the Manager: plan, expanded outputs, replica bytes
    mb = 0
    mgr.local_replica_weight_buffer.view(torch.uint8).random_(0, 256)
    if sizes[2]:
        mgr.local_replica_weight_scale_buffer_raw.random_(0, 256)
    before_w = mgr.local_replica_weight_buffer.view(torch.uint8).clone()
    env.barrier()
    ep, em = dense_step(mb)
    env.barrier()
    mgr.check_status()
    parts = [torch.empty((T, K), dtype=torch.int64, device=dev) for _ in range(N)]
    dist.all_gather(parts, ids_dev[mb])
    lpr = np.stack([np.bincount(p.cpu().numpy().reshape(-1), minlength=L) for p in parts]).astype(np.int32)
    plan = O.solve_placement(lpr, M, R, N, r)
    vid = 1  # real layer 1, max_microbatches 1
    got = {"p2l": mgr.physical_to_logical_map[vid], "l2p": mgr.logical_to_physical_map[vid], "lcnts": mgr.logical_replica_counts[vid],
           "quota": mgr.logical_instance_quota[vid], "quota_prefix": mgr.logical_instance_quota_prefix[vid],
           "rank_quota_prefix": mgr.rank_quota_prefix[vid]}
    ok = True
    for f, v in plan.fields().items():
        ok &= env.check(f"manager: plan field {f}", np.array_equal(got[f].cpu().numpy(), v))
    o_probs, o_map = O.dense_reroute_forward(maps[mb].cpu().numpy(), probs[mb].cpu().numpy(), plan, P, True)
    ok &= env.check("manager: expanded routing map", np.array_equal(em.cpu().numpy(), o_map))
    ok &= env.check("manager: expanded probabilities", np.array_equal(ep.cpu().numpy().view(np.uint32), o_probs.view(np.uint32)))
    Lp = M + R
    w_now = mgr.local_replica_weight_buffer.view(torch.uint8)
    for slot in range(R):
        l = int(plan.p2l[r * Lp + M + slot])
        if l < 0:
            ok &= env.check(f"manager: unused slot {slot} written", torch.equal(w_now[slot], before_w[slot]))
        else:
            ok &= env.check(f"manager: fc1 bytes in slot {slot}", torch.equal(w_now[slot, :sizes[0]], seeded_bytes(torch, dev, master_key(cfg, l, 0), sizes[0])))
            ok &= env.check(f"manager: fc2 bytes in slot {slot}", torch.equal(w_now[slot, sizes[0]:], seeded_bytes(torch, dev, master_key(cfg, l, 1), sizes[1])))
            if sizes[2]:
                ok &= env.check(f"manager: fc1 scales in slot {slot}",
                                torch.equal(mgr.local_replica_fc1_weight_scale_buffer[slot], seeded_bytes(torch, dev, master_key(cfg, l, 2), sizes[2])))
    res["parity"] = env.all_true(ok)
    mgr.destroy()
    del mine
    torch.cuda.empty_cache()
    return res, sparse


# ------------------------------------------------------------------------------------------
# backward path
# ------------------------------------------------------------------------------------------
class Backward:
    """Gradients of one training group: master gradients of the hosted ranks (fp32, seeded per expert) and the
    replica gradient slots (seeded per physical slot), so that the fixed-order sums can be rebuilt anywhere."""

    def __init__(self, env, cfg, group, ranks):
        torch = env.torch
        self.env, self.cfg, self.group, self.ranks = env, cfg, group, ranks
        M = cfg.masters
        self.g1 = [torch.empty((M, cfg.fc1_numel), dtype=torch.float32, device=env.dev).normal_(0, 1e-4) for _ in ranks]
        self.g2 = [torch.empty((M, cfg.fc2_numel), dtype=torch.float32, device=env.dev).normal_(0, 1e-4) for _ in ranks]
        self.t1 = group.pointer_tables([[g[m] for m in range(M)] for g in self.g1])
        self.t2 = group.pointer_tables([[g[m] for m in range(M)] for g in self.g2])

    def fill_replicas(self, plan, salt):
        """Used replica slots get seeded N(0, 1e-4) values (not exactly summable: the order is really pinned);
        unused slots a sentinel. Returns copies of what was there."""
        from ultra_ep_b200 import capi

        torch, cfg = self.env.torch, self.cfg
        M, R = cfg.masters, cfg.redundant
        Lp = M + R
        numel = cfg.fc1_numel + cfg.fc2_numel
        for li, r in enumerate(self.ranks):
            rep = self.group.buffer(li, capi.BUF_REPLICA_GRAD)
            for slot in range(R):
                phys = r * Lp + M + slot
                if int(plan.p2l[phys]) >= 0:
                    rep[slot].copy_(seeded_normal(torch, self.env.dev, salt * 100003 + phys, numel, 1e-4))
                else:
                    rep[slot].fill_(float(slot + 1))

    def check_reduce(self, plan, salt, before1, before2, tag):
        """master == ((master + g_1) + g_2) + ... in plan slot order, bit for bit; used replica slots zero."""
        from ultra_ep_b200 import capi

        torch, cfg, env = self.env.torch, self.cfg, self.env
        M, R = cfg.masters, cfg.redundant
        Lp = M + R
        numel = cfg.fc1_numel + cfg.fc2_numel
        ok = True
        for li, r in enumerate(self.ranks):
            for m in range(M):
                l = r * M + m
                c = int(plan.lcnts[l])
                if c <= 1:
                    continue
                e1, e2 = before1[li][m].clone(), before2[li][m].clone()
                for j in range(1, c):
                    g = seeded_normal(torch, env.dev, salt * 100003 + int(plan.l2p[l, j]), numel, 1e-4)
                    e1 += g[:cfg.fc1_numel]
                    e2 += g[cfg.fc1_numel:]
                ok &= env.check(f"{tag}: reduced fc1 gradient of expert {l}", torch.equal(self.g1[li][m].view(torch.int32), e1.view(torch.int32)))
                ok &= env.check(f"{tag}: reduced fc2 gradient of expert {l}", torch.equal(self.g2[li][m].view(torch.int32), e2.view(torch.int32)))
            rep = self.group.buffer(li, capi.BUF_REPLICA_GRAD)
            for slot in range(R):
                if int(plan.p2l[r * Lp + M + slot]) >= 0:
                    ok &= env.check(f"{tag}: replica gradient slot {slot} of rank {r} not zeroed", not bool(rep[slot].any()))
                else:
                    ok &= env.check(f"{tag}: unused replica gradient slot {slot} of rank {r} written",
                                    bool((rep[slot] == float(slot + 1)).all()))
        return ok

    def snapshot(self, plan):
        """Copies of the master gradients that have replicas (the others are not touched)."""
        cfg = self.cfg
        M = cfg.masters
        b1, b2 = [], []
        for li, r in enumerate(self.ranks):
            b1.append({m: self.g1[li][m].clone() for m in range(M) if int(plan.lcnts[r * M + m]) > 1})
            b2.append({m: self.g2[li][m].clone() for m in range(M) if int(plan.lcnts[r * M + m]) > 1})
        return b1, b2

    def reduce_volumes(self, plan):
        cfg = self.cfg
        M, R, N = cfg.masters, cfg.redundant, cfg.ep
        numel = cfg.fc1_numel + cfg.fc2_numel
        p2l = plan.p2l.reshape(N, M + R)
        hbm = link = 0
        for r in self.ranks:
            mine = plan.lcnts[r * M:(r + 1) * M]
            n_rep = int((mine - 1).clip(min=0).sum())
            hbm += int((mine > 1).sum()) * 8 * numel + n_rep * 8 * numel  # masters read+written; replicas read+zeroed
            used = int((p2l[r, M:] >= 0).sum())
            link = max(link, n_rep * 4 * numel, used * 4 * numel)
        return hbm, link


def run_backward(env, args, peak_hbm, link):
    """Backward balancing path of the cfg-4 layer: the fp32 Wgrad reduce of the replicas into their masters
    (checked bit for bit at full size), the token-gradient row gather ([T*K, hidden] bf16, physical-expert
    order back to (token,k) order) and the dense reroute forward/backward."""
    from oracle import uep_oracle as O
    from ultra_ep_b200 import capi
    from ultra_ep_b200 import workloads as W

    torch, dev = env.torch, env.dev
    lib = capi.lib()
    base = W.CONFIGS["cfg4_qwen3_235b_bwd"]
    cfg = base.with_ep(env.world) if env.world > 1 else base
    N, M, R, L = cfg.ep, cfg.masters, cfg.redundant, cfg.num_experts
    P = N * (M + R)
    group, ranks = make_group(env, cfg, 1, True, args)
    ids = [torch.from_numpy(W.routing_ids(cfg, r)).to(dev) for r in ranks]
    group.update_placement(0, ids)
    phys = group.reroute_sparse(0, ids)
    env.barrier()
    plans = oracle_plans(cfg, env.gather_ids(ids), ranks)
    plan = plans[ranks[0]]
    reps = 6
    out = {"workload": f"{cfg.name}: backward of the same layer, " + ("EP8 simulated on one GPU" if env.world == 1 else f"EP{env.world}")}

    # -- Wgrad reduce ------------------------------------------------------------------------
    bw = Backward(env, cfg, group, ranks)
    hbm_bytes, link_bytes = bw.reduce_volumes(plan)
    comm = group.comm_stream()
    red = []
    ok_reduce = True
    for it in range(3 + reps):
        bw.fill_replicas(plan, salt=it)
        b1, b2 = bw.snapshot(plan) if it in (0, 3 + reps - 1) else (None, None)
        env.barrier()
        with torch.cuda.stream(comm):
            env.flush_l2()
            a, b = timed(torch, lambda: group.grad_reduce(0, bw.t1, bw.t2), stream=comm)
        env.barrier()
        if it >= 3:
            red.append(a.elapsed_time(b))
        if b1 is not None:  # first and last launch: the full-size result against the fixed-order sum
            ok_reduce &= bw.check_reduce(plan, it, b1, b2, f"cfg4 grad_reduce launch {it}")
    group.check_status()
    red = env.max_each(red)
    red_ms = sum(red) / len(red)
    out["grad_reduce_us"] = round(red_ms * 1e3, 1)
    out["grad_reduce_parity"] = env.all_true(ok_reduce)
    if env.world == 1:
        ach = hbm_bytes / 1e9 / (red_ms / 1e3)
        out["grad_reduce_roofline"] = {"kernel": "grad_reduce_kernel", "bound": "hbm", "achieved": round(ach, 1), "peak": peak_hbm,
                                       "unit": "GB/s", "frac": round(ach / peak_hbm, 4), "algorithmic_bytes_per_launch": hbm_bytes,
                                       "ctas": 8 * min(args.reduce_sms, lib.uep_manager_num_sms(group.handle) // 8),
                                       "note": "simulated EP: masters read+written, replicas read+zeroed, all through HBM; "
                                               "ctas = all eight hosted ranks' CTAs of the one launch"}
    else:
        busiest = max(env.max_each([float(link_bytes)]))
        ach = busiest / 1e9 / (red_ms / 1e3)
        rl = {"kernel": "grad_reduce_kernel", "bound": "nvlink", "achieved": round(ach, 1), "peak": NVLINK_NOMINAL_GBS, "unit": "GB/s",
              "frac": round(ach / NVLINK_NOMINAL_GBS, 4), "algorithmic_bytes_per_launch": int(busiest), "ctas": args.reduce_sms,
              "note": "bytes = replica gradients the busiest GPU pulls in over NVLink (used replica slots are cleared by the rank that hosts them, locally)"}
        if link:
            best = max(link.get("copy_engine_gbs") or 0.0, link.get("kernel_gbs") or 0.0)
            if best > 0:
                rl["frac_of_measured"] = round(ach / best, 4)
        out["grad_reduce_roofline"] = rl
    del bw
    torch.cuda.empty_cache()

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
        env.barrier()
        env.flush_l2()
        a, b = timed(torch, lambda: capi.check(lib.uep_dispatch_positions(
            phys[0].data_ptr(), rows, P, pos.data_ptr(), offs.data_ptr(), scratch.data_ptr(), st), "uep_dispatch_positions"))
        c, d = timed(torch, lambda: capi.check(lib.uep_gather_rows(
            src.data_ptr(), pos.data_ptr(), dst.data_ptr(), rows, rows, H * 2, status.data_ptr(), st), "uep_gather_rows"))
        env.barrier()
        if it >= 3:
            pos_t.append(a.elapsed_time(b))
            gat_t.append(c.elapsed_time(d))
    ok_gather = env.check("cfg4 gather_rows: status word", int(status[0].item()) == 0)
    ok_gather &= env.check("cfg4 gather_rows: rows", torch.equal(dst, src[pos.long()]))
    gat = env.max_each(gat_t)
    gat_ms = sum(gat) / len(gat)
    gbytes = 2 * rows * H * 2
    ach = gbytes / 1e9 / (gat_ms / 1e3)
    out["dispatch_positions_us"] = round(max(env.max_each([sum(pos_t) / len(pos_t)])) * 1e3, 1)
    out["gather_rows_us"] = round(gat_ms * 1e3, 1)
    out["gather_rows_parity"] = env.all_true(ok_gather)
    out["gather_rows_roofline"] = {"kernel": "gather_rows_kernel", "bound": "hbm", "achieved": round(ach, 1), "peak": peak_hbm,
                                   "unit": "GB/s", "frac": round(ach / peak_hbm, 4), "algorithmic_bytes_per_launch": gbytes,
                                   "note": f"[{rows},{H}] bf16 rows read once and written once, one rank per launch"}
    del src, dst

    # -- dense reroute forward / backward (probabilities) --------------------------------------
    maps = [torch.from_numpy(W.ids_to_map(x.cpu().numpy(), L)).to(dev) for x in ids]
    probs = [torch.rand(m.shape, dtype=torch.float32, device=dev) * m for m in maps]
    ex_probs, ex_maps = group.reroute_dense(0, maps, probs)
    fwd = []
    for it in range(3 + reps):
        env.barrier()
        env.flush_l2()
        a, b = timed(torch, lambda: group.reroute_dense(0, maps, probs, out=(ex_probs, ex_maps)))
        env.barrier()
        if it >= 3:
            fwd.append(a.elapsed_time(b))
    ok_dense = True
    for li, r in enumerate(ranks):
        o_probs, o_map = O.dense_reroute_forward(maps[li].cpu().numpy(), probs[li].cpu().numpy(), plans[r], P, True)
        ok_dense &= env.check(f"cfg4 dense reroute forward: map of rank {r}", np.array_equal(ex_maps[li].cpu().numpy(), o_map))
        ok_dense &= env.check(f"cfg4 dense reroute forward: probabilities of rank {r}",
                              np.array_equal(ex_probs[li].cpu().numpy().view(np.uint32), o_probs.view(np.uint32)))
    fwd = env.max_each(fwd)
    fwd_ms = sum(fwd) / len(fwd)
    T_ = cfg.tokens_per_rank
    fwd_bytes = len(ranks) * T_ * (L + P * 5 + cfg.topk * 4)  # bool map + routed probabilities in; bool map + fp32 probabilities out, once
    out["dense_reroute_forward_us"] = round(fwd_ms * 1e3, 1)
    out["dense_reroute_forward_per_rank_us"] = round(fwd_ms * 1e3 / (1 if env.world > 1 else 1), 1) if env.world > 1 else None
    out["dense_reroute_forward_parity"] = env.all_true(ok_dense)
    out["dense_reroute_forward_roofline"] = {"kernel": "dense_count_kernel + dense_scatter_kernel", "bound": "hbm",
                                             "achieved": round(fwd_bytes / 1e9 / (fwd_ms / 1e3), 1), "peak": peak_hbm, "unit": "GB/s",
                                             "frac": round(fwd_bytes / 1e9 / (fwd_ms / 1e3) / peak_hbm, 4),
                                             "algorithmic_bytes_per_launch": fwd_bytes,
                                             "note": ("two launches (tile counts, scatter), the second a programmatic dependent launch; "
                                                      + ("one rank per GPU" if env.world > 1 else "all eight hosted ranks in one launch pair")
                                                      + "; latency-bound at this size (about 12 MB per rank)")}
    grads = [torch.rand_like(p_) for p_ in ex_probs]
    bwd = []
    for it in range(3 + reps):
        env.barrier()
        env.flush_l2()
        a, b = timed(torch, lambda: group.reroute_dense_backward(0, grads, maps, ex_maps))
        env.barrier()
        if it >= 3:
            bwd.append(a.elapsed_time(b))
    bwd = env.max_each(bwd)
    out["dense_reroute_backward_us"] = round(sum(bwd) / len(bwd) * 1e3, 1)
    group.check_status()
    group.destroy()
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------
# the other configurations
# ------------------------------------------------------------------------------------------
def config_forward(env, args, name, peak_hbm, peak_src, link):
    """Forward step of another configuration: same calls, own sizes; one checked step at the end."""
    from ultra_ep_b200 import workloads as W

    base = W.CONFIGS[name]
    cfg = base.with_ep(env.world) if env.world > 1 else base
    steps = min(args.steps, 16)
    pool = pool_size(steps)
    fw = Forward(env, cfg, args, num_layers=4, pool=pool)
    step_ms = fw.run_timed(fw.step, steps, 3)
    plan_ms, sync_ms, reroute_ms, vols = fw.breakdown(min(steps, 8))
    par = fw.parity([0], name)
    out = {"workload": f"{cfg.name}: forward " + ("plan + reroute (no weights)" if not fw.with_weights else "plan + weight_sync + reroute")
                       + (", EP8 simulated" if env.world == 1 else f", EP{env.world}"),
           "experts": cfg.num_experts, "tokens_per_rank": cfg.tokens_per_rank, "redundant_per_rank": cfg.redundant,
           "expert_bytes": cfg.expert_bytes, "step_us": stats_us(step_ms),
           "breakdown_us": {"plan": round(sum(plan_ms) / len(plan_ms) * 1e3, 2),
                            "weight_sync": round(sum(sync_ms) / len(sync_ms) * 1e3, 2) if sync_ms else None,
                            "reroute": round(sum(reroute_ms) / len(reroute_ms) * 1e3, 2)},
           "parity": par}
    if sync_ms:
        out["weight_sync_roofline"] = sync_roofline(env, fw, sync_ms, vols, peak_hbm, peak_src, link)
    fw.close()
    return out


def config5_forward_backward(env, args, peak_hbm, link):
    """cfg 5: forward + backward of the DeepSeek-V3-shaped layer with four microbatch slots in flight: the plans
    of four microbatches are made (and their weights pushed, their tokens rerouted) before the first backward
    re-pushes the weights of its slot and reduces its gradients. One timed unit is the whole 4 + 4 sequence."""
    from ultra_ep_b200 import capi
    from ultra_ep_b200 import workloads as W

    torch = env.torch
    base = W.CONFIGS["cfg5_dsv3_stress"]
    cfg = base.with_ep(env.world) if env.world > 1 else base
    slots = cfg.max_microbatches
    fw = Forward(env, cfg, args, num_layers=slots, pool=slots, is_train=True)
    g = fw.group
    bw = Backward(env, cfg, g, fw.ranks)
    t = fw.masters.tables

    def sequence(_i=0):
        for s in range(slots):  # four forwards: each slot keeps its own plan
            fw.step(s, layer=s)
        for s in reversed(range(slots)):  # four backwards, last microbatch first
            g.weight_sync(s, t[0], t[1], t[2], t[3])
            ev = g.grad_reduce(s, bw.t1, bw.t2, async_finish=True)
            g.wait_event(ev)

    reps = 4
    times = []
    for it in range(2 + reps):
        env.barrier()
        env.flush_l2()
        a, b = timed(torch, sequence)
        env.barrier()
        if it >= 2:
            times.append(a.elapsed_time(b))
    g.check_status()
    times = env.max_each(times)
    # parity: all four slots hold the plan of their own microbatch; routing and bytes of the last forward;
    # one backward at full size against the fixed-order sum
    ok = {"plan": True, "routing": True, "sync_bytes": True, "reduce": True}
    for s in range(slots):
        p, _, plans = check_plan_and_routing(env, cfg, g, fw.ranks, s, fw.ids_dev[s], None, f"cfg5 slot {s}")
        ok["plan"] &= p
    par = fw.parity([slots - 1], "cfg5")
    ok["routing"] &= par["routing"]
    ok["sync_bytes"] &= par["sync_bytes"]
    ok["plan"] &= par["plan"]
    plan = fw.last_plans[fw.ranks[0]]
    bw.fill_replicas(plan, salt=77)
    b1, b2 = bw.snapshot(plan)
    env.barrier()
    g.grad_reduce(slots - 1, bw.t1, bw.t2)
    env.barrier()
    g.check_status()
    ok["reduce"] &= bw.check_reduce(plan, 77, b1, b2, "cfg5 grad_reduce")
    hbm_bytes, link_bytes = bw.reduce_volumes(plan)
    # the reduce alone, for its bandwidth
    red = []
    comm = g.comm_stream()
    for it in range(4):
        env.barrier()
        with torch.cuda.stream(comm):
            env.flush_l2()
            a, b = timed(torch, lambda: g.grad_reduce(slots - 1, bw.t1, bw.t2), stream=comm)
        env.barrier()
        if it >= 1:
            red.append(a.elapsed_time(b))
    red = env.max_each(red)
    red_ms = sum(red) / len(red)
    if env.world == 1:
        rl = {"bound": "hbm", "achieved": round(hbm_bytes / 1e9 / (red_ms / 1e3), 1), "peak": peak_hbm, "unit": "GB/s"}
    else:
        busiest = max(env.max_each([float(link_bytes)]))
        rl = {"bound": "nvlink", "achieved": round(busiest / 1e9 / (red_ms / 1e3), 1), "peak": NVLINK_NOMINAL_GBS, "unit": "GB/s"}
    rl["frac"] = round(rl["achieved"] / rl["peak"], 4)
    out = {"workload": f"{cfg.name}: forward + backward, {slots} microbatch slots in flight"
                       + (", EP8 simulated" if env.world == 1 else f", EP{env.world}"),
           "experts": cfg.num_experts, "tokens_per_rank": cfg.tokens_per_rank, "redundant_per_rank": cfg.redundant,
           "expert_bytes": cfg.expert_bytes, "hot_expert": "present in every token's top-k (12.5 % of all assignments, the most top-8 allows)",
           "sequence_us": stats_us(times), "per_layer_forward_backward_us": round(sum(times) / len(times) * 1e3 / slots, 1),
           "grad_reduce_us": round(red_ms * 1e3, 1), "grad_reduce_roofline": rl,
           "parity": {k: env.all_true(v) for k, v in ok.items()}}
    del bw
    fw.close()
    return out


def ep64_replay(env, args):
    """The reference's own test workload (EP64, 256 experts, 4 masters + 2 redundant slots per rank, top-8,
    8192 tokens per rank, max/mean rank load 1.5 / 2.0 / 3.0) through the stateless solver and the dense reroute
    of one rank on one GPU, next to the reference's kernels on the same inputs. Times are CUDA-event microseconds."""
    import ctypes as C

    from oracle import uep_oracle as O
    from ultra_ep_b200 import capi
    from ultra_ep_b200 import workloads as W

    torch, dev = env.torch, env.dev
    lib = capi.lib()
    N, M, R, K, T = 64, 4, 2, 8, 8192
    L, P, D = N * M, N * (M + R), N
    try:
        from oracle import uep_ref

        ref = uep_ref if uep_ref.available() else None
    except Exception:
        ref = None
    res = {}
    st = torch.cuda.current_stream().cuda_stream
    for ratio in (1.5, 2.0, 3.0):
        lpr_np, ids0 = W.reference_style_loads(N, M, K, T, ratio, seed=33)
        lpr = torch.from_numpy(lpr_np).to(dev)
        out = {k: torch.empty(s, dtype=torch.int32, device=dev) for k, s in
               [("p2l", (P,)), ("l2p", (L, D)), ("lcnts", (L,)), ("quota", (L, D)), ("qp", (L, D)), ("rqp", (L, D))]}
        gl = torch.empty(L, dtype=torch.int32, device=dev)
        status = torch.zeros(2, dtype=torch.int32, device=dev)
        prm = capi.SolverParams.defaults()

        def solve():
            capi.check(lib.uep_solve_placement(lpr.data_ptr(), gl.data_ptr(), out["p2l"].data_ptr(), out["l2p"].data_ptr(),
                                               out["lcnts"].data_ptr(), out["quota"].data_ptr(), out["qp"].data_ptr(),
                                               out["rqp"].data_ptr(), N, N, M, R, D, C.byref(prm), 0, status.data_ptr(), st))
        ts = []
        for it in range(8):
            env.flush_l2()
            a, b = timed(torch, solve)
            torch.cuda.synchronize()
            if it >= 3:
                ts.append(a.elapsed_time(b))
        plan = O.solve_placement(lpr_np, M, R, N, 0)
        ok = all(np.array_equal(out[k].cpu().numpy(), v) for k, v in
                 zip(("p2l", "l2p", "lcnts", "quota", "qp", "rqp"), plan.fields().values()))
        env.check(f"ep64 replay (ratio {ratio}): plan against the oracle", ok)
        rmap = torch.from_numpy(W.ids_to_map(ids0, L)).to(dev)
        probs = torch.rand(rmap.shape, dtype=torch.float32, device=dev) * rmap
        o_map = torch.empty((T, P), dtype=torch.bool, device=dev)
        o_probs = torch.empty((T, P), dtype=torch.float32, device=dev)
        scratch = torch.empty(int(lib.uep_reroute_scratch_elems(T, 0, L)), dtype=torch.int32, device=dev)

        def reroute():
            capi.check(lib.uep_dense_reroute_forward(rmap.data_ptr(), probs.data_ptr(), out["l2p"].data_ptr(), out["lcnts"].data_ptr(),
                                                     out["rqp"].data_ptr(), o_map.data_ptr(), o_probs.data_ptr(), scratch.data_ptr(),
                                                     T, L, P, D, 1, 1, st))
        tr = []
        for it in range(8):
            env.flush_l2()
            a, b = timed(torch, reroute)
            torch.cuda.synchronize()
            if it >= 3:
                tr.append(a.elapsed_time(b))
        e_probs, e_map = O.dense_reroute_forward(rmap.cpu().numpy(), probs.cpu().numpy(), plan, P, True)
        ok_r = np.array_equal(o_map.cpu().numpy(), e_map) and np.array_equal(o_probs.cpu().numpy().view(np.uint32), e_probs.view(np.uint32))
        env.check(f"ep64 replay (ratio {ratio}): dense reroute against the oracle", ok_r)
        rank_loads = lpr_np.sum(0).reshape(N, M).sum(1)
        row = {"initial_imbalance": round(float(rank_loads.max() / rank_loads.mean()), 3),
               "replicas_total": int((plan.lcnts - 1).sum()), "replicas_max_per_expert": int((plan.lcnts - 1).max()),
               "solve_us": round(sum(ts) / len(ts) * 1e3, 2), "dense_reroute_us": round(sum(tr) / len(tr) * 1e3, 2),
               "parity": bool(ok and ok_r)}
        if ref is not None:
            tsr, trr = [], []
            for it in range(8):
                env.flush_l2()
                a, b = timed(torch, lambda: ref.solve_placement(lpr, M, R, my_rank=0))
                torch.cuda.synchronize()
                env.flush_l2()
                c, d = timed(torch, lambda: ref.dense_reroute_forward(rmap, probs, out["l2p"], out["lcnts"], out["rqp"], P, True))
                torch.cuda.synchronize()
                if it >= 3:
                    tsr.append(a.elapsed_time(b))
                    trr.append(c.elapsed_time(d))
            row["reference_solve_us"] = round(sum(tsr) / len(tsr) * 1e3, 2)
            row["reference_dense_reroute_us"] = round(sum(trr) / len(trr) * 1e3, 2)
        res[f"imbalance_{ratio}"] = row
    res["note"] = ("solver through uep_solve_placement (one launch: reduce + solve), dense reroute of rank 0 through "
                   "uep_dense_reroute_forward; reference figures: its solve_placement launcher (output clearing + solver "
                   "kernel, including the allocation of its outputs) and its dense reroute (zero-fill + two kernels) on the same "
                   "GPU and inputs")
    return res


# ------------------------------------------------------------------------------------------
# baselines on the host cores
# ------------------------------------------------------------------------------------------
def cpu_forward_layer(cfg, iters_cap=200, budget_s=10.0, threads=None):
    """The oracle's whole-group forward layer on host threads (plan + reroute + weight copy)."""
    import ctypes as C

    from oracle import uep_oracle as O
    from ultra_ep_b200 import workloads as W

    lib = O.lib()
    N, M, R = cfg.ep, cfg.masters, cfg.redundant
    online = lib.uep_oracle_hardware_threads() or 1
    threads = threads or min(N, online)
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
            "sync_us": parts[2].value / iters * 1e6, "cores_online": online}


def cpu_baseline(cfg, args):
    r = cpu_forward_layer(cfg, budget_s=args.cpu_budget_s)
    return {"value": round(r["us_per_layer"], 1), "unit": UNIT, "cores": r["threads"], "kind": "port",
            "sample": f"{r['iters']} layers of the same {cfg.ep}-rank workload (one host thread per rank: the path has "
                      f"no finer parallelism than its ranks; plan {r['plan_us']:.0f} us, reroute {r['reroute_us']:.0f} us, "
                      f"weight copy {r['sync_us']:.0f} us)",
            "host_threads_online": r["cores_online"]}


def run_reference(args):
    """Reference arm: the reference's logic for this path on host cores (bounded sample)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from ultra_ep_b200 import workloads as W

    base = W.CONFIGS[args.config]
    cfg = base.with_ep(args.gpus) if args.gpus > 1 else base  # the same group shape as the other arm at this N
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
        "config": {"workload": f"{cfg.name}: forward update_placement + weight_sync + reroute, EP{cfg.ep}, all ranks on host threads",
                   "experts": cfg.num_experts, "topk": cfg.topk, "tokens_per_rank": cfg.tokens_per_rank,
                   "redundant_per_rank": cfg.redundant, "expert_bytes": cfg.expert_bytes},
        "cpu_baseline": {"value": round(value, 1), "unit": UNIT, "cores": r["threads"], "kind": "port",
                         "sample": f"{len(per_step)} samples of {r['iters']} layers each; the reference has no CPU "
                                   "implementation of this path, the CPU restatement under oracle/ is timed, one host thread per rank",
                         "host_threads_online": r["cores_online"]},
        "e2e": {"value": round(value, 1), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out))


# ------------------------------------------------------------------------------------------
# small fixed cases of single kernels, for profiler captures (a few hundred MB on the device, a handful of launches)
# ------------------------------------------------------------------------------------------
def run_device_trace(args):
    """Device-side time stamps of weight_sync (and of the plan kernel in front of it) at full size, one rank per GPU or
    EP8 simulated: per rank and launch the CUDA-event time and the kernel's own stamps (set-up done, last copy issued,
    last copy complete, ticket, end). The stamps are a tuning aid of the library (UEP_SYNC_TRACE=1)."""
    os.environ["UEP_SYNC_TRACE"] = "1"
    import ctypes as C  # noqa: F401

    from ultra_ep_b200 import capi
    from ultra_ep_b200 import workloads as W

    env = Env()
    torch = env.torch
    args.plan_mode_resolved = args.plan_mode if args.plan_mode >= 0 else (0 if env.world == 1 else 1)
    base = W.CONFIGS[args.config]
    cfg = base.with_ep(env.world) if env.world > 1 else base
    fw = Forward(env, cfg, args, 2, 10)
    g, t = fw.group, fw.masters.tables
    comm = g.comm_stream()
    rows = []
    for mb in range(10):
        ids = fw.ids_dev[mb]
        for rep in range(2):  # the second launch of a microbatch is the one reported
            env.barrier()
            with torch.cuda.stream(comm):
                env.flush_l2()
                g.update_placement(0, ids)
                a, b = timed(torch, lambda: g.weight_sync(0, t[0], t[1], t[2], t[3]), stream=comm)
            env.barrier()
        buf = np.zeros((1024, 8), np.uint64)
        capi.check(g.lib.uep_debug_sync_trace(g.handle, buf.ctypes.data, 1024))
        st = buf[:512]
        st = st[st[:, 0] > 0].astype(np.int64)
        t0 = st[:, 0].min()
        rel = (st - t0) / 1e3
        vol = fw.volumes(0)
        pl = buf[1000].astype(np.int64)
        rows.append({"microbatch": mb, "rank": env.rank, "event_us": round(a.elapsed_time(b) * 1e3, 1),
                     "egress_experts": [round(float(v["egress"]), 2) for v in vol], "ingress_experts": [v["ingress"] for v in vol],
                     "ctas": int(len(st)), "setup_us": round(float(np.median(rel[:, 1])), 1),
                     "last_copy_complete_us": round(float(rel[:, 3].max()), 1), "last_ticket_us": round(float(rel[:, 5].max()), 1),
                     "end_us": round(float(rel[:, 6].max()), 1),
                     "plan_kernel_us": {"partials": round((pl[0] - pl[5]) / 1e3, 1), "published": round((pl[1] - pl[5]) / 1e3, 1),
                                        "gathered": round((pl[2] - pl[5]) / 1e3, 1), "solved": round((pl[4] - pl[5]) / 1e3, 1)}})
    g.check_status()
    if env.world > 1:
        allrows = [None] * env.world
        env.dist.all_gather_object(allrows, rows)
    else:
        allrows = [rows]
    if env.rank == 0:
        for mb in range(10):
            for r in range(len(allrows)):
                print(json.dumps(allrows[r][mb]))
    fw.close()


def run_profile_case(args):
    import ctypes as C

    from ultra_ep_b200 import capi, sim
    from ultra_ep_b200 import workloads as W

    env = Env()
    torch, dev = env.torch, env.dev
    lib = capi.lib()
    case = args.profile_case
    reps = 3 + 3
    st = torch.cuda.current_stream().cuda_stream

    def own_plan(cfg):
        """Plan of rank 0 from this library's solver (device tensors), and rank 0's ids."""
        N, M, R, L = cfg.ep, cfg.masters, cfg.redundant, cfg.num_experts
        P, D = N * (M + R), N
        lpr = torch.from_numpy(W.loads_per_rank(cfg)).to(dev)
        out = {k: torch.empty(s_, dtype=torch.int32, device=dev) for k, s_ in
               [("p2l", (P,)), ("l2p", (L, D)), ("lcnts", (L,)), ("quota", (L, D)), ("qp", (L, D)), ("rqp", (L, D))]}
        gl = torch.empty(L, dtype=torch.int32, device=dev)
        prm = capi.SolverParams.defaults()
        capi.check(lib.uep_solve_placement(lpr.data_ptr(), gl.data_ptr(), out["p2l"].data_ptr(), out["l2p"].data_ptr(),
                                           out["lcnts"].data_ptr(), out["quota"].data_ptr(), out["qp"].data_ptr(),
                                           out["rqp"].data_ptr(), N, N, M, R, D, C.byref(prm), 0, None, st))
        return out, torch.from_numpy(W.routing_ids(cfg, 0)).to(dev)

    if case in ("dense", "sparse"):
        cfg = W.CONFIGS["cfg3_qwen3_235b_fp8"]
        N, M, R, L, T, K = cfg.ep, cfg.masters, cfg.redundant, cfg.num_experts, cfg.tokens_per_rank, cfg.topk
        P, D = N * (M + R), N
        plan, ids = own_plan(cfg)
        if case == "dense":
            rmap = torch.zeros((T, L), dtype=torch.bool, device=dev).scatter_(1, ids.long(), True)
            probs = torch.rand((T, L), dtype=torch.float32, device=dev) * rmap
            om = torch.empty((T, P), dtype=torch.bool, device=dev)
            op = torch.empty((T, P), dtype=torch.float32, device=dev)
            scr = torch.empty(int(lib.uep_reroute_scratch_elems(T, 0, L)), dtype=torch.int32, device=dev)
            fn = lambda: capi.check(lib.uep_dense_reroute_forward(
                rmap.data_ptr(), probs.data_ptr(), plan["l2p"].data_ptr(), plan["lcnts"].data_ptr(), plan["rqp"].data_ptr(),
                om.data_ptr(), op.data_ptr(), scr.data_ptr(), T, L, P, D, 1, 1, st))
        else:
            out = torch.empty_like(ids)
            scr = torch.empty(int(lib.uep_reroute_scratch_elems(T, K, L)), dtype=torch.int32, device=dev)
            fn = lambda: capi.check(lib.uep_sparse_reroute_i32(
                ids.data_ptr(), out.data_ptr(), T, K, L, plan["l2p"].data_ptr(), plan["lcnts"].data_ptr(),
                plan["rqp"].data_ptr(), D, 1, scr.data_ptr(), st))
    elif case == "gather":
        rows, H = 16384, 4096
        src = torch.empty((rows, H), dtype=torch.bfloat16, device=dev).normal_(0, 1e-3)
        dst = torch.empty_like(src)
        pos = torch.randperm(rows, device=dev).to(torch.int32)
        status = torch.zeros(2, dtype=torch.int32, device=dev)
        fn = lambda: capi.check(lib.uep_gather_rows(src.data_ptr(), pos.data_ptr(), dst.data_ptr(), rows, rows, H * 2,
                                                    status.data_ptr(), st))
    elif case in ("reduce", "plan", "sync"):
        cfg = W.CONFIGS["profile_small_fp8"]
        args.plan_mode_resolved = 0
        group, ranks = make_group(env, cfg, 2, case == "reduce", args)
        ids = [torch.from_numpy(W.routing_ids(cfg, r)).to(dev) for r in ranks]
        group.update_placement(0, ids)
        if case == "reduce":
            M = cfg.masters
            g1 = [torch.empty((M, cfg.fc1_numel), dtype=torch.float32, device=dev).normal_(0, 1e-4) for _ in ranks]
            g2 = [torch.empty((M, cfg.fc2_numel), dtype=torch.float32, device=dev).normal_(0, 1e-4) for _ in ranks]
            t1 = group.pointer_tables([[g[m] for m in range(M)] for g in g1])
            t2 = group.pointer_tables([[g[m] for m in range(M)] for g in g2])
            fn = lambda: group.grad_reduce(0, t1, t2)
        elif case == "sync":
            masters = Masters(env, cfg, group, ranks)
            t = masters.tables
            fn = lambda: group.weight_sync(0, t[0], t[1], t[2], t[3])
        else:
            fn = lambda: group.update_placement(1, ids)
    else:
        raise SystemExit(f"unknown profile case {case}")
    times = []
    for i in range(reps):
        env.flush_l2()
        a, b = timed(torch, fn)
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    print(json.dumps({"profile_case": case, "launch_us": [round(x, 1) for x in times]}))


def run_ours(args):
    from ultra_ep_b200 import capi
    from ultra_ep_b200 import workloads as W

    env = Env()
    torch = env.torch
    world, rank = env.world, env.rank
    if args.gpus != world and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")
    # plan mode: direct on the simulated group (its peers are buffers of one device: there is no link to relieve),
    # adaptive relay over NVLink
    args.plan_mode_resolved = args.plan_mode if args.plan_mode >= 0 else (0 if world == 1 else 1)
    base = W.CONFIGS[args.config]
    cfg = base.with_ep(world) if world > 1 else base
    num_layers = 8
    pool = pool_size(args.steps)
    warmup = max(args.warmup, 3)
    peak_hbm, peak_src = load_peaks()
    lib = capi.lib()

    fw = Forward(env, cfg, args, num_layers, pool)
    # ---- timed: K steps, device-resident inputs, L2 flushed between steps ------------------
    sampler = ClockSampler(env.local_rank)
    if rank == 0:
        sampler.start()
    lib.uep_reset_launch_count()
    t_wall0 = time.perf_counter()
    step_ms = fw.run_timed(fw.step, args.steps, warmup)
    rank_mean_max_ms = fw.rank_mean_max_ms
    t_wall = time.perf_counter() - t_wall0
    launches = int(lib.uep_launch_count())
    # ---- e2e through the C ABI: host buffers in, host buffers out, every step -----------------
    e2e_ms = fw.run_timed(fw.step_e2e, args.steps, 3)
    clocks = sampler.stop() if rank == 0 else None

    # ---- the same step captured once into a CUDA graph and replayed (device-resident inputs) ---
    graph_ms = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fw.step(0, fw.ids_stage)  # sizes are final: nothing allocates during the capture
        torch.cuda.current_stream().wait_stream(side)
        env.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fw.step(0, fw.ids_stage)
        env.barrier()
        for i in range(3):  # untimed: the first replay uploads the instantiated graph to the device
            fw.stage_all.copy_(fw.ids_all_dev[i % pool], non_blocking=True)
            env.flush_l2()
            graph.replay()
        env.barrier()
        evs = []
        for i in range(args.steps):
            fw.stage_all.copy_(fw.ids_all_dev[i % pool], non_blocking=True)
            env.flush_l2()
            evs.append(timed(torch, graph.replay))
        env.barrier()
        fw.group.check_status()
        graph_ms = env.max_each([a.elapsed_time(b) for a, b in evs])
        del graph

    # ---- checks at full size: plan, routing, replica bytes --------------------------------------
    parity = fw.parity(sorted({0, 1 % pool, pool - 1}), cfg.name)

    # ---- per-operation breakdown, link measurement, roofline -------------------------------------
    link = link_probe(env, fw.group, cfg) if world > 1 else None
    plan_ms, sync_ms, reroute_ms, vols = fw.breakdown(min(args.steps, 2 * pool))
    roofline = sync_roofline(env, fw, sync_ms, vols, peak_hbm, peak_src, link)
    ref = ref_sm100(env, fw, args) if not args.no_ref else None
    if ref is not None and "weight_sync_bytes_ok" in ref:
        parity["ref_sync_bytes"] = bool(ref["weight_sync_bytes_ok"])
    fw.close()

    # ---- the drop-in Manager -----------------------------------------------------------------------
    manager_api, mgr_sparse = None, None
    if world > 1 and not args.no_manager:
        manager_api, mgr_sparse = manager_section(env, cfg, args, pool)
        parity["manager_api"] = bool(manager_api["parity"])

    # ---- backward, the other configurations, the reference's own test workload ------------------
    backward = run_backward(env, args, peak_hbm, link) if not args.no_backward else None
    if backward is not None:
        parity["reduce"] = bool(backward["grad_reduce_parity"])
        parity["gather_rows"] = bool(backward["gather_rows_parity"])
        parity["dense_reroute"] = bool(backward["dense_reroute_forward_parity"])
    configs = None
    if not args.no_configs:
        configs = {}
        for name in ("cfg1_plan_reroute", "cfg2_qwen3_30b_bf16"):
            configs[name] = config_forward(env, args, name, peak_hbm, peak_src, link)
        configs["cfg5_dsv3_stress"] = config5_forward_backward(env, args, peak_hbm, link)
        parity["configs"] = all(all(c["parity"].values()) for c in configs.values())
    replay = ep64_replay(env, args) if (world == 1 and not args.no_configs) else None
    if replay is not None:
        parity["ep64_replay"] = all(v["parity"] for k, v in replay.items() if k.startswith("imbalance_"))

    failed = bool(env.failures) or not all(bool(v) for v in parity.values())
    failed = not env.all_true(not failed)
    if rank == 0:
        mean_ms = sum(step_ms) / len(step_ms)
        e2e_abi = sum(e2e_ms) / len(e2e_ms)
        if mgr_sparse is not None:
            e2e_val = sum(mgr_sparse) / len(mgr_sparse)
            e2e = {"value": round(e2e_val * 1e3, 2), "unit": UNIT, "h2d_bytes_per_step": manager_api["sparse_e2e"]["h2d_bytes_per_step"],
                   "d2h_bytes_per_step": manager_api["sparse_e2e"]["d2h_bytes_per_step"],
                   "api": "ultra_ep_b200.Manager (update_placement_sparse, weight_sync, reroute_sparse on int64 ids), pinned host buffers",
                   "stats": stats_us(mgr_sparse), "c_abi_value": round(e2e_abi * 1e3, 2)}
        else:
            e2e = {"value": round(e2e_abi * 1e3, 2), "unit": UNIT, "h2d_bytes_per_step": fw.h2d_bytes, "d2h_bytes_per_step": fw.d2h_bytes,
                   "api": "C ABI on the simulated group (uep_update_placement, uep_weight_sync, uep_reroute_sparse), pinned host buffers; "
                          "the Manager hosts one rank per process and cannot simulate EP8", "stats": stats_us(e2e_ms)}
        out = {
            "metric": METRIC, "value": round(mean_ms * 1e3, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(mean_ms, 5), "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {
                "workload": f"{cfg.name}: forward update_placement + weight_sync + reroute, "
                            + ("EP8 simulated on one GPU (8 ranks per launch)" if world == 1 else f"EP{world}, one rank per GPU"),
                "experts": cfg.num_experts, "topk": cfg.topk, "tokens_per_rank": cfg.tokens_per_rank,
                "redundant_per_rank": cfg.redundant, "expert_bytes": cfg.expert_bytes, "zipf_s": cfg.zipf_s,
                "weight_sync_plan_mode": args.plan_mode_resolved,
                "l2": "between timed steps a 256 MiB buffer is written, then a second 256 MiB buffer is read",
                "rank_alignment": ("none (one process)" if world == 1 else
                                   "a one-word NCCL all-reduce is queued on the stream in front of every L2 flush, outside the timed "
                                   "events: the ranks enter each step together; the host never waits inside the loop"),
                "microbatch_pool": pool,
            },
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "parity": parity, "roofline": roofline,
            "step_stats_us": stats_us(step_ms),
            "value_statistic": {"value": "mean over the timed steps of the SLOWEST rank's CUDA-event time of that step (a layer is done "
                                         "when its slowest rank is)",
                                "max_over_ranks_of_own_mean_us": round(rank_mean_max_ms * 1e3, 2),
                                "note": "the second figure is each rank's own mean step, then the largest of them: what a loop of K "
                                        "steps bracketed by barriers gives per rank; lower, because the busiest rank changes from "
                                        "microbatch to microbatch"},
            "breakdown_us": {"plan": round(sum(plan_ms) / len(plan_ms) * 1e3, 2),
                             "weight_sync": round(sum(sync_ms) / len(sync_ms) * 1e3, 2),
                             "reroute": round(sum(reroute_ms) / len(reroute_ms) * 1e3, 2),
                             "medians": {"plan": round(statistics.median(plan_ms) * 1e3, 2),
                                         "weight_sync": round(statistics.median(sync_ms) * 1e3, 2) if sync_ms else None,
                                         "reroute": round(statistics.median(reroute_ms) * 1e3, 2)},
                             "weight_sync_per_launch": [round(x * 1e3, 1) for x in sync_ms]},
            "wall_s_timed_region": round(t_wall, 3),
        }
        if graph_ms is not None:
            out["graph_replay"] = {"value": round(sum(graph_ms) / len(graph_ms) * 1e3, 2), "unit": UNIT, "stats": stats_us(graph_ms),
                                   "note": "the same step (same three calls) captured once into a CUDA graph and replayed; "
                                           "a step always works on layer slot 0 of the plan storage"}
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(cfg, args)
        for key, val in (("ref_sm100", ref), ("manager_api", manager_api), ("backward", backward), ("configs", configs),
                         ("reference_test_workload_ep64", replay)):
            if val is not None:
                out[key] = val
        if env.failures:
            out["parity_failures"] = env.failures[:20]
        print(json.dumps(out), flush=True)
    if world > 1:
        env.dist.barrier()
        env.dist.destroy_process_group()
    if failed:
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg3_qwen3_235b_fp8")
    ap.add_argument("--sync-sms", type=int, default=0, help="CTAs per rank of the weight_sync kernel (0 = default)")
    ap.add_argument("--plan-mode", type=int, default=-1, choices=[-1, 0, 1, 2],
                    help="weight_sync: 0 direct fan-out, 1 adaptive relay, 2 relay every expert with >= 2 replicas; "
                         "-1 (default): 0 on the simulated group, 1 over NVLink")
    ap.add_argument("--relay-min-replicas", type=int, default=4)
    ap.add_argument("--cpu-budget-s", type=float, default=10.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="skip the CUDA-graph replay figure")
    ap.add_argument("--no-backward", action="store_true", help="skip the backward-path figures (cfg4)")
    ap.add_argument("--no-configs", action="store_true", help="skip cfg 1, 2, 5 and the EP64 replay")
    ap.add_argument("--no-manager", action="store_true", help="skip the Manager-API section (N > 1)")
    ap.add_argument("--reduce-sms", type=int, default=42, help="CTAs of the Wgrad reduce kernel (reference default 42)")
    ap.add_argument("--profile-case", default="", choices=["", "dense", "sparse", "gather", "reduce", "plan", "sync", "trace"],
                    help="run six launches of one kernel family on a small fixed case and exit (for profiler captures); "
                         "trace: print the device-side time stamps of weight_sync at full size, at any N, and exit")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.profile_case == "trace":
        run_device_trace(args)
    elif args.profile_case:
        run_profile_case(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
