"""Named solver / reroute cases shared by the CPU tests, the GPU parity tests and the
script that records the reference's outputs (tests/golden/make_golden.py).

A case is a per-rank load matrix plus solver parameters. The set covers the five benchmark
configurations, every branch of the threshold search (fast path, precheck, four-probe
search, no search at all), several NVLink-domain shapes (1-3 ranks per solver lane,
several domains) and degenerate loads.
"""

from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from ultra_ep_b200 import workloads as W  # noqa: E402


@dataclass
class SolveCase:
    name: str
    loads_per_rank: np.ndarray  # int32 [N, L]
    M: int
    R: int
    nvl: int
    balance_threshold: float = 1.0
    min_tokens: int = 1024
    allow_zero: bool = False
    locality: bool = True
    eps: float = 0.01
    ranks: tuple = (0,)  # ranks whose rank_quota_prefix is checked
    tags: tuple = field(default_factory=tuple)

    @property
    def N(self):
        return self.loads_per_rank.shape[0]

    @property
    def L(self):
        return self.loads_per_rank.shape[1]


def _zipf_loads(N, M, T, K, s, seed, hot_rank_bias=0.0):
    """Per-rank loads from a cheap multinomial (not distinct per token; only totals matter here)."""
    L = N * M
    rng = np.random.default_rng(seed)
    w = np.arange(1, L + 1, dtype=np.float64) ** (-s)
    p = np.empty(L)
    p[rng.permutation(L)] = w
    if hot_rank_bias:
        p[:M] *= (1.0 + hot_rank_bias)
    p /= p.sum()
    return np.stack([rng.multinomial(T * K, p) for _ in range(N)]).astype(np.int32)


def solve_cases(full: bool = True):
    cases = []
    # 1. the five benchmark configurations, all ranks for the headline one
    for name, cfg in W.CONFIGS.items():
        if name == "cfg4_qwen3_235b_bwd":
            continue  # same routing as cfg3
        if not full and name == "cfg5_dsv3_stress":
            continue
        lpr = W.loads_per_rank(cfg)
        ranks = tuple(range(cfg.ep)) if name in ("cfg1_plan_reroute", "cfg3_qwen3_235b_fp8") else (0, cfg.ep - 1)
        cases.append(SolveCase(name, lpr, cfg.masters, cfg.redundant, cfg.ep, ranks=ranks, tags=("config",)))
    cfg1 = W.CONFIGS["cfg1_plan_reroute"]
    lpr1 = W.loads_per_rank(cfg1)
    # 2. parameter variants on cfg1
    cases += [
        SolveCase("cfg1_R1", lpr1, 8, 1, 8, ranks=(0, 3)),
        SolveCase("cfg1_R0", lpr1, 8, 0, 8, ranks=(0, 5)),
        SolveCase("cfg1_min1", lpr1, 8, 2, 8, min_tokens=1, ranks=(1,)),
        SolveCase("cfg1_min_huge", lpr1, 8, 2, 8, min_tokens=1 << 20, ranks=(2,)),
        SolveCase("cfg1_nolocality", lpr1, 8, 2, 8, locality=False, ranks=(0, 7)),
        SolveCase("cfg1_allow_zero", lpr1, 8, 2, 8, allow_zero=True, ranks=(4,)),
        SolveCase("cfg1_eps0", lpr1, 8, 2, 8, eps=0.0, ranks=(0,)),
        SolveCase("cfg1_eps_neg", lpr1, 8, 2, 8, eps=-1.0, ranks=(0,)),
        SolveCase("cfg1_bt1p2", lpr1, 8, 2, 8, balance_threshold=1.2, ranks=(6,)),
        SolveCase("cfg1_bt0p5", lpr1, 8, 2, 8, balance_threshold=0.5, ranks=(6,)),
        SolveCase("cfg1_two_domains", lpr1, 8, 2, 4, ranks=(0, 4, 7)),
        SolveCase("cfg1_four_domains", lpr1, 8, 2, 2, ranks=(1, 6)),
    ]
    # EP < 8 for cfg5-like shapes (M grows)
    cfg5 = W.CONFIGS["cfg5_dsv3_stress"]
    if full:
        lpr5 = W.loads_per_rank(cfg5)
        for ep in (2, 4):
            M = 256 // ep
            # regroup the 8-rank loads onto ep ranks (sum of source ranks), keeps totals
            grouped = lpr5.reshape(ep, 8 // ep, 256).sum(1).astype(np.int32)
            cases.append(SolveCase(f"cfg5_ep{ep}", grouped, M, 8, ep, ranks=(0, ep - 1)))
    # 3. search branches: tight slots and skew that defeat the fast path
    for i, (N, M, R, s, bias, mt) in enumerate([
        (8, 4, 1, 1.6, 3.0, 1024), (8, 2, 1, 2.0, 8.0, 1), (4, 4, 1, 1.8, 5.0, 64), (8, 8, 1, 1.5, 6.0, 1024),
        (8, 1, 1, 1.2, 0.0, 1), (8, 1, 2, 2.5, 0.0, 1), (16, 2, 1, 1.7, 10.0, 256), (8, 16, 2, 2.2, 12.0, 4096),
        (8, 4, 1, 3.0, 20.0, 1), (3, 5, 2, 1.4, 2.0, 16), (5, 3, 1, 1.9, 7.0, 1), (8, 4, 2, 1.3, 0.5, 100000),
    ]):
        lpr = _zipf_loads(N, M, 2048, 8, s, 1000 + i, bias)
        cases.append(SolveCase(f"skew{i}_N{N}_M{M}_R{R}", lpr, M, R, N, min_tokens=mt, ranks=(0, N - 1), tags=("skew",)))
    # many small experts on one hot rank: the dynamic floor of the fast path exceeds what any
    # single expert can export, the static floor of the fallback does not
    small = np.zeros((4, 32), np.int32); small[:, :8] = 25; small[:, 8:] = 1; small[1, 8:] = 3
    cases.append(SolveCase("many_small_R2", small, 8, 2, 4, min_tokens=1, ranks=(0, 2), tags=("skew",)))
    cases.append(SolveCase("many_small_R1", small, 8, 1, 4, min_tokens=1, ranks=(0, 3), tags=("skew",)))
    cases.append(SolveCase("many_small_R3_min8", small, 8, 3, 4, min_tokens=8, ranks=(1,), tags=("skew",)))
    big = np.zeros((8, 64), np.int32); big[:, :8] = 9000; big[:, 8:] = np.arange(56)[None, :] * 37 % 400
    cases.append(SolveCase("many_small_wide", big, 8, 2, 8, min_tokens=1, ranks=(0, 7), tags=("skew",)))
    cases.append(SolveCase("many_small_wide_R1", big, 8, 1, 8, min_tokens=1, ranks=(0, 7), tags=("skew",)))
    # fast path fails, the precheck at the capacity threshold succeeds
    for seed in (4, 11, 41, 48):
        rng = np.random.default_rng(seed)
        G = int(rng.integers(2, 9)); M = int(rng.integers(2, 10)); R = int(rng.integers(1, 4))
        lpr = rng.integers(0, 60, size=(G, G * M)).astype(np.int32)
        hot_rank = int(rng.integers(0, G)); lpr[:, hot_rank * M:(hot_rank + 1) * M] += int(rng.integers(20, 200))
        mt = int(rng.choice([1, 4, 16]))
        cases.append(SolveCase(f"precheck_seed{seed}", lpr, M, R, G, min_tokens=mt, ranks=(0, G - 1), tags=("skew",)))
    # 4. degenerate loads
    z = np.zeros((4, 8), np.int32)
    cases.append(SolveCase("all_zero", z, 2, 2, 4, ranks=(0, 3)))
    one = z.copy(); one[2, 5] = 1
    cases.append(SolveCase("single_token", one, 2, 2, 4, min_tokens=1, ranks=(0, 2)))
    eq = np.full((4, 8), 100, np.int32)
    cases.append(SolveCase("all_equal", eq, 2, 2, 4, ranks=(1,)))
    hot = np.zeros((8, 16), np.int32); hot[:, 3] = 5000; hot[:, 0] = 1
    cases.append(SolveCase("one_hot_expert", hot, 2, 2, 8, ranks=(0, 1, 7)))
    hot1 = hot.copy()
    cases.append(SolveCase("one_hot_expert_min1", hot1, 2, 3, 8, min_tokens=1, ranks=(0, 1)))
    rank_hot = np.zeros((8, 32), np.int32); rank_hot[:, 8:12] = np.arange(1, 5) * 700
    cases.append(SolveCase("one_hot_rank", rank_hot, 4, 2, 8, min_tokens=1, ranks=(0, 2, 5)))
    single = np.array([[5, 7, 9, 11]], np.int32)
    cases.append(SolveCase("single_rank", single, 4, 2, 1, ranks=(0,)))
    ties = np.tile(np.array([[10, 10, 10, 10, 50, 50, 50, 50]], np.int32), (4, 1))
    cases.append(SolveCase("ties", ties, 2, 1, 4, min_tokens=1, ranks=(0, 3)))
    # local-only tokens: locality split with hosts that own all of their quota
    loc = np.zeros((4, 8), np.int32); loc[0, 0] = 4000; loc[1, 0] = 10; loc[2, 0] = 3000; loc[3, 4] = 50
    cases.append(SolveCase("locality_mix", loc, 2, 2, 4, min_tokens=1, ranks=(0, 1, 2, 3)))
    # 5. wide domains: 2 and 3 ranks per solver lane, and a replica count above 8
    if full:
        cases.append(SolveCase("ep64", _zipf_loads(64, 4, 8192, 8, 1.1, 7, 4.0), 4, 2, 64, ranks=(0, 31, 63), tags=("wide",)))
        cases.append(SolveCase("ep72", _zipf_loads(72, 4, 4096, 8, 1.3, 8, 6.0), 4, 2, 72, ranks=(0, 40, 71), tags=("wide",)))
        many = np.zeros((16, 32), np.int32); many[:, 1] = 40000; many[:, 0] = 3
        many[np.arange(16), 2 * np.arange(16)] += 50
        cases.append(SolveCase("replicas_gt8", many, 2, 2, 16, min_tokens=1, ranks=(0, 9, 15), tags=("wide",)))
        cases.append(SolveCase("ep64_two_domains", _zipf_loads(64, 2, 4096, 8, 1.5, 9, 5.0), 2, 2, 32, ranks=(0, 33), tags=("wide",)))
    return cases


def random_small_cases(n: int, seed: int = 5):
    """Many tiny random cases for sweeps (E <= 16, G <= 4 and a few larger)."""
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        G = int(rng.integers(1, 5))
        domains = int(rng.integers(1, 3))
        N = G * domains
        M = int(rng.integers(1, 5))
        R = int(rng.integers(0, 4))
        scale = int(rng.choice([1, 3, 10, 100, 1000, 5000]))
        lpr = rng.integers(0, scale + 1, size=(N, N * M)).astype(np.int32)
        if rng.random() < 0.5:
            lpr[:, int(rng.integers(0, N * M))] *= int(rng.integers(2, 40))
        if rng.random() < 0.2:
            lpr[int(rng.integers(0, N))] = 0
        out.append(SolveCase(
            f"rand{i}", lpr, M, R, G,
            balance_threshold=float(rng.choice([1.0, 1.0, 1.1, 2.0])),
            min_tokens=int(rng.choice([1, 1, 2, 16, 1024])),
            allow_zero=bool(rng.random() < 0.3), locality=bool(rng.random() < 0.7),
            eps=float(rng.choice([0.01, 0.0, 0.1, 0.5])), ranks=(int(rng.integers(0, N)),), tags=("random",)))
    return out


@dataclass
class RerouteCase:
    name: str
    solve: SolveCase
    rank: int
    T: int
    K: int
    seed: int
    interleave: bool = True


def reroute_cases(full: bool = True):
    sc = {c.name: c for c in solve_cases(full)}
    cases = [
        RerouteCase("rr_cfg1_r0", sc["cfg1_plan_reroute"], 0, 4096, 8, 11),
        RerouteCase("rr_cfg1_r5_nointerleave", sc["cfg1_plan_reroute"], 5, 4096, 8, 12, interleave=False),
        RerouteCase("rr_cfg1_ragged", sc["cfg1_plan_reroute"], 3, 1000, 8, 13),
        RerouteCase("rr_cfg1_tiny", sc["cfg1_plan_reroute"], 2, 3, 8, 14),
        RerouteCase("rr_cfg1_empty", sc["cfg1_plan_reroute"], 2, 0, 8, 15),
        RerouteCase("rr_cfg3_r6", sc["cfg3_qwen3_235b_fp8"], 6, 8192, 8, 16),
        RerouteCase("rr_hot_min1", sc["one_hot_expert_min1"], 1, 700, 2, 17),
        RerouteCase("rr_locality_mix", sc["locality_mix"], 0, 512, 1, 18),
        RerouteCase("rr_odd_L15", sc["skew9_N3_M5_R2"], 2, 333, 3, 21),  # L not a multiple of 4: scalar row paths
    ]
    if full:
        cases.append(RerouteCase("rr_replicas_gt8", sc["replicas_gt8"], 9, 2500, 2, 19))
        cases.append(RerouteCase("rr_cfg5_r1", sc["cfg5_dsv3_stress"], 1, 16384, 8, 20))
    return cases


def reroute_inputs(rc: RerouteCase):
    """Routing ids consistent with the case's per-rank loads: exactly loads_per_rank[rank, e]
    entries name expert e when T*K equals the row sum; otherwise ids are drawn proportionally."""
    lpr = rc.solve.loads_per_rank
    L = lpr.shape[1]
    cfg = W.CONFIGS.get(rc.solve.name)
    if cfg is not None and rc.T == cfg.tokens_per_rank and rc.K == cfg.topk:
        return W.routing_ids(cfg, rc.rank)
    rng = np.random.default_rng(rc.seed)
    row = lpr[rc.rank].astype(np.float64)
    T, K = rc.T, rc.K
    if T == 0:
        return np.empty((0, K), np.int32)
    p = row + 1e-3
    p /= p.sum()
    keys = np.log(p)[None, :] + rng.gumbel(size=(T, L))
    part = np.argpartition(-keys, K - 1, axis=1)[:, :K] if K < L else np.tile(np.arange(L), (T, 1))
    return part.astype(np.int32)


def legacy_cases():
    """Load vectors for the legacy (host-side) placement solver: dicts with name, loads [L], N, M, R, nvl,
    balance_threshold. Covers: no redundancy, one-rank domains, thresholds that stop the granting early,
    ties between experts and between ranks, all-zero loads, more slots than useful instances, several domains."""
    out = []

    def add(name, loads, N, M, R, nvl, bt):
        out.append(dict(name=name, loads=np.ascontiguousarray(loads, np.int32), N=N, M=M, R=R, nvl=nvl, balance_threshold=bt))

    for i, (N, M, R, T, K, s, seed) in enumerate([(8, 8, 2, 4096, 8, 1.2, 33), (8, 16, 4, 8192, 8, 1.3, 34),
                                                   (8, 32, 8, 16384, 8, 1.5, 35), (4, 4, 1, 512, 2, 1.1, 36),
                                                   (2, 8, 3, 1024, 4, 2.0, 37), (16, 4, 2, 2048, 4, 1.4, 38)]):
        lpr = _zipf_loads(N, M, T, K, s, seed)
        for bt in (1.0, 1.25, 2.0):
            add(f"zipf{i}_bt{bt}", lpr.sum(0), N, M, R, N, bt)
    lpr = _zipf_loads(8, 8, 4096, 8, 1.3, 41)
    add("two_domains", lpr.sum(0), 8, 8, 2, 4, 1.0)
    add("one_rank_domains", lpr.sum(0), 8, 8, 2, 1, 1.0)
    add("no_redundant", lpr.sum(0), 8, 8, 0, 8, 1.0)
    add("all_zero", np.zeros(64, np.int32), 8, 8, 2, 8, 1.0)
    add("all_equal", np.full(64, 1000, np.int32), 8, 8, 2, 8, 1.0)
    add("all_equal_bt", np.full(64, 1000, np.int32), 8, 8, 2, 8, 1.5)
    one_hot = np.zeros(32, np.int32)
    one_hot[5] = 100000
    add("one_hot_many_slots", one_hot, 4, 8, 6, 4, 1.0)  # an expert gets at most G-1 extra instances
    rng = np.random.Generator(np.random.PCG64(77))
    for i in range(12):
        N = int(rng.choice([2, 4, 8]))
        M = int(rng.integers(1, 9))
        R = int(rng.integers(1, 5))
        loads = rng.integers(0, 50, N * M).astype(np.int32) * int(rng.choice([1, 1, 100]))  # small values: many ties
        add(f"random{i}", loads, N, M, R, N, float(rng.choice([1.0, 1.1, 3.0])))
    return out
