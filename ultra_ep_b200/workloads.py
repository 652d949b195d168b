"""Seeded synthetic workloads with the shapes and value distributions of the five
benchmark configurations (routing ids, expert weights, gradients).

Router output is stood in for by draws without replacement from a Zipf popularity over a
seed-permuted expert order; nothing here reproduces a dataset. numpy's PCG64 generator is
used so that the same seed gives the same inputs on every machine.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np


@dataclass(frozen=True)
class LayerConfig:
    name: str
    num_experts: int  # L (global logical experts)
    ep: int  # N
    redundant: int  # R per rank
    topk: int
    tokens_per_rank: int
    zipf_s: float
    hidden: int = 0
    moe_ffn: int = 0
    weight_dtype: str = "none"  # "bf16" | "fp8" | "none"
    hot_expert_every_token: bool = False  # cfg5: one expert present in every token's top-k
    max_microbatches: int = 1
    redraw_popularity: bool = False  # cfg3: new popularity order each microbatch
    seed: int = 33  # default seed of the reference's own test scripts

    @property
    def masters(self) -> int:
        return self.num_experts // self.ep

    @property
    def fc1_numel(self) -> int:
        return 2 * self.hidden * self.moe_ffn

    @property
    def fc2_numel(self) -> int:
        return self.hidden * self.moe_ffn

    @property
    def weight_elem_bytes(self) -> int:
        return {"bf16": 2, "fp8": 1, "none": 2}[self.weight_dtype]

    @property
    def fc1_scale_numel(self) -> int:  # one UE8M0 byte per 1x128 block
        return self.fc1_numel // 128 if self.weight_dtype == "fp8" else 0

    @property
    def fc2_scale_numel(self) -> int:
        return self.fc2_numel // 128 if self.weight_dtype == "fp8" else 0

    @property
    def expert_bytes(self) -> int:
        """Bytes one replica receives in weight_sync (weights + scales)."""
        return (self.fc1_numel + self.fc2_numel) * self.weight_elem_bytes + self.fc1_scale_numel + self.fc2_scale_numel

    def with_ep(self, ep: int) -> "LayerConfig":
        assert self.num_experts % ep == 0
        return replace(self, ep=ep)


CONFIGS = {
    # plan + reroute only
    "cfg1_plan_reroute": LayerConfig("cfg1_plan_reroute", 64, 8, 2, 8, 4096, 1.2),
    # Qwen3-30B-A3B-shaped layer, bf16 experts
    "cfg2_qwen3_30b_bf16": LayerConfig("cfg2_qwen3_30b_bf16", 128, 8, 4, 8, 8192, 1.2, 2048, 768, "bf16"),
    # Qwen3-235B-A22B-shaped layer, fp8 experts with UE8M0 scales: the headline forward
    "cfg3_qwen3_235b_fp8": LayerConfig("cfg3_qwen3_235b_fp8", 128, 8, 4, 8, 8192, 1.3, 4096, 1536, "fp8",
                                       redraw_popularity=True),
    # backward of the same layer (token-gradient gather + fp32 Wgrad reduce)
    "cfg4_qwen3_235b_bwd": LayerConfig("cfg4_qwen3_235b_bwd", 128, 8, 4, 8, 8192, 1.3, 4096, 1536, "fp8"),
    # small stand-in of cfg3 for profiler captures (same kernel paths, a few hundred MB on the device)
    "profile_small_fp8": LayerConfig("profile_small_fp8", 128, 8, 4, 8, 8192, 1.3, 2048, 768, "fp8",
                                     redraw_popularity=True),
    # DeepSeek-V3-shaped extreme skew
    "cfg5_dsv3_stress": LayerConfig("cfg5_dsv3_stress", 256, 8, 8, 8, 16384, 1.5, 7168, 2048, "fp8",
                                    hot_expert_every_token=True, max_microbatches=4),
}


def popularity(cfg: LayerConfig, microbatch: int = 0) -> np.ndarray:
    """Probability of each logical expert: Zipf(s) over a seed-permuted order."""
    L = cfg.num_experts
    w = (np.arange(1, L + 1, dtype=np.float64)) ** (-cfg.zipf_s)
    seed = cfg.seed + (microbatch if cfg.redraw_popularity else 0)
    perm = np.random.default_rng(seed).permutation(L)
    p = np.empty(L, np.float64)
    p[perm] = w  # expert perm[i] gets the i-th largest popularity
    return p / p.sum()


def routing_ids(cfg: LayerConfig, rank: int, microbatch: int = 0, tokens: int | None = None) -> np.ndarray:
    """int32 [T, K]: K distinct experts per token, drawn without replacement (Gumbel top-k,
    which is exactly sequential sampling without replacement from the popularity)."""
    T = cfg.tokens_per_rank if tokens is None else tokens
    K, L = cfg.topk, cfg.num_experts
    if T == 0:
        return np.empty((0, K), np.int32)
    p = popularity(cfg, microbatch)
    rng = np.random.default_rng(cfg.seed + 104729 * rank + 7907 * microbatch)
    keys = np.log(p)[None, :] + rng.gumbel(size=(T, L))
    if cfg.hot_expert_every_token:
        hot = int(np.argmax(p))
        keys[:, hot] = np.inf
    part = np.argpartition(-keys, K - 1, axis=1)[:, :K]
    order = np.argsort(-np.take_along_axis(keys, part, axis=1), axis=1, kind="stable")
    return np.take_along_axis(part, order, axis=1).astype(np.int32)


def ids_to_map(ids: np.ndarray, L: int) -> np.ndarray:
    """bool [T, L] routing map of int ids [T, K]."""
    T = ids.shape[0]
    m = np.zeros((T, L), np.bool_)
    if T:
        m[np.arange(T)[:, None], ids] = True
    return m


def probs_for_map(routing_map: np.ndarray, seed: int) -> np.ndarray:
    """fp32 [T, L]: U(0,1) on routed entries, 0 elsewhere."""
    rng = np.random.default_rng(seed)
    pr = np.zeros(routing_map.shape, np.float32)
    pr[routing_map] = rng.random(int(routing_map.sum()), dtype=np.float32)
    return pr


def loads_per_rank(cfg: LayerConfig, microbatch: int = 0) -> np.ndarray:
    """int32 [N, L] per-rank expert loads of the configuration."""
    L = cfg.num_experts
    rows = [np.bincount(routing_ids(cfg, r, microbatch).reshape(-1), minlength=L) for r in range(cfg.ep)]
    return np.stack(rows).astype(np.int32)


def expert_weight_bytes(cfg: LayerConfig, global_expert: int, shard: int, nbytes: int) -> np.ndarray:
    """uint8 bytes of one master shard. Only the bytes matter to the copy path, so the fp8 / bf16
    payload is drawn as N(0, 0.02) values reduced to their storage bytes by a fixed quantiser:
    bf16 keeps the upper 16 bits of the fp32 pattern; fp8 data and UE8M0 scale bytes are taken
    from the fp32 exponent/mantissa bits. Deterministic in (seed, expert, shard)."""
    rng = np.random.default_rng([cfg.seed, global_expert, shard])
    if cfg.weight_dtype == "bf16" and shard < 2:
        vals = rng.normal(0.0, 0.02, nbytes // 2).astype(np.float32)
        return (vals.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8)
    if shard < 2:
        vals = rng.normal(0.0, 0.02, nbytes).astype(np.float32)
        bits = vals.view(np.uint32)
        # sign | 4 exponent bits (rebased, clamped) | 3 mantissa bits
        sign = (bits >> 24) & 0x80
        exp = np.clip(((bits >> 23) & 0xFF).astype(np.int32) - 127 + 7 + 6, 0, 15).astype(np.uint32)
        man = (bits >> 20) & 0x7
        return (sign | (exp << 3) | man).astype(np.uint8)
    return rng.integers(118, 124, nbytes, dtype=np.uint8)  # UE8M0 exponents around 2^-6


def fp32_grads(seed_key, numel: int, std: float) -> np.ndarray:
    rng = np.random.default_rng(seed_key)
    return rng.normal(0.0, std, numel).astype(np.float32)


# ------------------------------------------------------------------------------------------
# The skew model of the reference's own test scripts (tests/utils.py:355-561 of the reference),
# restated on numpy: expert popularity = (rank weight ~ rank^-alpha) x (position weight ~ position^-4
# inside the rank), with alpha found by bisection so that the expected max/mean rank load, under top-k
# sampling WITHOUT replacement, meets a target ratio. Draws use numpy's generator (Gumbel top-k), so the
# tokens differ from the reference's torch.multinomial draws while following the same distribution.
# ------------------------------------------------------------------------------------------
def _topk_inclusion_probs(weights: np.ndarray, topk: int) -> np.ndarray:
    """Approximate probability that each expert is among the k drawn: 1 - exp(-c w) with sum = k."""
    w = weights.astype(np.float64)
    lo, hi = 0.0, 1.0
    while float((1.0 - np.exp(-hi * w)).sum()) < topk:
        hi *= 2.0
    for _ in range(48):
        mid = (lo + hi) * 0.5
        if float((1.0 - np.exp(-mid * w)).sum()) < topk:
            lo = mid
        else:
            hi = mid
    return 1.0 - np.exp(-hi * w)


def _rank_skew_weights(num_ranks: int, masters: int, rank_alpha: float, local_alpha: float) -> np.ndarray:
    rw = 1.0 / np.arange(1, num_ranks + 1, dtype=np.float64) ** rank_alpha
    lw = 1.0 / np.arange(1, masters + 1, dtype=np.float64) ** local_alpha
    w = (rw[:, None] * lw[None, :]).reshape(-1)
    return (w / w.sum()).astype(np.float32)


def rank_skew_popularity(num_ranks: int, masters: int, topk: int, imbalance_ratio: float) -> np.ndarray:
    """Expert popularity whose expected max/mean rank load is `imbalance_ratio` (>= 1)."""
    L = num_ranks * masters
    if imbalance_ratio <= 1.0:
        return np.full(L, 1.0 / L, np.float32)
    local_alpha = 4.0 if masters > 1 else 0.0

    def ratio(alpha: float) -> float:
        w = _rank_skew_weights(num_ranks, masters, alpha, local_alpha)
        loads = _topk_inclusion_probs(w, topk).reshape(num_ranks, masters).sum(1)
        return float(loads.max() / loads.mean())

    lo, hi = 0.0, 8.0
    for _ in range(32):
        mid = (lo + hi) * 0.5
        if ratio(mid) < imbalance_ratio:
            lo = mid
        else:
            hi = mid
    return _rank_skew_weights(num_ranks, masters, hi, local_alpha)


def reference_style_loads(num_ranks: int, masters: int, topk: int, tokens_per_rank: int, imbalance_ratio: float,
                          seed: int = 33):
    """(int32 [N, L] per-rank loads, int32 [T, K] routing ids of rank 0) under the skew model above."""
    L = num_ranks * masters
    p = rank_skew_popularity(num_ranks, masters, topk, imbalance_ratio).astype(np.float64)
    logp = np.log(p / p.sum())
    rows, ids0 = [], None
    for r in range(num_ranks):
        rng = np.random.default_rng(seed + r * 104729)
        u = rng.random((tokens_per_rank, L), dtype=np.float32)
        np.maximum(u, np.float32(1e-30), out=u)
        keys = logp.astype(np.float32)[None, :] - np.log(-np.log(u))  # Gumbel top-k = sampling without replacement
        part = np.argpartition(-keys, topk - 1, axis=1)[:, :topk]
        order = np.argsort(-np.take_along_axis(keys, part, axis=1), axis=1, kind="stable")
        ids = np.take_along_axis(part, order, axis=1).astype(np.int32)
        if r == 0:
            ids0 = ids
        rows.append(np.bincount(ids.reshape(-1), minlength=L))
    return np.stack(rows).astype(np.int32), ids0
