"""Record what the REFERENCE's own kernels produce on the shared test cases.

Runs on a machine with a B200 and oracle/_ref/libuep_ref.so (the reference's kernel sources
compiled unmodified; see oracle/Makefile). Writes tests/golden/ref_golden.npz, which the
CPU tests use to pin the oracle without a GPU:

    python tests/golden/make_golden.py [--out PATH]

Contents: for every solve case and checked rank, the six plan arrays of
quota_placement_solve_kernel; for every reroute case, the bit-packed expanded routing map of
the dense quota reroute kernels, a SHA-256 of the expanded probabilities and the backward
gather's SHA-256; the inputs (loads, ids) are stored next to them.
"""

import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases as Cs  # noqa: E402
from oracle import uep_ref  # noqa: E402
from ultra_ep_b200 import workloads as W  # noqa: E402

FIELDS = ("p2l", "l2p", "lcnts", "quota", "quota_prefix", "rank_quota_prefix")


def sha(t: np.ndarray) -> np.ndarray:
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(t).tobytes()).digest(), np.uint8).copy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "ref_golden.npz"))
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    store = {}
    names = []
    for case in Cs.solve_cases(True) + Cs.random_small_cases(60):
        names.append(case.name)
        key = f"solve/{case.name}"
        store[f"{key}/loads_per_rank"] = case.loads_per_rank
        store[f"{key}/params"] = np.array([case.M, case.R, case.nvl, case.min_tokens, int(case.allow_zero),
                                           int(case.locality)], np.int64)
        store[f"{key}/fparams"] = np.array([case.balance_threshold, case.eps], np.float32)
        store[f"{key}/ranks"] = np.array(case.ranks, np.int32)
        lpr = torch.from_numpy(case.loads_per_rank).to(dev)
        for rank in case.ranks:
            ref = uep_ref.solve_placement(lpr, case.M, case.R, case.nvl, rank, case.balance_threshold,
                                          case.min_tokens, case.allow_zero, case.locality, case.eps)
            torch.cuda.synchronize()
            for f in FIELDS:
                if f != "rank_quota_prefix" and rank != case.ranks[0]:
                    continue  # identical on every rank; checked below
                store[f"{key}/r{rank}/{f}"] = ref[f].cpu().numpy()
            if rank != case.ranks[0]:
                first = case.ranks[0]
                for f in FIELDS[:-1]:
                    assert np.array_equal(ref[f].cpu().numpy(), store[f"{key}/r{first}/{f}"]), "ranks disagree"
    store["solve_names"] = np.array(names)

    rnames = []
    for rc in Cs.reroute_cases(True):
        if rc.T == 0:
            continue
        rnames.append(rc.name)
        sc = rc.solve
        key = f"reroute/{rc.name}"
        lpr = torch.from_numpy(sc.loads_per_rank).to(dev)
        plan = uep_ref.solve_placement(lpr, sc.M, sc.R, sc.nvl, rc.rank, sc.balance_threshold, sc.min_tokens,
                                       sc.allow_zero, sc.locality, sc.eps)
        ids = Cs.reroute_inputs(rc)
        L, P = sc.L, sc.N * (sc.M + sc.R)
        rmap = W.ids_to_map(ids, L)
        probs = W.probs_for_map(rmap, rc.seed)
        d_map, d_probs = torch.from_numpy(rmap).to(dev), torch.from_numpy(probs).to(dev)
        out_probs, out_map = uep_ref.dense_reroute_forward(d_map, d_probs, plan["l2p"], plan["lcnts"],
                                                           plan["rank_quota_prefix"], P, rc.interleave)
        grad = torch.from_numpy(np.random.default_rng(rc.seed + 1).normal(size=(rc.T, P)).astype(np.float32)).to(dev)
        back = uep_ref.dense_reroute_backward(grad, d_map, out_map, plan["l2p"], plan["lcnts"])
        torch.cuda.synchronize()
        store[f"{key}/ids"] = ids
        store[f"{key}/meta"] = np.array([rc.rank, rc.T, rc.K, rc.seed, int(rc.interleave), L, P], np.int64)
        store[f"{key}/solve"] = np.array(sc.name)
        store[f"{key}/expanded_map_bits"] = np.packbits(out_map.cpu().numpy())
        store[f"{key}/expanded_probs_sha256"] = sha(out_probs.cpu().numpy())
        store[f"{key}/grad_probs_sha256"] = sha(back.cpu().numpy())
    store["reroute_names"] = np.array(rnames)
    store["provenance"] = np.array(
        f"reference kernels (oracle/_ref/libuep_ref.so) on {torch.cuda.get_device_name(0)}, torch {torch.__version__}")
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    np.savez_compressed(args.out, **store)
    print("wrote", args.out, os.path.getsize(args.out), "bytes;", len(names), "solve cases,", len(rnames), "reroute cases")


if __name__ == "__main__":
    main()
