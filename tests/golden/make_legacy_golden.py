"""Records what the reference's legacy host-side solver (csrc/kernels/legacy/placement_cpu.cpp, built in
place into oracle/_ref/libuep_ref_legacy.so by `make -C oracle ref`) produces for a set of seeded load
vectors: tests/golden/ref_legacy_golden.npz. Runs on CPU.

    python tests/golden/make_legacy_golden.py
"""

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases as Cs  # noqa: E402
from oracle import uep_ref  # noqa: E402


def main():
    out = {}
    names = []
    for case in Cs.legacy_cases():
        p2l, l2p, lcnts = uep_ref.legacy_solve_host(case["loads"], case["N"], case["M"], case["R"], case["nvl"],
                                                    case["balance_threshold"])
        names.append(case["name"])
        out[f"{case['name']}/p2l"], out[f"{case['name']}/l2p"], out[f"{case['name']}/lcnts"] = p2l, l2p, lcnts
    out["names"] = np.asarray(names)
    path = os.path.join(ROOT, "tests", "golden", "ref_legacy_golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(names)} cases")


if __name__ == "__main__":
    main()
