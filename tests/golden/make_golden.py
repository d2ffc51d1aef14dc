"""Generates tests/golden/legacy_ops_golden.npz from the reference's own CPU build
(oracle/_ref/libnd4jref.so, compiled from the reference sources by oracle/Makefile).

    python tests/golden/make_golden.py

Every record stores the seeded inputs' recipe (not the inputs), the call and the reference's
output, so that the oracle port and the CUDA path can both be held against it on machines where
the reference checkout is absent. Kept small on purpose (a few hundred KB).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from libnd4j_b200 import shape as S  # noqa: E402
from oracle.reference import Reference  # noqa: E402
from tests.cases import Layout, rand_input, result_info  # noqa: E402
from tests import golden_cases as G  # noqa: E402


def main():
    ref = Reference()
    out = {}
    for name, case in G.cases():
        out[name] = G.run_case(ref, case)
    # RNG table probes and TAD descriptors
    state, table = ref.init_random(119, 100000)
    out["rng/table_head"] = table[:8].copy()
    out["rng/table_tail"] = table[-4:].copy()
    out["rng/elements"] = np.array([ref.rng_element(state, p) for p in G.RNG_PROBES], dtype=np.uint64)
    ref.destroy_random(state)
    for i, (shape, order, dims) in enumerate(G.TAD_CASES):
        info, offs = ref.tad(S.shape_info(shape, order), dims)
        out["tad/%d/info" % i] = info
        out["tad/%d/offsets" % i] = offs
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "legacy_ops_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "records")


if __name__ == "__main__":
    main()
