"""Generates tests/golden/special_transforms_golden.npz from the reference's own CPU build (oracle/_ref): the
outputs of execTransformFloat for the whole-array transforms Col2Im 36, Im2col 37, Histogram 48, Reverse 70 and
Pooling2D 71 on seeded inputs, so that the numpy restatements and the CUDA path can be held against the reference
where its checkout is absent.

    python tests/golden/make_special_golden.py

Inputs are not stored: tests/special_golden_cases.py rebuilds them from the seeds."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.reference import Reference  # noqa: E402
from tests import special_golden_cases as G  # noqa: E402


def main():
    ref = Reference()
    out = {}
    for name, case in G.cases():
        op, x, x_info, z, z_info, extra = G.build(case)
        out[name] = ref.transform(op, x.copy(), x_info, z.copy(), z_info, extra).copy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "special_transforms_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, len(out), "records", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
