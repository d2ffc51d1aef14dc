"""The CUDA path against the committed golden vectors (tests/golden/legacy_ops_golden.npz, written by
tests/golden/make_golden.py from the reference's own CPU build): every record is replayed through the
C ABI on the GPU with the same seeded inputs. Needs neither the reference checkout nor its build."""
import os

import numpy as np
import pytest

from tests import golden_cases as G
from tests.cases import ulp_distance
from tests.gpu_adapter import GpuOps

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "legacy_ops_golden.npz")
CASES = list(G.cases())

# transforms whose reference value comes from the host libm (<= 2 ulp), and those whose formula cancels
# (measured in ulps of the O(1) intermediate, as in test_gpu_elementwise.py)
LIBM = {2, 3, 5, 10, 12, 13, 15, 16, 17, 18, 21, 22, 23, 29, 53, 54, 61, 62, 63, 64, 65, 67, 68, 74, 78, 86, 88, 90, 91}
CANCELLING = {13, 21, 22, 23, 29, 53, 54, 61, 62, 67, 68, 74, 88, 90, 91, 10, 63, 64, 65}


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


@pytest.mark.parametrize("name,case", CASES, ids=[n for n, _ in CASES])
def test_cuda_path_matches_golden(ops, gold, name, case):
    got = G.run_case(GpuOps(ops), case)
    want = gold[name]
    fam = case["fam"]
    if fam == "transform" and case["op"] in LIBM:
        if case["op"] in CANCELLING:
            scale = np.maximum(np.abs(want), 1.0).astype(np.float32)
            assert (np.abs(got.astype(np.float64) - want) / np.spacing(scale)).max() <= 8
        else:
            assert ulp_distance(got, want).max() <= 2
    elif fam == "transform" and case["op"] == 50:
        assert ulp_distance(got, want).max() <= 2      # 3*x*x: grouping differs inside the reference build
    elif fam == "scalar" and case["op"] == 3:
        assert ulp_distance(got, want).max() <= 1      # the reference multiplies by a hoisted 1/scalar
    elif fam in ("reduce", "reduce3", "reduce3_all", "stats"):
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=2e-6)
    elif fam == "softmax":
        finite = np.isfinite(want)
        np.testing.assert_allclose(got[finite], want[finite], rtol=1e-5, atol=1e-7 if case["op"] != 40 else 1e-5)
        assert np.array_equal(np.isneginf(got), np.isneginf(want))
    elif fam == "random":
        n = case["n"]
        for k, (op, arity, extra) in enumerate(case["calls"]):
            a, b = got[k * n:(k + 1) * n], want[k * n:(k + 1) * n]
            if op == 6:
                np.testing.assert_allclose(a, b, atol=1e-5, rtol=0)
            else:
                np.testing.assert_array_equal(a, b)
        np.testing.assert_array_equal(got[-2:], want[-2:])
    else:
        # index reductions, arithmetic transforms / pairwise / scalar / broadcast, Binomial / Choice / Uniform
        np.testing.assert_array_equal(got, want)
