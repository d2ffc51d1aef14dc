"""The whole-array transforms against the committed outputs of the reference's CPU code
(tests/golden/special_transforms_golden.npz, made by tests/golden/make_special_golden.py): the numpy restatements
on CPU and the CUDA path on the GPU, on machines where the reference checkout is absent."""
import os

import numpy as np
import pytest

from tests import special_golden_cases as G
from tests import special_truth as T
from tests.cases import Layout

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "special_transforms_golden.npz")
CASES = list(G.cases())


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def same(got, want, case):
    if case[0] == "pooling" and case[3] != 0:      # the reference leaves the order of these sums to the compiler
        return np.allclose(got, want, rtol=1e-5, atol=1e-6, equal_nan=True)
    return np.array_equal(got, want, equal_nan=True)


def test_every_case_has_a_record(golden):
    assert sorted(golden.files) == sorted(name for name, _ in CASES)


@pytest.mark.parametrize("name,case", CASES, ids=[n for n, _ in CASES])
def test_restatement_matches_the_reference_output(golden, name, case):
    op, x, x_info, z, z_info, extra = G.build(case)
    kind = case[0]
    want = golden[name]
    if kind == "histogram":
        assert np.array_equal(T.histogram(x, z, case[2], -1.5, 2.5), want)
        return
    if kind == "reverse":
        shape, kinds = case[1], case[2]
        logical = np.random.default_rng(len(shape)).standard_normal(shape).astype(np.float32)
        lx, lz = Layout(logical, kinds[0]), Layout(np.zeros(shape, np.float32), kinds[1])
        from tests.test_oracle_special_transforms import offsets
        mine = lz.buffer.copy()
        mine[offsets(lz)[::-1]] = lx.buffer[offsets(lx)]
        assert np.array_equal(mine, want, equal_nan=True)
        return
    g, kinds = case[1], case[2]
    b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
    oH, oW = T.out_size(h, kH, sH, pH, dH), T.out_size(w, kW, sW, pW, dW)
    rng = np.random.default_rng(sum(g) + len(kind))
    if kind == "im2col":
        logical = rng.standard_normal((b, c, h, w)).astype(np.float32)
        lz = Layout(np.zeros((b, c, kH, kW, oH, oW), np.float32), kinds[1])
        assert np.array_equal(lz.read(want).reshape(b, c, kH, kW, oH, oW), T.im2col(logical, kH, kW, sH, sW, pH, pW, dH, dW, oH, oW))
    elif kind == "col2im":
        logical = rng.standard_normal((b, c, kH, kW, oH, oW)).astype(np.float32)
        lz = Layout(np.zeros((b, c, h, w), np.float32), kinds[1])
        assert np.array_equal(lz.read(want).reshape(b, c, h, w), T.col2im(logical, sH, sW, pH, pW, h, w, dH, dW))
    else:
        logical = rng.standard_normal((b, c, h, w)).astype(np.float32)
        lz = Layout(np.zeros((b, c, oH, oW), np.float32), kinds[1])
        mine = T.pooling2d(logical, kH, kW, sH, sW, pH, pW, dH, dW, oH, oW, case[3], case[4])
        got = lz.read(want).reshape(b, c, oH, oW).astype(np.float64)
        assert same(got, mine, case)


@pytest.mark.gpu
@pytest.mark.parametrize("name,case", CASES, ids=[n for n, _ in CASES])
def test_cuda_path_matches_the_reference_output(ops, golden, name, case):
    import torch
    op, x, x_info, z, z_info, extra = G.build(case)
    dx, dz = torch.from_numpy(x.copy()).cuda(), torch.from_numpy(z.copy()).cuda()
    ops.execTransformFloat(None, op, dx, x_info, dz, z_info, None if extra is None else torch.from_numpy(extra).cuda())
    assert same(dz.cpu().numpy(), golden[name], case), name
