"""Pins the oracle. (1) The port (oracle/port.c + port.py) against the golden vectors generated
from the reference's own CPU build; (2) the port against the live reference build on further
seeded inputs; (3) the reference build against the known answers of the reference's own tests.
CPU only."""
import os

import numpy as np
import pytest

from libnd4j_b200 import shape as S
from oracle import port as port_mod
from tests import golden_cases as G
from tests.cases import Layout, rand_input, result_info, ulp_distance

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "legacy_ops_golden.npz")


@pytest.fixture(scope="module")
def port():
    return port_mod.Port()


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


# libm-backed results may differ in the last place between glibc builds; everything else is exact
LIBM_TRANSFORMS = {2, 3, 5, 10, 12, 13, 15, 16, 17, 18, 21, 22, 23, 29, 53, 54, 61, 62, 63, 64, 65, 67, 68, 74, 78,
                   86, 88, 90, 91}


PORT_CASES = [(n, c) for n, c in G.cases() if c.get("port", True)]


@pytest.mark.parametrize("name,case", PORT_CASES, ids=[n for n, _ in PORT_CASES])
def test_port_matches_golden(port, gold, name, case):
    got = G.run_case(port, case)
    want = gold[name]
    fam = case["fam"]
    if fam == "transform" and case["op"] in LIBM_TRANSFORMS:
        # the reference is built with associative-math / reciprocal-math, so composite formulas
        # are evaluated in a slightly different order than written: compare in ulps of the larger
        # of the result and the O(1) intermediates
        scale = np.maximum(np.abs(want), 1.0).astype(np.float32)
        assert (np.abs(got.astype(np.float64) - want) / np.spacing(scale)).max() <= 4
        if case["op"] in (2, 3, 5, 12, 15, 16, 17, 18, 63, 64, 65, 78, 86, 90):   # a single libm call
            assert ulp_distance(got, want).max() <= 1
    elif fam == "transform" and case["op"] == 50:
        # 3*x*x is grouped differently by the reference's single-thread and OpenMP code paths
        assert ulp_distance(got, want).max() <= 2
    elif fam == "scalar" and case["op"] == 3:
        # x / scalar: the reference's reciprocal-math build multiplies by a hoisted 1/scalar
        assert ulp_distance(got, want).max() <= 1
    elif fam in ("reduce", "reduce3", "reduce3_all", "stats"):
        np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-6)
    elif fam == "softmax":
        finite = np.isfinite(want)
        np.testing.assert_allclose(got[finite], want[finite], rtol=2e-6, atol=1e-7 if case["op"] != 40 else 2e-6)
        assert np.array_equal(np.isneginf(got), np.isneginf(want))
    elif fam == "random":
        n = case["n"]
        for k, (op, arity, extra) in enumerate(case["calls"]):
            a, b = got[k * n:(k + 1) * n], want[k * n:(k + 1) * n]
            if op == 6:
                np.testing.assert_allclose(a, b, atol=2e-6, rtol=0)
            else:
                np.testing.assert_array_equal(a, b)
        np.testing.assert_array_equal(got[-2:], want[-2:])
    else:
        np.testing.assert_array_equal(got, want)


def test_port_rng_matches_golden_probes(port, gold):
    state, table = port.init_random(119, 100000)
    np.testing.assert_array_equal(table[:8], gold["rng/table_head"])
    np.testing.assert_array_equal(table[-4:], gold["rng/table_tail"])
    got = np.array([port.rng_element(state, p) for p in G.RNG_PROBES], dtype=np.uint64)
    np.testing.assert_array_equal(got, gold["rng/elements"])
    # values the reference prints for this fixture (seed 119, table of 100000 words)
    assert table[0] == 7465776281147007380 and table[3] == 11482182524184260395
    assert got[3] == 4744429461797627110 and got[5] == 511762323991934140


def test_port_tad_matches_golden(port, gold):
    for i, (shape, order, dims) in enumerate(G.TAD_CASES):
        info, offs = port.tad(S.shape_info(shape, order), dims)
        np.testing.assert_array_equal(info, gold["tad/%d/info" % i])
        np.testing.assert_array_equal(offs, gold["tad/%d/offsets" % i])


def test_reference_known_answers(real_ref):
    """Known answers of the reference's own tests, run on the reference build."""
    x = np.array([1, 2, 3, 4], dtype=np.float32)
    y = np.arange(1, 17, dtype=np.float32)
    z = real_ref.reduce3(1, x, S.shape_info([1, 4]), y, S.shape_info([4, 4]), np.zeros(4, np.float32),
                         S.shape_info([4, 1]), [1])
    np.testing.assert_array_equal(z, [0, 8, 16, 24])                      # Reduce3Tests.cpp:10-45
    lin = np.arange(1, 26, dtype=np.float64)
    info = S.shape_info([5, 5])
    assert real_ref.index_reduce_scalar(0, lin, info) == 24               # LegacyOpsTests.cpp:222-239
    z = real_ref.index_reduce(0, lin, info, np.zeros(5), S.shape_info([5, 1]), [1])
    np.testing.assert_array_equal(z, [4, 4, 4, 4, 4])                     # LegacyOpsTests.cpp:242-261
    m = np.arange(1, 13, dtype=np.float32)
    z = real_ref.reduce(1, m, S.shape_info([4, 3]), np.zeros(4, np.float32), S.shape_info([4, 1]), [1])
    np.testing.assert_array_equal(z, [6, 15, 24, 33])


def test_port_known_answers(port):
    x = np.array([1, 2, 3, 4], dtype=np.float32)
    y = np.arange(1, 17, dtype=np.float32)
    z = port.reduce3(1, x, S.shape_info([1, 4]), y, S.shape_info([4, 4]), np.zeros(4, np.float32), S.shape_info([4, 1]), [1])
    np.testing.assert_array_equal(z, [0, 8, 16, 24])
    lin = np.arange(1, 26, dtype=np.float32)
    info = S.shape_info([5, 5])
    assert port.index_reduce_scalar(0, lin, info) == 24
    np.testing.assert_array_equal(port.index_reduce(0, lin, info, np.zeros(5, np.float32), S.shape_info([5, 1]), [1]), [4] * 5)


@pytest.mark.parametrize("kind", ["c", "f", "cview2", "fview2", "rowview2"])
@pytest.mark.parametrize("shape,dims", [((9, 14), [1]), ((9, 14), [0]), ((4, 5, 6), [0, 2]), ((3, 4, 5, 2), [1, 3])])
def test_port_vs_live_reference_layouts(port, real_ref, kind, shape, dims):
    rng = np.random.default_rng(len(shape) * 7 + len(kind))
    x = rand_input(rng, shape, np.float32, "levels")
    lx = Layout(x, kind)
    zi = result_info(shape, dims)
    n = S.length(zi)
    for fn in ("reduce", "index_reduce"):
        op = 1 if fn == "reduce" else 0
        want = getattr(real_ref, fn)(op, lx.buffer, lx.info, np.zeros(n, np.float32), zi, dims)
        got = getattr(port, fn)(op, lx.buffer, lx.info, np.zeros(n, np.float32), zi, dims)
        np.testing.assert_array_equal(got, want)
    lz = Layout(np.zeros(shape, np.float32), kind)
    zb1, zb2 = lz.buffer.copy(), lz.buffer.copy()
    real_ref.transform(6, lx.buffer, lx.info, zb1, lz.info)
    port.transform(6, lx.buffer, lx.info, zb2, lz.info)
    np.testing.assert_array_equal(lz.read(zb1), lz.read(zb2))


def test_port_vs_live_reference_random_states(port, real_ref):
    ps, _ = port.init_random(4242, 5000)
    rs, _ = real_ref.init_random(4242, 5000)
    zi = S.shape_info([1, 17003])
    for op, extra in ((0, [0, 1]), (7, [0.4]), (0, [1, 2])):
        a = port.random(op, ps, np.zeros(17003, np.float32), zi, np.array(extra, np.float32))
        b = real_ref.random(op, rs, np.zeros(17003, np.float32), zi, np.array(extra, np.float32))
        np.testing.assert_array_equal(a, b)
    port.reseed(ps, 99)
    real_ref.reseed(rs, 99)
    a = port.random(0, ps, np.zeros(17003, np.float32), zi, np.array([0, 1], np.float32))
    b = real_ref.random(0, rs, np.zeros(17003, np.float32), zi, np.array([0, 1], np.float32))
    np.testing.assert_array_equal(a, b)
    assert port.rng_position(ps) == real_ref.rng_position(rs) and port.rng_generation(ps) == real_ref.rng_generation(rs)


def test_convert_types_restatement_matches_reference(real_ref):
    """The numpy restatement the GPU tests use, against NativeOps::convertTypes of the reference itself: every
    served pair, including the out-of-range, NaN and uint16 low-byte cases, and the pairs it leaves untouched."""
    from tests.convert_truth import CODES, SOURCES, RESULTS, convert_truth, convert_inputs
    for src in SOURCES:
        x = convert_inputs(src)
        for dst in RESULTS:
            z = real_ref.convert_types(CODES[src], x, CODES[dst], np.full(x.size, 7, dst))
            if src == dst and src in (np.int8, np.float32, np.float64):
                assert (z == 7).all()
                continue
            want = convert_truth(x, dst)
            if np.issubdtype(dst, np.floating):
                nan = np.isnan(want)
                assert np.array_equal(np.isnan(z), nan)
                z, want = np.where(nan, 0, z).astype(dst), np.where(nan, 0, want).astype(dst)
            assert np.array_equal(z.view(np.uint8), want.view(np.uint8)), (src, dst)


def test_float8_restatement_matches_reference(real_ref):
    """float8 <-> everything through NativeOps::convertTypes of the reference itself: all 256 float8 values as
    sources, and a dense sweep of floats (every exponent, the thresholds, NaN, infinities) as float8 results."""
    from tests import convert_truth as C
    q = C.float8_inputs()
    for dst in C.RESULTS:
        z = real_ref.convert_types(C.FLOAT8, q, C.CODES[dst], np.full(q.size, 7, dst))
        want = C.convert_truth_from_float8(q, dst)
        if np.issubdtype(dst, np.floating):
            nan = np.isnan(want)
            assert np.array_equal(np.isnan(z), nan)
            z, want = np.where(nan, 0, z).astype(dst), np.where(nan, 0, want).astype(dst)
        assert np.array_equal(z.view(np.uint8), want.view(np.uint8)), dst
    rng = np.random.default_rng(0)
    bits = np.concatenate([rng.integers(0, 2 ** 32, 200000, dtype=np.uint64).astype(np.uint32),
                           np.arange(0x33000000 - 40, 0x33000000 + 40, dtype=np.uint32),
                           np.arange(0x477FEFFF - 40, 0x477FEFFF + 40, dtype=np.uint32)])
    f = bits.view(np.float32)
    got = real_ref.convert_types(C.CODES[np.float32], f.copy(), C.FLOAT8, np.full(f.size, 9, np.uint8))
    np.testing.assert_array_equal(got, C.float_to_float8(f))
    for src in C.SOURCES:
        x = C.convert_inputs(src)
        got = real_ref.convert_types(C.CODES[src], x, C.FLOAT8, np.full(x.size, 9, np.uint8))
        np.testing.assert_array_equal(got, C.convert_truth_to_float8(x), err_msg=str(src))
