"""Edge cases of the hot path on the GPU: empty and one-element operands, lengths that are not a
multiple of the 128-bit pack, operands that do not start on a 16-byte boundary, TADs of length 1,
a single TAD, millions of tiny TADs, and tile counts beyond 65535."""
import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S
from tests.cases import result_info

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.mark.parametrize("n", [0, 1, 2, 3, 5, 255, 257])
def test_elementwise_tiny_and_ragged_lengths(ops, n):
    x = np.arange(n, dtype=np.float32) - 2
    y = np.full(n, 3, np.float32)
    info = S.shape_info([1, max(n, 1)]) if n else S.shape_info([1, 1])
    if n == 0:
        # the reference has no empty arrays (a shape holds at least one element); a zero-length
        # strided call is the empty case of this interface and must be a no-op
        z = torch.full((4,), 9.0, device="cuda")
        ops.execTransformFloat(None, 0, z, 1, z, 1, None, 0)
        ops.execPairwiseTransformFloat(None, 0, z, 1, z, 1, z, 1, None, 0)
        ops.execScalarFloat(None, 0, z, 1, z, 1, 1.0, None, 0)
        assert (host(z) == 9).all()
        return
    dz = torch.zeros(n, device="cuda")
    ops.execTransformFloat(None, 0, dev(x), info, dz, info, None)          # Abs
    np.testing.assert_array_equal(host(dz), np.abs(x))
    ops.execPairwiseTransformFloat(None, 6, dev(x), info, dev(y), info, dz, info, None)   # Multiply
    np.testing.assert_array_equal(host(dz), x * y)
    ops.execScalarFloat(None, 0, dev(x), info, dz, info, 0.5, None)
    np.testing.assert_array_equal(host(dz), x + np.float32(0.5))


@pytest.mark.parametrize("offset", [1, 2, 3])
def test_operands_off_the_16_byte_boundary(ops, offset):
    """Sub-buffers starting 4, 8 or 12 bytes into an allocation take the scalar-load paths."""
    n = 10007
    rng = np.random.default_rng(offset)
    x = rng.standard_normal(n + 8).astype(np.float32)
    dx, dz = dev(x), torch.zeros(n + 8, device="cuda")
    info = S.shape_info([1, n])
    ops.execTransformFloat(None, 0, dx[offset:], info, dz[offset:], info, None)
    np.testing.assert_array_equal(host(dz)[offset:offset + n], np.abs(x[offset:offset + n]))
    assert host(dz)[:offset].sum() == 0 and host(dz)[offset + n:].sum() == 0
    # reductions: rows of a [50, 200] array that starts off the boundary
    m = x[offset:offset + 10000].reshape(50, 200)
    xi, zi = S.shape_info([50, 200]), result_info((50, 200), [1])
    out = torch.zeros(50, device="cuda")
    ops.execReduceFloat(None, 1, dx[offset:], xi, None, out, zi, [1], 1)
    np.testing.assert_allclose(host(out), m.astype(np.float64).sum(1), rtol=1e-5, atol=1e-5)
    outc = torch.zeros(200, device="cuda")
    ops.execReduceFloat(None, 1, dx[offset:], xi, None, outc, result_info((50, 200), [0]), [0], 1)
    np.testing.assert_allclose(host(outc), m.astype(np.float64).sum(0), rtol=1e-5, atol=1e-5)
    idx = torch.zeros(50, device="cuda")
    ops.execIndexReduceFloat(None, 0, dx[offset:], xi, None, idx, zi, [1], 1)
    np.testing.assert_array_equal(host(idx), m.argmax(1))


def test_tads_of_length_one_and_a_single_tad(ops):
    x = np.arange(1, 4097, dtype=np.float32)
    xi = S.shape_info([4096, 1])
    out = torch.zeros(4096, device="cuda")
    ops.execReduceFloat(None, 1, dev(x), xi, None, out, S.shape_info([4096, 1]), [1], 1)     # every TAD is one element
    np.testing.assert_array_equal(host(out), x)
    idx = torch.full((4096,), -1.0, device="cuda")
    ops.execIndexReduceFloat(None, 0, dev(x), xi, None, idx, S.shape_info([4096, 1]), [1], 1)
    assert (host(idx) == 0).all()
    one = torch.zeros(1, device="cuda")
    ops.execReduceFloat(None, 1, dev(x), xi, None, one, S.shape_info([1, 1]), [0], 1)        # one TAD: the whole column
    assert host(one)[0] == x.astype(np.float64).sum()
    var = torch.zeros(4096, device="cuda")
    ops.execSummaryStatsFloat(None, 0, dev(x), xi, None, var, S.shape_info([4096, 1]), [1], 1, True)
    assert (host(var) == 0).all()          # one observation: variance 0, as in the reference


def test_millions_of_tiny_tads_and_wide_tiles(ops):
    rng = np.random.default_rng(1)
    x = rng.integers(-8, 8, (1 << 21, 3)).astype(np.float32)       # 2M TADs of 3 elements
    xi = S.shape_info(list(x.shape))
    out = torch.zeros(x.shape[0], device="cuda")
    ops.execReduceFloat(None, 1, dev(x), xi, None, out, S.shape_info([x.shape[0], 1]), [1], 1)
    np.testing.assert_array_equal(host(out), x.sum(1))
    # dimension-0 reduction of a very wide, short array: 2^23 columns -> 65536 column tiles of 128
    w = rng.integers(-8, 8, (3, 1 << 23)).astype(np.float32)
    wi = S.shape_info(list(w.shape))
    outw = torch.zeros(w.shape[1], device="cuda")
    ops.execReduceFloat(None, 1, dev(w), wi, None, outw, S.shape_info([1, w.shape[1]]), [0], 1)
    np.testing.assert_array_equal(host(outw), w.sum(0))
    idx = torch.zeros(w.shape[1], device="cuda")
    ops.execIndexReduceFloat(None, 0, dev(w), wi, None, idx, S.shape_info([1, w.shape[1]]), [0], 1)
    np.testing.assert_array_equal(host(idx), w.argmax(0))


def test_whole_array_reductions_at_awkward_lengths(ops):
    for n in (1, 2, 31, 33, 1023, 65537, (1 << 24) + 5):
        x = np.ones(n, np.float32)
        x[n // 2] = 5
        info = S.shape_info([1, n])
        assert ops.execReduceScalarFloat(None, 1, dev(x), info, None) == np.float32(n + 4)   # exact up to float rounding of the result
        assert ops.execIndexReduceScalarFloat(None, 0, dev(x), info, None) == n // 2


def test_two_streams_and_two_host_threads_do_not_share_scratch(ops):
    """Split reductions keep partial states and arrival counters in a per-stream workspace: calls issued
    concurrently from two host threads on two streams must not disturb each other."""
    import threading
    rng = np.random.default_rng(2)
    data = [rng.integers(-4, 5, (2048, 4096)).astype(np.float32) for _ in range(2)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    results = [None, None]

    def worker(k):
        torch.cuda.set_device(0)
        st = streams[k]
        extra = [None, st.cuda_stream]
        with torch.cuda.stream(st):
            dx = dev(data[k])
            cols = torch.zeros(4096, device="cuda")
            out = []
            xi = S.shape_info([2048, 4096])
            for _ in range(30):
                ops.execReduceFloat(extra, 1, dx, xi, None, cols, S.shape_info([1, 4096]), [0], 1)   # split across-TAD
                total = ops.execReduceScalarFloat(extra, 1, dx, xi, None)                             # split whole-array
                out.append((host(cols).copy(), total))
        results[k] = out

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for k in range(2):
        want_cols, want_total = data[k].sum(0), float(data[k].astype(np.float64).sum())
        for cols, total in results[k]:
            np.testing.assert_array_equal(cols, want_cols)      # small integers: exact in any order
            assert total == want_total


@pytest.mark.parametrize("shape", [(64, 2000, 40), (48, 3000, 37), (3, 5000, 260)])
def test_middle_axis_reductions_split_into_clusters(ops, shape):
    """Reductions over the middle axis of rank-3 arrays: neighbouring TADs are adjacent, every TAD is a long
    strided walk that is cut into segments (thread-block clusters plus, for the longest, arrival counters),
    tiles are only partly filled, and the odd width takes the scalar-load path. Small integers: exact."""
    rng = np.random.default_rng(shape[2])
    x = rng.integers(-6, 7, shape).astype(np.float32)
    y = rng.integers(-6, 7, shape).astype(np.float32)
    xi = S.shape_info(list(shape))
    zi = S.shape_info([shape[0], 1, shape[2]])
    n = shape[0] * shape[2]
    dx, dy = dev(x), dev(y)
    out = torch.zeros(n, device="cuda")
    ops.execReduceFloat(None, 1, dx, xi, None, out, zi, [1], 1)
    np.testing.assert_array_equal(host(out).reshape(shape[0], shape[2]), x.sum(1))
    ops.execIndexReduceFloat(None, 0, dx, xi, None, out, zi, [1], 1)
    np.testing.assert_array_equal(host(out).reshape(shape[0], shape[2]), x.argmax(1))
    ops.execReduce3Float(None, 0, dx, xi, None, dy, xi, out, zi, [1], 1)          # Manhattan: exact on integers
    np.testing.assert_array_equal(host(out).reshape(shape[0], shape[2]), np.abs(x - y).sum(1))
    ops.execSummaryStatsFloat(None, 0, dx, xi, None, out, zi, [1], 1, True)
    np.testing.assert_allclose(host(out).reshape(shape[0], shape[2]), x.astype(np.float64).var(1, ddof=1), rtol=1e-5)
    for cluster in (1, 2, 8):                 # same results whatever the cluster size
        ops.lib.nd4jb200_set_tuning(4, cluster)
        ops.execReduceFloat(None, 1, dx, xi, None, out, zi, [1], 1)
        np.testing.assert_array_equal(host(out).reshape(shape[0], shape[2]), x.sum(1))
    ops.lib.nd4jb200_set_tuning(4, 4)
