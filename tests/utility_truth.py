"""numpy restatements of the reference's memory-movement loops, shared by the GPU tests (expected values)
and by tests/test_oracle_utilities.py, which pins each of them against the reference's own CPU NativeOps
members compiled into oracle/_ref (oracle/ref_nativeops.cpp)."""
import numpy as np


def flatten_truth(z_before, offset, order, logical):
    """blas/cpu/NativeOps.cpp:1530-1660: x enumerated in `order` lands at z[offset:]."""
    want = z_before.copy()
    want[offset:offset + logical.size] = logical.ravel(order="C" if order == "c" else "F")
    return want


def average_truth(xs, dt):
    """include/ops/impl/specials.cpp:374-433: z = sum_k x_k / n, every step rounded to the element type."""
    n = len(xs)
    acc = np.zeros(xs[0].size, dt)
    for t in xs:
        acc = (acc + (t / dt(n)).astype(dt)).astype(dt)
    return acc


def accumulate_truth(xs, start, dt):
    """include/ops/impl/specials.cpp:344-371: z += x_k in source order, rounded after each addition."""
    acc = start.copy()
    for t in xs:
        acc = (acc + t).astype(dt)
    return acc


def shuffled(x, axis, shuffle_map):
    """The reference's loop: swaps applied one after another (blas/cpu/NativeOps.cpp:2289-2324)."""
    out = np.moveaxis(x.copy(), axis, 0)
    for r in range(out.shape[0]):
        m = shuffle_map[r]
        if m < 0:
            continue
        tmp = out[r].copy()
        out[r] = out[m]
        out[m] = tmp
    return np.moveaxis(out, 0, axis)


def half_map(n, rng):
    """The usual map: every TAD of the first half meets one of the second half, nothing else moves."""
    m = np.full(n, -1, np.int32)
    m[:n // 2] = n // 2 + rng.permutation(n // 2)
    return m


MAPS = {
    "pairs": lambda n, rng: half_map(n, rng),
    "chain": lambda n, rng: np.array([r + 1 if r + 1 < n else -1 for r in range(n)], np.int32),
    "random": lambda n, rng: rng.integers(-1, n, n).astype(np.int32),
    "identity": lambda n, rng: np.arange(n, dtype=np.int32),
}


def sort_values(rng, n, dt):
    x = (rng.standard_normal(n) * 100).astype(dt)
    if n > 8:
        x[:4] = [np.inf, -np.inf, 0.0, x[5]]          # infinities (the padding value) and a duplicate
    return x


def coo_sorted(indices, values):
    """Rows of `indices` (length x rank) in lexicographic order with their values carried along
    (include/ops/impl/specials_sparse.cpp: quicksort on coordinate tuples)."""
    order = np.lexsort(indices.T[::-1])
    return indices[order], values[order]
