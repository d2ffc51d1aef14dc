"""The list of golden cases shared by the generator (tests/golden/make_golden.py), the oracle
tests and the GPU tests. A case is a dict; inputs are re-created from (seed, kind, shape)."""
import numpy as np

from libnd4j_b200 import shape as S
from tests.cases import Layout, rand_input, result_info

RNG_PROBES = [0, 1, 99999, 100000, 100001, 250007, 1 << 20, (1 << 30) + 5]

TAD_CASES = [((4, 5), "c", [0]), ((4, 5), "c", [1]), ((4, 5), "f", [0]), ((4, 5), "f", [1]),
             ((2, 3, 4), "c", [0]), ((2, 3, 4), "c", [1]), ((2, 3, 4), "c", [2]), ((2, 3, 4), "c", [0, 1]),
             ((2, 3, 4), "c", [0, 2]), ((2, 3, 4), "c", [1, 2]), ((2, 3, 4), "f", [0]), ((2, 3, 4), "f", [1]),
             ((2, 3, 4), "f", [2]), ((2, 3, 4), "f", [0, 1]), ((2, 3, 4), "f", [0, 2]), ((2, 3, 4), "f", [1, 2]),
             ((2, 3, 4, 5), "c", [1, 2]), ((2, 3, 4, 5), "c", [0, 3]), ((2, 3, 4, 5), "c", [1, 2, 3]),
             ((2, 3, 4, 5), "c", [0, 2, 3]), ((2, 3, 4, 5), "f", [1, 3]), ((8192, 4096), "c", [1]),
             ((8192, 4096), "c", [0]), ((6, 7, 8, 9, 3), "c", [0, 2, 4]), ((6, 7, 8, 9, 3), "f", [1, 3])]

TRANSFORM_OPS = [0, 1, 2, 3, 4, 5, 6, 8, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23, 24, 25, 26, 27, 29, 30,
                 35, 42, 47, 49, 50, 51, 52, 53, 54, 61, 62, 63, 64, 65, 67, 68, 74, 76, 78, 86, 87, 88, 90, 91, 94, 95]
TRANSFORM_POSITIVE = {5, 14, 76}
PAIRWISE_OPS = [0, 1, 2, 3, 4, 5, 6, 8, 9, 11, 12, 13, 14, 15, 18, 22, 24]
REDUCE_OPS = [0, 1, 3, 4, 5, 6, 7, 8, 11, 13, 14, 15, 20, 21, 22, 23, 25, 26]


def cases():
    for op in TRANSFORM_OPS:
        yield "transform/%d" % op, dict(fam="transform", op=op, seed=1000 + op, n=513,
                                        kind="positive" if op in TRANSFORM_POSITIVE else ("uniform" if op in (16, 17) else "normal"))
    for op in PAIRWISE_OPS:
        yield "pairwise/%d" % op, dict(fam="pairwise", op=op, seed=2000 + op, n=300)
    for op in range(0, 14):
        yield "scalar/%d" % op, dict(fam="scalar", op=op, seed=3000 + op, n=300, scalar=1.75)
    for op in range(0, 18):
        yield "broadcast/%d" % op, dict(fam="broadcast", op=op, seed=4000 + op, shape=(7, 12), dims=[1])
    for op in REDUCE_OPS:
        for shape, dims, kind in (((9, 40), [1], "c"), ((9, 40), [0], "c"), ((4, 5, 6), [0, 2], "f")):
            yield "reduce/%d/%s%s%s" % (op, "x".join(map(str, shape)), "d" + "".join(map(str, dims)), kind), \
                dict(fam="reduce", op=op, seed=5000 + op, shape=shape, dims=dims, layout=kind)
    for op in range(4):
        for shape, dims, kind in (((12, 33), [1], "c"), ((12, 33), [0], "c"), ((4, 5, 6), [1, 2], "f")):
            yield "index/%d/%s%s%s" % (op, "x".join(map(str, shape)), "d" + "".join(map(str, dims)), kind), \
                dict(fam="index", op=op, seed=6000 + op, shape=shape, dims=dims, layout=kind)
    for op in (0, 1):
        for bias in (0, 1):
            yield "stats/%d/%d" % (op, bias), dict(fam="stats", op=op, seed=7000 + op, shape=(50, 16), dims=[0], bias=bias)
    for op in (0, 1, 2, 3, 5, 6, 7):
        yield "reduce3/%d" % op, dict(fam="reduce3", op=op, seed=8000 + op, shape=(10, 64), dims=[1])
    seq = [(0, 0, [0.0, 1.0]), (6, 2, [0.0, 1.0]), (7, 0, [0.3]), (2, 1, [0.5]), (0, 0, [-2.0, 3.0]), (1, 1, [0.8])]
    yield "random/sequence", dict(fam="random", seed=119, table=100000, n=70001, calls=seq)
    for op in (0, 1, 2, 3, 5, 6, 7):
        yield "reduce3_all/%d" % op, dict(fam="reduce3_all", op=op, seed=9000 + op, xshape=(9, 37), yshape=(5, 37), dims=[1])
    for op in (38, 39, 40):
        for shape in ((12, 10), (5, 700)):
            yield "softmax/%d/%dx%d" % (op, shape[0], shape[1]), dict(fam="softmax", op=op, seed=9100 + op, shape=shape)
    yield "random/special", dict(fam="random_special", seed=119, table=100000, n=3001, trials=5, choices=23)


def _inputs(case):
    rng = np.random.default_rng(case["seed"])
    return rng


def run_case(ref, case):
    """Runs one case on a Reference-like object and returns the output array."""
    fam, rng = case["fam"], _inputs(case)
    if fam == "transform":
        x = rand_input(rng, case["n"], np.float32, case["kind"])
        info = S.shape_info([1, case["n"]])
        return ref.transform(case["op"], x, info, np.empty_like(x), info)
    if fam == "pairwise":
        kind = "levels" if case["op"] in (3, 15) else "normal"
        x, y = rand_input(rng, case["n"], np.float32, kind), rand_input(rng, case["n"], np.float32, kind)
        info = S.shape_info([1, case["n"]])
        return ref.pairwise(case["op"], x, info, y, info, np.empty_like(x), info)
    if fam == "scalar":
        x = rand_input(rng, case["n"], np.float32)
        info = S.shape_info([1, case["n"]])
        return ref.scalar(case["op"], x, info, np.empty_like(x), info, case["scalar"])
    if fam == "broadcast":
        x = rand_input(rng, case["shape"], np.float32)
        y = rand_input(rng, case["shape"][1], np.float32)
        xi, yi = S.shape_info(case["shape"]), S.shape_info([1, case["shape"][1]])
        return ref.broadcast(case["op"], x.ravel(), xi, y, yi, np.empty(x.size, np.float32), xi, case["dims"])
    if fam in ("reduce", "index"):
        kind = "levels" if (fam == "index" or case["op"] in (22, 26)) else ("near1" if case["op"] in (8, 21) else "normal")
        x = (1.0 + rng.uniform(-0.01, 0.01, case["shape"])).astype(np.float32) if kind == "near1" \
            else rand_input(rng, case["shape"], np.float32, kind)
        lx = Layout(x, case["layout"])
        zi = result_info(case["shape"], case["dims"])
        z = np.zeros(S.length(zi), np.float32)
        fn = ref.reduce if fam == "reduce" else ref.index_reduce
        return fn(case["op"], lx.buffer, lx.info, z, zi, case["dims"])
    if fam == "stats":
        x = (rand_input(rng, case["shape"], np.float64) * 2 + 10).astype(np.float32)
        xi, zi = S.shape_info(case["shape"]), result_info(case["shape"], case["dims"])
        return ref.summary_stats(case["op"], x.ravel(), xi, np.zeros(S.length(zi), np.float32), zi, case["dims"], bool(case["bias"]))
    if fam == "reduce3":
        kind = "positive" if case["op"] == 6 else ("levels" if case["op"] == 7 else "normal")
        x, y = rand_input(rng, case["shape"], np.float32, kind), rand_input(rng, case["shape"], np.float32, kind)
        xi, zi = S.shape_info(case["shape"]), result_info(case["shape"], case["dims"])
        return ref.reduce3(case["op"], x.ravel(), xi, y.ravel(), xi, np.zeros(S.length(zi), np.float32), zi, case["dims"])
    if fam == "random":
        state, _ = ref.init_random(case["seed"], case["table"])
        n = case["n"]
        zi = S.shape_info([1, n])
        xs = rand_input(rng, n, np.float32)
        outs = []
        for op, arity, extra in case["calls"]:
            z = np.zeros(n, np.float32)
            ex = np.array(extra, np.float32)
            if arity == 0:
                ref.random(op, state, z, zi, ex)
            elif arity == 1:
                ref.random_x(op, state, xs, zi, z, zi, ex)
            else:
                ref.random_xy(op, state, z, zi, z, zi, z, zi, ex)
            outs.append(z)
        outs.append(np.array([ref.rng_position(state), ref.rng_generation(state)], np.float32))
        ref.destroy_random(state)
        return np.concatenate(outs)
    if fam == "reduce3_all":
        kind = "positive" if case["op"] == 6 else ("levels" if case["op"] == 7 else "normal")
        x, y = rand_input(rng, case["xshape"], np.float32, kind), rand_input(rng, case["yshape"], np.float32, kind)
        xi, yi = S.shape_info(case["xshape"]), S.shape_info(case["yshape"])
        nz = case["xshape"][0] * case["yshape"][0]
        zi = S.shape_info([case["xshape"][0], case["yshape"][0]])
        return ref.reduce3_all(case["op"], x.ravel(), xi, y.ravel(), yi, np.zeros(nz, np.float32), zi, case["dims"])
    if fam == "softmax":
        x = (rand_input(rng, case["shape"], np.float32) * 3).astype(np.float32).ravel()
        info = S.shape_info(case["shape"])
        z = x.copy()                      # in place: the derivative is only well defined that way in the reference
        return ref.transform(case["op"], z, info, z, info)
    if fam == "random_special":
        # Binomial (scalar probability, then one probability per trial), BinomialEx, Choice, then a Uniform call
        # whose values show that the state advanced as in the reference
        state, _ = ref.init_random(case["seed"], case["table"])
        n, trials, k = case["n"], case["trials"], case["choices"]
        zi, ti, ki = S.shape_info([1, n]), S.shape_info([1, trials]), S.shape_info([1, k])
        ex = np.array([trials, 0.4], np.float32)
        outs = []
        z = np.zeros(n, np.float32)
        outs.append(ref.random_xy(8, state, z, zi, z, zi, z, zi, ex).copy())
        probs = rng.uniform(0.1, 0.9, trials).astype(np.float32)
        z = np.zeros(n, np.float32)
        outs.append(ref.random_xy(8, state, z, zi, probs, ti, z, zi, ex).copy())
        pe = rng.uniform(0.0, 1.0, n).astype(np.float32)
        z = np.zeros(n, np.float32)
        outs.append(ref.random_xy(9, state, z, zi, pe, zi, z, zi, ex).copy())
        values = rng.standard_normal(k).astype(np.float32)
        pk = rng.uniform(0.0, 1.0, k)
        pk = (pk / pk.sum()).astype(np.float32)
        z = np.zeros(n, np.float32)
        outs.append(ref.random_xy(5, state, values, ki, pk, ki, z, zi, np.array([1.0], np.float32)).copy())
        z = np.zeros(n, np.float32)
        outs.append(ref.random(0, state, z, zi, np.array([0.0, 1.0], np.float32)).copy())
        outs.append(np.array([ref.rng_position(state), ref.rng_generation(state)], np.float32))
        ref.destroy_random(state)
        return np.concatenate(outs)
    raise ValueError(fam)
