"""The in-library multi-GPU layer (nd4jb200_comm_*, nd4jb200_exec_reduce_scalar_sharded, *_across) on one GPU:
a communicator of world size 1 runs the same local kernels, state exchange buffers and fixed-order combine
as a multi-rank job, without NCCL. What several ranks add is the all-gather between the two steps; that path is
exercised by `bench.py --gpus N` (its families table reports the combined value, which must not depend on N
for a fixed shard grid) and its host-side ordering logic by tests/test_sharding_gloo.py."""
import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def comm(ops):
    ops.commInit(None, 0, 1)
    yield ops
    ops.commDestroy()


@pytest.mark.parametrize("n", [1 << 20, 1 << 24, (1 << 24) + (1 << 10)])
def test_sum_depends_on_the_shard_grid_only(comm, real_ref, n):
    ops = comm
    x = np.random.default_rng(n % 1000).uniform(-1, 1, n).astype(np.float32)
    dx = dev(x)
    truth, mag = float(x.astype(np.float64).sum()), float(np.abs(x).astype(np.float64).sum())
    want = float(real_ref.reduce_scalar(1, x, S.shape_info([1, n])))
    for shards in (1, 2, 8):
        got = ops.execReduceScalarSharded(0, None, 1, dx, n, None, shards, n)
        assert abs(got - truth) <= max(1e-5 * mag, abs(want - truth) * 1.0000001)
        # the value is the in-order float sum of the shards' own sums, each of which is what a rank holding only
        # that shard computes: 8 shards on one rank == 8 ranks with one shard each
        per = n // shards
        parts = [ops.execReduceScalarSharded(0, None, 1, dx[k * per:(k + 1) * per], per, None, 1, per) for k in range(shards)]
        acc = np.float32(parts[0])
        for p in parts[1:]:
            acc = np.float32(acc + np.float32(p))
        assert np.float32(got) == acc, (shards, got, acc)
    # and a second run gives the same bits
    assert ops.execReduceScalarSharded(0, None, 1, dx, n, None, 8, n) == ops.execReduceScalarSharded(0, None, 1, dx, n, None, 8, n)


@pytest.mark.parametrize("dt,code", [(np.float32, 0), (np.float64, 1), (np.float16, 2)])
@pytest.mark.parametrize("op", [0, 1, 3, 4, 6, 19, 25])
def test_other_ops_and_types_against_the_unsharded_call(comm, dt, code, op):
    ops = comm
    n = 1 << (14 if dt == np.float16 else 18)          # half: sums of squares must stay below 65504
    x = np.random.default_rng(op).uniform(-1, 1, n).astype(dt)
    dx = dev(x)
    name = {0: "Float", 1: "Double", 2: "Half"}[code]
    whole = getattr(ops, "execReduceScalar" + name)(None, op, dx, S.shape_info([1, n]), None)
    got = ops.execReduceScalarSharded(code, None, op, dx, n, None, 4, n)
    tol = {0: 1e-5, 1: 1e-12, 2: 1e-2}[code]
    scale = float(np.abs(x).astype(np.float64).sum()) if op in (0, 1) else max(abs(whole), 1e-30)
    if op == 0:
        scale /= n
    assert abs(got - whole) <= tol * scale, (op, got, whole)


def test_result_on_the_device_without_a_host_round_trip(comm):
    ops = comm
    n = 1 << 22
    x = torch.rand(n, device="cuda")
    z = torch.zeros(1, device="cuda")
    assert ops.execReduceScalarSharded(0, None, 1, x, n, None, 8, n, z=z, fetch=False) is None
    want = ops.execReduceScalarSharded(0, None, 1, x, n, None, 8, n)
    torch.cuda.synchronize()
    assert float(z.item()) == np.float32(want)
    with pytest.raises(RuntimeError):
        ops.execReduceScalarSharded(0, None, 1, x, n, None, 3, n)          # 3 does not divide the length
    with pytest.raises(RuntimeError):
        ops.execReduceScalarSharded(0, None, 1, x, n, None, 65, n)


def test_average_and_accumulate_across_one_rank(comm):
    ops = comm
    x = torch.randn(100003, device="cuda")
    z = torch.zeros_like(x)
    ops.accumulateAcross(0, None, x, z, x.numel())
    assert torch.equal(z, x)
    z.zero_()
    ops.averageAcross(0, None, x, z, x.numel(), False)
    assert torch.equal(z, x)                                               # x / 1
