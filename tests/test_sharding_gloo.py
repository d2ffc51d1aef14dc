"""Multi-process checks of the sharding layer on CPU: world_size 2 and 3 over gloo. The local
work of a rank is done with numpy here; on GPU ranks the same functions wrap the C ABI."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from libnd4j_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


NP_LOCAL = {1: lambda a: a.astype(np.float64).sum(), 3: lambda a: a.max(), 4: lambda a: a.min(),
            5: lambda a: np.abs(a).astype(np.float64).sum(), 11: lambda a: np.abs(a).astype(np.float64).sum(),
            25: lambda a: (a.astype(np.float64) ** 2).sum(), 7: lambda a: np.abs(a).max(), 13: lambda a: np.abs(a).max(),
            14: lambda a: np.abs(a).min(), 8: lambda a: a.astype(np.float64).prod(),
            22: lambda a: float((a != 0).sum()), 26: lambda a: float((a == 0).sum())}
NP_FULL = {1: lambda a: a.astype(np.float64).sum(), 0: lambda a: a.astype(np.float64).mean(), 3: lambda a: a.max(),
           4: lambda a: a.min(), 6: lambda a: np.sqrt((a.astype(np.float64) ** 2).sum()), 7: lambda a: np.abs(a).max(),
           22: lambda a: float((a != 0).sum()), 15: lambda a: np.abs(a).astype(np.float64).mean()}


def _worker(rank, world, port, n, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = np.random.default_rng(8).uniform(-1, 1, n).astype(np.float32)
    x[::97] = 0.0
    first, count = sharding.shard_range(n, world, rank)
    shard = x[first:first + count]
    out = {}
    for op, full in NP_FULL.items():
        got = sharding.sharded_reduce_scalar(dist, op, lambda lop: NP_LOCAL[lop](shard), n)
        out[op] = (got, float(full(x)))
    lv = (np.arange(16) / 8.0 - 1.0).astype(np.float32)
    t = lv[np.random.default_rng(4).integers(0, 16, n)]
    ts = t[first:first + count]
    out["imax"] = (sharding.sharded_index_reduce_scalar(dist, 0, (int(ts.argmax()), float(ts.max())), first), int(t.argmax()))
    out["imin"] = (sharding.sharded_index_reduce_scalar(dist, 1, (int(ts.argmin()), float(ts.min())), first), int(t.argmin()))
    if rank == 0:
        results.update(out)
    dist.barrier()
    dist.destroy_process_group()


def _grid_worker(rank, world, port, n, grid, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = np.random.default_rng(8).uniform(-1, 1, n).astype(np.float32)
    per_shard = n // grid
    k = grid // world
    # what a rank's local kernels deliver: one float32 state per shard it holds, each a function of that shard alone
    mine = [np.float32(x[(rank * k + j) * per_shard:(rank * k + j + 1) * per_shard].sum(dtype=np.float32)) for j in range(k)]
    got = sharding.fold_states_in_shard_order(dist, mine, lambda a, b: np.float32(a + b))
    results[rank] = float(got)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_fixed_shard_grid_gives_the_same_bits_in_every_world(world):
    """The combine order of the sharded whole-array reduction: states meet in global shard order whatever the
    number of ranks, so a grid of 8 shards sums to the same float32 bits on 1, 2 or 4 ranks."""
    n, grid = 8 * 12500, 8
    x = np.random.default_rng(8).uniform(-1, 1, n).astype(np.float32)
    shards = [np.float32(x[j * (n // grid):(j + 1) * (n // grid)].sum(dtype=np.float32)) for j in range(grid)]
    want = sharding.fold_states_in_shard_order(None, shards, lambda a, b: np.float32(a + b))
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_grid_worker, args=(world, _free_port(), n, grid, results), nprocs=world, join=True)
        results = dict(results)
    assert len(results) == world
    for rank, got in results.items():
        assert np.float32(got) == np.float32(want), (rank, got, want)


def _lonely(rank, port, flag):
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=3))
    if rank == 0:
        try:
            sharding.gather_partials(dist, 1.0)
            flag["result"] = "no error"
        except Exception as e:   # gloo reports the missing peer / the timeout as a RuntimeError
            flag["result"] = "error: " + type(e).__name__
    # rank 1 leaves without joining the collective


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_whole_array_reductions_match_single_process(world):
    n = 100003
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), n, results), nprocs=world, join=True)
        results = dict(results)
    for key, (got, want) in results.items():
        if isinstance(key, str):
            assert got == want, key          # ties resolve to the lowest global index
        else:
            assert abs(got - want) <= 1e-9 * max(1.0, abs(want)), key


def test_shard_ranges_cover_everything_with_even_boundaries():
    for n in (0, 1, 7, 1 << 20, (1 << 30) + 6):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == n
            for (f0, c0), (f1, _) in zip(spans[:-1], spans[1:]):
                assert f0 + c0 == f1 and f1 % 2 == 0
    with pytest.raises(ValueError):
        sharding.shard_range(10, 2, 2)


def test_a_rank_that_never_joins_is_detected_by_the_timeout():
    """Failure detection on the host: one rank of a two-rank job never calls the collective; the
    other rank's gather ends with an error after the process-group timeout instead of hanging."""
    with mp.Manager() as manager:
        flag = manager.dict()
        try:
            mp.spawn(_lonely, args=(_free_port(), flag), nprocs=2, join=True)
        except Exception:
            pass
        assert str(flag.get("result", "missing")).startswith("error"), dict(flag)
