"""Host-side sharding of the legacy op families across the GPUs of one box (one process per GPU,
torch.distributed for the plumbing).

Nothing in the reference shards anything: its only multi-device facility averages whole arrays
through peer pointers (include/loops/special_kernels.h:711-821). The rules here follow from the
families themselves:

  * along-dimension reductions, elementwise ops and broadcast: TADs / elements are independent,
    so every rank works on a contiguous block of TADs or elements and nothing is exchanged;
  * random ops: element e depends only on (table, state, e), so rank g produces the global index
    range [first, first + count) with nd4jb200_exec_random_range and the state owner rewinds once
    by the full length; range boundaries are even so that Gaussian pairs never straddle ranks;
  * whole-array reductions: every rank reduces its contiguous shard to a partial, the partials
    are gathered (a few bytes per rank) and combined in rank order, which keeps the result
    independent of arrival order; plain sums may use an all-reduce instead.
"""
import math

import numpy as np

# reduce opNum -> (local opNum, combine rule) for whole-array reductions over contiguous shards
# (numbers: REDUCE_OPS, include/loops/legacy_ops.h:195-221)
_COMBINE = {
    1: (1, "sum"), 0: (1, "mean"), 3: (3, "max"), 4: (4, "min"), 5: (5, "sum"), 11: (11, "sum"), 15: (11, "mean"),
    6: (25, "sqrt_sum"), 23: (25, "sqrt_sum"), 25: (25, "sum"), 7: (7, "max"), 13: (13, "max"), 14: (14, "min"),
    8: (8, "prod"), 22: (22, "sum"), 26: (26, "sum"), 20: (1, "any"), 21: (8, "all"),
}


def shard_range(length, world, rank, quantum=2):
    """Contiguous [first, first + count) of `length` items for `rank`; every boundary is a
    multiple of `quantum` (2 keeps Box-Muller pairs together), the remainder goes to the last rank."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("rank %d outside a world of %d" % (rank, world))
    per = (length // world) // quantum * quantum
    first = rank * per
    count = per if rank < world - 1 else length - first
    return first, count


def shard_tads(num_tads, world, rank):
    """Block of TAD indices [first, first + count) for `rank` (no alignment requirement)."""
    return shard_range(num_tads, world, rank, quantum=1)


def local_op(op_num):
    """The opNum each rank runs on its shard for a whole-array reduction `op_num`."""
    if op_num not in _COMBINE:
        raise NotImplementedError("whole-array reduce op %d has no sharded form" % op_num)
    return _COMBINE[op_num][0]


def combine_partials(op_num, partials, total_length):
    """Combines per-rank partials (in rank order, float64) into the result of the whole-array op."""
    rule = _COMBINE[op_num][1]
    vals = [float(p) for p in partials]
    if rule == "sum":
        return math.fsum(vals)
    if rule == "mean":
        return math.fsum(vals) / total_length
    if rule == "max":
        return max(vals)
    if rule == "min":
        return min(vals)
    if rule == "prod":
        out = 1.0
        for v in vals:
            out *= v
        return out
    if rule == "sqrt_sum":
        return math.sqrt(math.fsum(vals))
    if rule == "any":
        return 1.0 if math.fsum(vals) > 0 else 0.0
    if rule == "all":
        out = 1.0
        for v in vals:
            out *= v
        return 1.0 if out > 0 else 0.0
    raise AssertionError(rule)


def gather_partials(dist, value, device=None):
    """All-gathers one float64 per rank (rank order). `dist` is torch.distributed (initialised)."""
    import torch
    world = dist.get_world_size()
    mine = torch.tensor([float(value)], dtype=torch.float64, device=device)
    out = [torch.zeros(1, dtype=torch.float64, device=device) for _ in range(world)]
    dist.all_gather(out, mine)
    return [float(t.item()) for t in out]


def fold_states_in_shard_order(dist, local_states, merge, device=None):
    """The combine step of nd4jb200_exec_reduce_scalar_sharded, stated on the host: every rank holds the
    accumulator states of its consecutive shards (a float32 vector, one entry per shard); the states of all ranks
    are gathered rank-major, which is global shard order, and folded from the left with `merge`. The value then
    depends on the shard grid only: 8 shards give the same bits in a world of 1, 2, 4 or 8."""
    import torch
    mine = torch.tensor(np.asarray(local_states, dtype=np.float32), device=device)
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        states = [mine]
    else:
        states = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
        dist.all_gather(states, mine)
    flat = np.concatenate([t.cpu().numpy() for t in states]).astype(np.float32)
    acc = flat[0]
    for v in flat[1:]:
        acc = merge(acc, v)
    return acc


def sharded_reduce_scalar(dist, op_num, local_reduce, total_length, device=None):
    """Whole-array reduction over shards. `local_reduce(local_op_num)` returns this rank's partial
    (on a GPU rank it calls execReduceScalar on the shard). Every rank returns the same value."""
    part = local_reduce(local_op(op_num))
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return combine_partials(op_num, [part], total_length)
    return combine_partials(op_num, gather_partials(dist, part, device), total_length)


def sharded_index_reduce_scalar(dist, op_num, local_index_value, shard_first, device=None):
    """Whole-array IndexMax (0) / IndexMin (1): each rank passes (local index, local value); the
    winner is the extreme value with the lowest GLOBAL index, so ties resolve as in one process."""
    import torch
    idx, val = local_index_value
    mine = torch.tensor([float(val), float(shard_first + idx)], dtype=torch.float64, device=device)
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return int(shard_first + idx)
    out = [torch.zeros(2, dtype=torch.float64, device=device) for _ in range(dist.get_world_size())]
    dist.all_gather(out, mine)
    pairs = [(float(t[0]), int(t[1])) for t in out]
    if op_num == 0:
        best = max(pairs, key=lambda p: (p[0], -p[1]))
    elif op_num == 1:
        best = min(pairs, key=lambda p: (p[0], p[1]))
    else:
        raise NotImplementedError("sharded index reduce supports IndexMax (0) and IndexMin (1)")
    return best[1]


def sharded_random(ops, dtype_code, op_num, arity, state, x, y, z, extra, length, world, rank, stream=None):
    """Fills this rank's slice of a logical `length`-element random call. x, y, z are this rank's
    dense shard buffers. The caller that owns the state rewinds it once by `length` afterwards."""
    first, count = shard_range(length, world, rank)
    ops.execRandomRange(dtype_code, [None, stream] if stream else None, op_num, arity, state, x, y, z, extra, first,
                        count, length)
    return first, count
