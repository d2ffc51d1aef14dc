"""An object with the oracle's calling interface (oracle/reference.py) whose methods run on the GPU
through the NativeOps mirror, so that one case runner (tests/golden_cases.py) serves the reference,
the port and the CUDA path. float32 only, like the golden records."""
import numpy as np
import torch


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


class GpuOps:
    def __init__(self, ops):
        self.ops = ops

    def _out(self, z, dz):
        z[...] = dz.cpu().numpy().reshape(z.shape)
        return z

    def transform(self, op, x, x_info, z, z_info, extra=None):
        dz = _dev(z)
        self.ops.execTransformFloat(None, op, _dev(x), x_info, dz, z_info, None if extra is None else _dev(extra))
        return self._out(z, dz)

    def pairwise(self, op, x, x_info, y, y_info, z, z_info, extra=None):
        dz = _dev(z)
        self.ops.execPairwiseTransformFloat(None, op, _dev(x), x_info, _dev(y), y_info, dz, z_info,
                                            None if extra is None else _dev(extra))
        return self._out(z, dz)

    def scalar(self, op, x, x_info, z, z_info, scalar, extra=None):
        dz = _dev(z)
        self.ops.execScalarFloat(None, op, _dev(x), x_info, dz, z_info, scalar, None if extra is None else _dev(extra))
        return self._out(z, dz)

    def broadcast(self, op, x, x_info, y, y_info, z, z_info, dims):
        dz = _dev(z)
        self.ops.execBroadcastFloat(None, op, _dev(x), x_info, _dev(y), y_info, dz, z_info, dims, len(dims))
        return self._out(z, dz)

    def reduce(self, op, x, x_info, z, z_info, dims, extra=None):
        dz = _dev(z)
        self.ops.execReduceFloat(None, op, _dev(x), x_info, None if extra is None else _dev(extra), dz, z_info, dims, len(dims))
        return self._out(z, dz)

    def index_reduce(self, op, x, x_info, z, z_info, dims, extra=None):
        dz = _dev(z)
        self.ops.execIndexReduceFloat(None, op, _dev(x), x_info, None if extra is None else _dev(extra), dz, z_info, dims,
                                      len(dims))
        return self._out(z, dz)

    def summary_stats(self, op, x, x_info, z, z_info, dims, bias):
        dz = _dev(z)
        self.ops.execSummaryStatsFloat(None, op, _dev(x), x_info, None, dz, z_info, dims, len(dims), bias)
        return self._out(z, dz)

    def reduce3(self, op, x, x_info, y, y_info, z, z_info, dims, extra=None):
        dz = _dev(z)
        self.ops.execReduce3Float(None, op, _dev(x), x_info, None if extra is None else _dev(extra), _dev(y), y_info, dz,
                                  z_info, dims, len(dims))
        return self._out(z, dz)

    def reduce3_all(self, op, x, x_info, y, y_info, z, z_info, dims, extra=None):
        dz = _dev(z)
        self.ops.execReduce3AllFloat(None, op, _dev(x), x_info, None, _dev(y), y_info, dz, z_info, dims, len(dims),
                                     None, None, None, None)
        return self._out(z, dz)

    # ---- random ----------------------------------------------------------------------------------
    def init_random(self, seed, size):
        return self.ops.initRandom(None, seed, size, None), None

    def destroy_random(self, state):
        self.ops.destroyRandom(state)

    def rng_position(self, state):
        return self.ops.rngState(state)[1]

    def rng_generation(self, state):
        return self.ops.rngState(state)[2]

    def random(self, op, state, z, z_info, extra):
        dz = _dev(z)
        self.ops.execRandomFloat(None, op, state, dz, z_info, _dev(extra))
        return self._out(z, dz)

    def random_x(self, op, state, x, x_info, z, z_info, extra):
        dz = _dev(z)
        self.ops.execRandomFloat(None, op, state, _dev(x), x_info, dz, z_info, _dev(extra))
        return self._out(z, dz)

    def random_xy(self, op, state, x, x_info, y, y_info, z, z_info, extra):
        dz = _dev(z)
        dx = dz if x is z else _dev(x)
        dy = dz if y is z else _dev(y)
        self.ops.execRandomFloat(None, op, state, dx, x_info, dy, y_info, dz, z_info, _dev(extra))
        return self._out(z, dz)
