"""The allocation-free whole-array reduction (nd4jb200_exec_reduce_scalar_noalloc) against the
regular entry point, through the C ABI.

Who needs it: callers that may not allocate device memory - code living inside an arena that
already owns the whole device, latency-critical loops where an allocation could stall every
stream, sandboxed processes. The regular entry point obtains a workspace with cudaMalloc on first
use; this one keeps its partial states in a fixed array inside the library image. The file name
sorts last on purpose: a run that stops at the first failure has then exercised everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S

pytestmark = pytest.mark.gpu


def _bind(ops):
    fn = ops.lib.nd4jb200_exec_reduce_scalar_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_longlong),
                   ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _info(a):
    arr = np.ascontiguousarray(a, dtype=np.int64)
    return arr, arr.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong))


@pytest.mark.parametrize("n", [1, 1000, 65536, 65537, (1 << 22) + 3, 1 << 27])
def test_two_calls_in_a_row_match_the_regular_entry_point(ops, n):
    fn = _bind(ops)
    g = torch.Generator(device="cuda")
    g.manual_seed(n)
    x = torch.empty(n, device="cuda").uniform_(-1, 1, generator=g)
    keep, info = _info(S.shape_info([1, n]))
    z = torch.full((1,), float("nan"), device="cuda")
    for op in (1, 3):                         # Sum, then Max: the second call reuses the same scratch
        for _ in range(2):                    # and each op runs twice back to back
            z.fill_(float("nan"))
            rc = fn(None, 0, op, ctypes.c_void_p(x.data_ptr()), info, None, ctypes.c_void_p(z.data_ptr()))
            assert rc == 0, ops.lastError()
            torch.cuda.synchronize()
            want = ops.execReduceScalarFloat(None, op, x, keep, None)
            got = float(z.item())
            if op == 3:
                assert got == want
            else:
                # both split the array into segments of different sizes: same tolerance as the
                # reduction parity tests, relative to the sum of magnitudes
                assert abs(got - want) <= 1e-5 * float(x.abs().double().sum())


def test_other_types_and_strided_input(ops):
    fn = _bind(ops)
    x = torch.arange(1, 200001, device="cuda", dtype=torch.float64)
    keep, info = _info(S.shape_info([1, 200000]))
    z = torch.zeros(1, device="cuda", dtype=torch.float64)
    assert fn(None, 1, 1, ctypes.c_void_p(x.data_ptr()), info, None, ctypes.c_void_p(z.data_ptr())) == 0
    torch.cuda.synchronize()
    assert float(z.item()) == 200000 * 200001 / 2
    keep2, view = _info(S.shape_info([100000], "c", [2]))   # every second element
    assert fn(None, 1, 1, ctypes.c_void_p(x.data_ptr()), view, None, ctypes.c_void_p(z.data_ptr())) == 0
    torch.cuda.synchronize()
    assert float(z.item()) == 100000 ** 2


@pytest.mark.parametrize("n", [65537, (1 << 22) + 3])
def test_float_sum_against_the_reference_and_an_fp64_truth(ops, real_ref, n):
    """Independent of the entry point it shares kernels with: the value is held against a float64 sum of the
    same data and against the reference's own whole-array loop, with the bound the reduction tests use."""
    fn = _bind(ops)
    x = np.random.default_rng(n).uniform(-1, 1, n).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    keep, info = _info(S.shape_info([1, n]))
    z = torch.zeros(1, device="cuda")
    truth, mag = float(x.astype(np.float64).sum()), float(np.abs(x).astype(np.float64).sum())
    want = float(real_ref.reduce_scalar(1, x, keep))
    for _ in range(2):
        assert fn(None, 0, 1, ctypes.c_void_p(dx.data_ptr()), info, None, ctypes.c_void_p(z.data_ptr())) == 0
        torch.cuda.synchronize()
        assert abs(float(z.item()) - truth) <= max(1e-5 * mag, abs(want - truth) * 1.0000001)


def test_half_precision_sum_and_max(ops):
    fn = _bind(ops)
    n = 300001
    x = (np.random.default_rng(3).uniform(-1, 1, n) / 64).astype(np.float16)     # the sum stays far below 65504
    dx = torch.from_numpy(x).cuda()
    keep, info = _info(S.shape_info([1, n]))
    z = torch.zeros(1, device="cuda", dtype=torch.float16)
    truth, mag = float(x.astype(np.float64).sum()), float(np.abs(x).astype(np.float64).sum())
    for _ in range(2):
        assert fn(None, 2, 1, ctypes.c_void_p(dx.data_ptr()), info, None, ctypes.c_void_p(z.data_ptr())) == 0
        torch.cuda.synchronize()
        got = float(z.item())
        # accumulated in float, rounded to half once: half an ulp of the result plus the float sum's own error
        assert abs(got - truth) <= 1e-2 * mag and abs(got - truth) <= 2 ** -10 * abs(truth) + 1e-5 * mag
    assert fn(None, 2, 3, ctypes.c_void_p(dx.data_ptr()), info, None, ctypes.c_void_p(z.data_ptr())) == 0
    torch.cuda.synchronize()
    assert float(z.item()) == float(x.max())


def test_inputs_beyond_the_built_in_scratch_are_refused(ops):
    fn = _bind(ops)
    x = torch.zeros(16, device="cuda")
    z = torch.zeros(1, device="cuda")
    keep, info = _info(S.shape_info([1, (1 << 27) + 1]))     # only the descriptor is large
    rc = fn(None, 0, 1, ctypes.c_void_p(x.data_ptr()), info, None, ctypes.c_void_p(z.data_ptr()))
    assert rc == 5
    assert "built-in scratch" in ops.lastError()
