"""Accuracy against exact arithmetic: for every op of the suite the GPU result and
the float32 CPU result are both compared with the same op evaluated in float64.
The parity tolerances are stated relative to the float32 CPU backend; this test
shows that where the two differ, the GPU is not the less accurate one (sums and
GEMMs: tree / chunked accumulation against numpy's sequential float32 sums)."""
import numpy as np
import pytest

from oracle.numpy_oracle import OracleHandler, op_suite_inputs

pytestmark = pytest.mark.gpu
ROWS, COLS = 1024, 1024


def _ops(d, O):
    a, b, dy, div, row, col = d['a'], d['b'], d['dy'], d['div'], d['row'], d['col']
    z = np.zeros_like(a)
    y = np.zeros_like(a)
    O.tanh(a, y)
    yield 'add_tt', (a, b, z)
    yield 'divide_tt', (a, div, z)
    yield 'mult_mv', (a, row, z)
    yield 'sigmoid', (a, z)
    yield 'tanh', (a, z)
    yield 'el', (a, z)
    yield 'sigmoid_deriv', (a, y, dy, z)
    yield 'tanh_deriv', (a, y, dy, z)
    yield 'sqrt_t', (np.abs(a), z)
    yield 'softmax_m', (a, z)
    yield 'sum_t', (a, 0, np.zeros((1, COLS), a.dtype))
    yield 'sum_t', (a, 1, np.zeros((ROWS, 1), a.dtype))
    yield 'sum_t', (a, None, np.zeros((), a.dtype))
    yield 'dot_mm', (a, b, z)


def test_gpu_is_at_least_as_accurate_as_float32_cpu():
    from brainstorm_b200 import B200Handler
    H = B200Handler(seed=1)
    d32 = op_suite_inputs(ROWS, COLS, 0)
    d64 = {k: v.astype(np.float64) for k, v in d32.items()}
    O32, O64 = OracleHandler(np.float32), OracleHandler(np.float64)
    report = []
    for (op, a32), (_, a64) in zip(_ops(d32, O32), _ops(d64, O64)):
        a32 = [x.copy() if isinstance(x, np.ndarray) else x for x in a32]
        a64 = [x.copy() if isinstance(x, np.ndarray) else x for x in a64]
        dev = [H.create_from_numpy(x) if isinstance(x, np.ndarray) else x for x in a32]
        getattr(O32, op)(*a32)
        getattr(O64, op)(*a64)
        getattr(H, op)(*dev)
        exact, cpu, gpu = a64[-1], a32[-1].astype(np.float64), H.get_numpy_copy(dev[-1]).astype(np.float64)
        scale = np.abs(exact).max()
        e_cpu, e_gpu = np.abs(cpu - exact).max() / scale, np.abs(gpu - exact).max() / scale
        report.append((op, e_cpu, e_gpu))
        # elementwise: within a few ulp of each other; reductions / GEMM: the GPU may not be worse
        # than 4x the float32 CPU error (it is usually better)
        assert e_gpu <= max(4 * e_cpu, 3e-7), (op, e_cpu, e_gpu)
    for op, e_cpu, e_gpu in report:
        print('%-14s max err / max|exact|: float32 CPU %.2e   B200 %.2e' % (op, e_cpu, e_gpu))
