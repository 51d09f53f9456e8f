"""The op suite at the benchmark's full size, (65536, 4096) fp32 = 1 GiB per
operand, where the CPU oracle would take minutes: size-independent properties
checked on the device, plus spot rows against the oracle."""
import numpy as np
import pytest

import parity
from oracle.numpy_oracle import OracleHandler

pytestmark = pytest.mark.gpu
ROWS, COLS = 65536, 4096


@pytest.fixture(scope='module')
def world():
    from brainstorm_b200 import B200Handler
    H = B200Handler(seed=2, rng_mode='device')
    a = H.allocate((ROWS, COLS))
    H.fill_gaussian(0.0, 2.0, a)                   # device-generated operand
    b = H.allocate((ROWS, COLS))
    H.fill_gaussian(0.5, 1.0, b)
    out = H.allocate((ROWS, COLS))
    rs = np.random.RandomState(3)
    rows = np.sort(rs.choice(ROWS, 6, replace=False))
    return H, a, b, out, rows


def _rows(H, arr, rows):
    return np.stack([H.get_numpy_copy(arr[int(r)]) for r in rows])


def test_elementwise_round_trips_and_spot_rows(world):
    H, a, b, out, rows = world
    O = OracleHandler(np.float32)
    ha, hb = _rows(H, a, rows), _rows(H, b, rows)
    for op in ('add_tt', 'subtract_tt', 'mult_tt', 'divide_tt'):
        getattr(H, op)(a, b, out)
        want = np.zeros_like(ha)
        getattr(O, op)(ha, hb, want)
        parity.assert_elementwise_close(_rows(H, out, rows), want, op)
    for op in ('sigmoid', 'tanh', 'rel', 'el', 'abs_t', 'sign_t'):
        getattr(H, op)(a, out)
        want = np.zeros_like(ha)
        getattr(O, op)(ha, want)
        parity.assert_elementwise_close(_rows(H, out, rows), want, op)
    # (a + b) - b == a up to one rounding of the sum
    H.add_tt(a, b, out)
    H.subtract_tt(out, b, out)
    H.subtract_tt(out, a, out)
    H.abs_t(out, out)
    worst = H.zeros(())
    H.sum_t(out, None, worst)
    mean_err = float(H.get_numpy_copy(worst)) / (ROWS * COLS)
    assert mean_err < 2e-7, mean_err


def test_sums_agree_with_each_other_and_with_float64(world):
    H, a, b, out, rows = world
    s0, s1, sall = H.zeros((1, COLS)), H.zeros((ROWS, 1)), H.zeros(())
    H.sum_t(a, 0, s0)
    H.sum_t(a, 1, s1)
    H.sum_t(a, None, sall)
    h0, h1, hall = H.get_numpy_copy(s0), H.get_numpy_copy(s1), float(H.get_numpy_copy(sall))
    H.abs_t(a, out)
    sabs = H.zeros(())
    H.sum_t(out, None, sabs)
    scale = float(H.get_numpy_copy(sabs))
    assert abs(h0.astype(np.float64).sum() - hall) <= 1e-5 * scale
    assert abs(h1.astype(np.float64).sum() - hall) <= 1e-5 * scale
    ha = _rows(H, a, rows)
    parity.assert_reduction_close(h1[rows, 0], ha.astype(np.float64).sum(1), np.abs(ha).astype(np.float64).sum(1), 'sum_t', 'axis 1 rows')
    # twice the same input gives the same bits (deterministic trees)
    again = H.zeros((1, COLS))
    H.sum_t(a, 0, again)
    assert np.array_equal(H.get_numpy_copy(again), h0)


def test_softmax_rows_are_distributions(world):
    H, a, b, out, rows = world
    H.softmax_m(a, out)
    s1 = H.zeros((ROWS, 1))
    H.sum_t(out, 1, s1)
    sums = H.get_numpy_copy(s1)
    assert np.abs(sums - 1.0).max() < 1e-5
    ha = _rows(H, a, rows)
    e = np.exp(ha.astype(np.float64) - ha.max(1, keepdims=True))
    parity.assert_reduction_close(_rows(H, out, rows), e / e.sum(1, keepdims=True), 0.0, 'softmax_m')


def test_binarize_and_index_invert_each_other(world):
    H, a, b, out, rows = world
    labels = np.random.RandomState(5).randint(0, COLS, (ROWS, 1)).astype(np.float32)
    dl = H.create_from_numpy(labels)
    H.binarize_v(dl, out)
    s1 = H.zeros((ROWS, 1))
    H.sum_t(out, 1, s1)
    assert np.array_equal(H.get_numpy_copy(s1), np.ones((ROWS, 1), np.float32))   # exactly one 1 per row
    picked = H.zeros((ROWS, 1))
    H.index_m_by_v(out, dl, picked)
    assert np.array_equal(H.get_numpy_copy(picked), np.ones((ROWS, 1), np.float32))  # and it sits at the label
    H.index_m_by_v(a, dl, picked)
    got = H.get_numpy_copy(picked)
    ha = _rows(H, a, rows)
    assert np.array_equal(got[rows, 0], ha[np.arange(len(rows)), labels[rows, 0].astype(int)])


def test_broadcast_linearity(world):
    H, a, b, out, rows = world
    rs = np.random.RandomState(7)
    row = H.create_from_numpy(rs.uniform(-4, 4, (1, COLS)).astype(np.float32))
    col = H.create_from_numpy(rs.uniform(-4, 4, (ROWS, 1)).astype(np.float32))
    ha = _rows(H, a, rows)
    hrow, hcol = H.get_numpy_copy(row), H.get_numpy_copy(col)
    H.add_mv(a, row, out)
    parity.assert_elementwise_close(_rows(H, out, rows), ha + hrow, 'add_mv')
    H.mult_mv(a, col, out)
    parity.assert_elementwise_close(_rows(H, out, rows), ha * hcol[rows], 'mult_mv')
    H.mult_st(0.37, a, out)
    parity.assert_elementwise_close(_rows(H, out, rows), np.float32(0.37) * ha, 'mult_st')


def test_more_than_2_to_31_elements():
    """64-bit indexing: a flat array of 2^31 + 5 elements (8 GiB) through the
    elementwise, scalar and reduction kernels."""
    from brainstorm_b200 import B200Handler
    H = B200Handler(seed=2)
    n = (1 << 31) + 5
    a, out = H.allocate((n,)), H.allocate((n,))
    H.fill(a, 0.5)
    H.mult_st(3.0, a, out)              # 1.5 everywhere
    H.add_tt(out, a, out)               # 2.0 everywhere, in place
    tail = H.get_numpy_copy(out[n - 7:])
    assert tail.tolist() == [2.0] * 7
    head = H.get_numpy_copy(out[:3])
    assert head.tolist() == [2.0] * 3
    total = H.zeros(())
    H.sum_t(out, None, total)
    # every partial is exactly representable; the total rounds to the nearest float32 (ulp 512 at 2^32)
    assert float(H.get_numpy_copy(total)) == float(np.float32(2.0 * n))
    m = out[:(1 << 31)].reshape((1 << 20, 1 << 11))
    s1 = H.zeros((1 << 20, 1))
    H.sum_t(m, 1, s1)
    assert np.array_equal(H.get_numpy_copy(s1), np.full((1 << 20, 1), 4096.0, np.float32))
    s0 = H.zeros((1, 1 << 11))
    H.sum_t(m, 0, s0)
    assert np.array_equal(H.get_numpy_copy(s0), np.full((1, 1 << 11), float(1 << 21), np.float32))
