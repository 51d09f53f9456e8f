"""Column sums whose second pass runs inside the first kernel (the block that finishes a column
group last adds the group's partial sums) against the same sums with the second pass as a
launch of its own: same bits, call after call, on both library streams."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _sum0(H, lib, check, a, fold):
    check(lib.b200_set_tuning(11, fold))
    out = H.create_from_numpy(np.full((1, a.shape[1]), np.nan, np.float32))
    H.sum_t(a, 0, out)
    return H.get_numpy_copy(out)


@pytest.mark.parametrize('rows,cols', [(64, 4), (129, 32), (1000, 128), (4096, 4096), (70000, 12), (5000, 1027),
                                       (8192, 516), (300000, 4)])
def test_folded_second_pass_gives_the_bits_of_the_two_launch_form(rows, cols):
    from brainstorm_b200 import B200Handler
    from brainstorm_b200._lib import lib, check
    H = B200Handler()
    rs = np.random.RandomState(rows + cols)
    x = rs.randn(rows, cols).astype(np.float32)
    a = H.create_from_numpy(x)
    try:
        want = _sum0(H, lib, check, a, 0)
        for _ in range(3):                           # the counters must be back at zero after every call
            assert np.array_equal(_sum0(H, lib, check, a, 1), want)
        check(lib.b200_use_stream(1))                # the side stream has counters of its own
        try:
            assert np.array_equal(_sum0(H, lib, check, a, 1), want)
        finally:
            check(lib.b200_use_stream(0))
        np.testing.assert_allclose(want[0], x.astype(np.float64).sum(0), rtol=1e-5, atol=1e-5 * np.abs(x).sum(0).max())
    finally:
        check(lib.b200_set_tuning(11, 1))


def test_folded_second_pass_in_the_fused_batchnorm_sums():
    from brainstorm_b200 import B200Handler, B200Array
    from brainstorm_b200._lib import lib, check
    H = B200Handler()
    rs = np.random.RandomState(3)
    rows, cols = 6000, 256
    d = H.create_from_numpy(rs.randn(rows, cols).astype(np.float32))
    xh = H.create_from_numpy(rs.randn(rows, cols).astype(np.float32))
    got = {}
    try:
        for fold in (0, 1, 1):
            check(lib.b200_set_tuning(11, fold))
            sums = H.create_from_numpy(np.full((2 * cols,), np.nan, np.float32))
            sp, sn = H._scratch_for(lib.b200_bn_scratch_floats(rows, cols))
            check(lib.b200_bn_backward_sums(d.ptr, xh.ptr, sums.ptr, rows, cols, sp, sn))
            got.setdefault(fold, []).append(H.get_numpy_copy(sums))
    finally:
        check(lib.b200_set_tuning(11, 1))
    assert np.array_equal(got[0][0], got[1][0]) and np.array_equal(got[0][0], got[1][1])
