"""sum_t without allocation (b200_sum_t_static): for hosts that cannot allocate
device memory while they run, e.g. because their own pool already owns the GPU or
because they must never enter the CUDA allocator mid-run.  The entry point keeps
its partial sums in an array built into the library; it must give exactly what
b200_sum_t gives with caller-provided scratch, also when called twice in a row
(the array still holds the previous call's partials)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _abi():
    from brainstorm_b200 import B200Handler
    from brainstorm_b200._lib import lib, check
    return B200Handler(seed=3), lib, check


@pytest.mark.parametrize('rows,cols,axis', [(4096, 1000, 0), (3000, 515, 0), (5000, 640, -1),
                                            (777, 333, 1), (65536, 16, 0)])
def test_static_scratch_sum_matches_scratch_sum_twice(rows, cols, axis):
    H, lib, check = _abi()
    rs = np.random.RandomState(rows + cols)
    nout = {0: cols, 1: rows, -1: 1}[axis]
    need = lib.b200_sum_t_scratch_floats(rows, cols, cols, axis)
    assert need <= lib.b200_sum_t_static_max_scratch_floats()
    scratch = H.allocate((max(int(need), 1),))
    for call in range(2):   # second call: the built-in array holds stale partials
        a = rs.uniform(-4, 4, (rows, cols)).astype(np.float32)
        da = H.create_from_numpy(a)
        want, got = H.zeros((nout,)), H.zeros((nout,))
        check(lib.b200_sum_t(da.ptr, rows, cols, cols, axis, want.ptr, scratch.ptr, scratch.size))
        check(lib.b200_sum_t_static(da.ptr, rows, cols, cols, axis, got.ptr))
        w, g = H.get_numpy_copy(want), H.get_numpy_copy(got)
        exact = a.astype(np.float64).sum(axis=None if axis < 0 else axis).reshape(nout)
        scale = np.abs(a).astype(np.float64).sum(axis=None if axis < 0 else axis).reshape(nout)
        assert np.all(np.abs(g - w) <= 1e-5 * np.abs(w) + 1e-5 * scale), (call, np.abs(g - w).max())
        assert np.array_equal(g, w), 'same kernels, same order: expected identical bits'
        assert np.all(np.abs(g - exact) <= 1e-5 * scale)


def test_static_scratch_rejects_oversize_and_does_not_touch_out():
    H, lib, check = _abi()
    rows, cols, ld = 300000, 3, 4         # the sum over everything of a pitched view keeps one partial per row
    assert lib.b200_sum_t_scratch_floats(rows, cols, ld, -1) > lib.b200_sum_t_static_max_scratch_floats()
    out = H.ones((1,))
    rc = lib.b200_sum_t_static(0, rows, cols, ld, -1, out.ptr)
    assert rc != 0
    msg = lib.b200_last_error().decode()
    assert 'built-in array' in msg and 'b200_sum_t' in msg
    assert (H.get_numpy_copy(out) == 1).all()


def test_static_scratch_sum_of_a_row_pitched_view():
    """Sum over everything of a view whose rows are 520 floats apart but 515 long: the
    row sums and the partials of their sum share the built-in array."""
    H, lib, check = _abi()
    rows, cols, ld = 3000, 515, 520
    rs = np.random.RandomState(11)
    need = lib.b200_sum_t_scratch_floats(rows, cols, ld, -1)
    assert 0 < need <= lib.b200_sum_t_static_max_scratch_floats()
    scratch = H.allocate((int(need),))
    for call in range(2):
        full = rs.uniform(-4, 4, (rows, ld)).astype(np.float32)
        d = H.create_from_numpy(full)
        want, got = H.zeros((1,)), H.zeros((1,))
        check(lib.b200_sum_t(d.ptr, rows, cols, ld, -1, want.ptr, scratch.ptr, scratch.size))
        check(lib.b200_sum_t_static(d.ptr, rows, cols, ld, -1, got.ptr))
        w, g = H.get_numpy_copy(want), H.get_numpy_copy(got)
        a = full[:, :cols].astype(np.float64)
        assert np.array_equal(g, w)
        assert abs(float(g[0]) - a.sum()) <= 1e-5 * np.abs(a).sum()
