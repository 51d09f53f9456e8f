"""B200Array must slice and reshape exactly like numpy for everything the
reference's memory layer does (buffers.py:82, buffer_structure.py:218-245,
lstm_layer.py:106-117, tests/test_array.py of the reference)."""
import numpy as np
import pytest

from brainstorm_b200.array import B200Array


def view_of(shape):
    """An unbacked view (no device memory) plus a numpy array whose values are
    the element offsets, so that offsets/strides can be compared."""
    n = int(np.prod(shape))
    return B200Array(None, 0, tuple(shape)), np.arange(n, dtype=np.int64).reshape(shape)


def same(view, ref):
    assert view.shape == ref.shape
    assert view.size == ref.size
    if ref.size == 0:
        return
    first = ref.reshape(-1)[0] if ref.flags.c_contiguous else ref[(0,) * ref.ndim]
    assert view.ptr == int(first) * 4
    for n, s, rs in zip(view.shape, view.strides, ref.strides):
        if n > 1:
            assert s * 8 == rs
    assert view.is_contiguous == (ref.flags.c_contiguous or ref.size <= 1)


KEYS = [0, -1, 2, slice(None), slice(1, None), slice(None, -1), slice(1, -1), slice(None, -2),
        (slice(None), 1), (0, slice(None), slice(2, 4)), (slice(1, 3), slice(None), slice(0, 3)),
        (slice(None), slice(1, 2)), (-1, -1), (1, 2, 3), (Ellipsis, 1), (slice(0, 0),),
        (slice(None), slice(None), slice(1, 5))]


@pytest.mark.parametrize('key', KEYS, ids=[str(k) for k in KEYS])
def test_getitem_matches_numpy(key):
    v, r = view_of((4, 3, 5))
    same(v[key], r[key])


def test_chained_views_and_reshape():
    v, r = view_of((101, 8, 10))
    same(v[:-1].reshape((100 * 8, 10)), r[:-1].reshape((800, 10)))
    same(v[5 - 6], r[-1])
    same(v[1:-1].reshape(99 * 8, 10)[3], r[1:-1].reshape(792, 10)[3])
    same(v.reshape(-1), r.reshape(-1))
    same(v.reshape((808, -1)), r.reshape((808, -1)))
    flat, rflat = view_of((1000,))
    same(flat[120:360].reshape((2, 12, 10)), rflat[120:360].reshape((2, 12, 10)))
    same(flat[7:8].reshape(()), rflat[7:8].reshape(()))


def test_strided_feature_slice_has_row_pitched_form():
    v, r = view_of((6, 4, 10))
    s = v[:, :, 2:7]
    assert not s.is_contiguous
    assert s.as_2d() == (24, 5, 10)
    same(s.reshape((24, 5)), r[:, :, 2:7].reshape((24, 5)))
    with pytest.raises(ValueError):
        s.reshape((120,))
    t = v[1:4, :, 2:7]
    assert t.as_2d() == (12, 5, 10)
    col = v.reshape((24, 10))[:, 3:4]
    assert col.as_2d() == (24, 1, 10)
    assert v[:, 1].as_2d() == (6, 10, 40)
    assert v[:, :, ::2].as_2d() == (120, 1, 2)
    assert v[:, ::2, ::2].as_2d() is None
    assert v[2].as_2d() == (1, 40, 40)


def test_zero_size_arrays():
    v, r = view_of((1, 0, 7))
    same(v[:-1], r[:-1])
    same(v.reshape((0, 7)), r.reshape((0, 7)))
    assert v.size == 0 and v[0:].shape == (1, 0, 7)
    with pytest.raises(ValueError):
        v.reshape((3, 3))


def test_index_errors():
    v, _ = view_of((4, 3))
    with pytest.raises(IndexError):
        v[4]
    with pytest.raises(IndexError):
        v[0, 0, 0]
    with pytest.raises(ValueError):
        v.reshape((5, 5))


@pytest.mark.gpu
def test_strided_views_on_device():
    from brainstorm_b200 import B200Handler
    import parity
    H = B200Handler(rng_mode='host', seed=1)
    rs = np.random.RandomState(5)
    big = rs.randn(6, 4, 10).astype(np.float32)
    dev = H.create_from_numpy(big)
    parity.assert_bits_equal(H.get_numpy_copy(dev[:, :, 2:7]), big[:, :, 2:7])
    # write through a strided view, neighbours untouched
    part = rs.randn(6, 4, 5).astype(np.float32)
    H.set_from_numpy(dev[:, :, 2:7], part)
    big[:, :, 2:7] = part
    parity.assert_bits_equal(H.get_numpy_copy(dev), big)
    # elementwise, broadcast, reduction and GEMM on strided operands
    a, b = dev[:, :, 0:5], dev[:, :, 5:10]
    out = H.zeros((6, 4, 5))
    H.add_tt(a, b, out)
    parity.assert_elementwise_close(H.get_numpy_copy(out), big[:, :, 0:5] + big[:, :, 5:10])
    H.tanh(a, a)
    big[:, :, 0:5] = np.tanh(big[:, :, 0:5])
    parity.assert_elementwise_close(H.get_numpy_copy(dev), big)
    m = dev.reshape((24, 10))[:, 1:9]
    rowv = H.create_from_numpy(rs.randn(1, 8).astype(np.float32))
    H.mult_mv(m, rowv, m)
    big.reshape(24, 10)[:, 1:9] *= H.get_numpy_copy(rowv)
    parity.assert_elementwise_close(H.get_numpy_copy(dev), big)
    s = H.zeros((1, 8))
    H.sum_t(m, 0, s)
    ref = big.reshape(24, 10)[:, 1:9]
    parity.assert_reduction_close(H.get_numpy_copy(s), ref.sum(0, keepdims=True), np.abs(ref).sum(0, keepdims=True))
    s1 = H.zeros((24,))
    H.sum_t(m, 1, s1)
    parity.assert_reduction_close(H.get_numpy_copy(s1), ref.sum(1), np.abs(ref).sum(1))
    s2 = H.zeros(())
    H.sum_t(m, None, s2)
    parity.assert_reduction_close(H.get_numpy_copy(s2), ref.sum(), np.abs(ref).sum())
    w = H.create_from_numpy(rs.randn(3, 8).astype(np.float32))
    o = H.zeros((24, 3))
    H.dot_mm(m, w, o, transb=True)
    wn = H.get_numpy_copy(w)
    parity.assert_reduction_close(H.get_numpy_copy(o), ref @ wn.T, np.abs(ref) @ np.abs(wn.T))
    sm = H.zeros((24, 8))
    H.softmax_m(m, sm)
    e = np.exp(ref - ref.max(1, keepdims=True))
    parity.assert_reduction_close(H.get_numpy_copy(sm), e / e.sum(1, keepdims=True), 0.0)
    H.fill(dev[:, :, 9:10], 7.0)
    big[:, :, 9:10] = 7.0
    got = H.get_numpy_copy(dev)
    parity.assert_elementwise_close(got, big)
    parity.assert_bits_equal(got[:, :, 9], big[:, :, 9])


@pytest.mark.gpu
def test_merge_split_broadcast_on_feature_slices():
    """merge_tt / split_add_tt / broadcast_t on the row-pitched views that a hub with
    several sources hands out (buffer[:, :, f0:f1], buffer_structure.py:232-245),
    against the same numpy expressions NumpyHandler uses (numpy_handler.py:221,251,103)."""
    from brainstorm_b200 import B200Handler
    import parity
    H = B200Handler(rng_mode='host', seed=1)
    rs = np.random.RandomState(8)
    T, B = 5, 7
    hub = rs.randn(T, B, 20).astype(np.float32)
    dev = H.create_from_numpy(hub)
    # merge: two strided sources into a strided destination of a second hub
    hub2 = rs.randn(T, B, 16).astype(np.float32)
    dev2 = H.create_from_numpy(hub2)
    H.merge_tt(dev[:, :, 2:7], dev[:, :, 11:15], dev2[:, :, 3:12])
    hub2[:, :, 3:12] = np.concatenate((hub[:, :, 2:7], hub[:, :, 11:15]), axis=-1)
    parity.assert_bits_equal(H.get_numpy_copy(dev2), hub2, 'merge_tt strided')
    # merge: contiguous sources, strided destination, and the other way round
    a, b = rs.randn(T, B, 4).astype(np.float32), rs.randn(T, B, 3).astype(np.float32)
    H.merge_tt(H.create_from_numpy(a), H.create_from_numpy(b), dev2[:, :, 0:7])
    hub2[:, :, 0:7] = np.concatenate((a, b), axis=-1)
    parity.assert_bits_equal(H.get_numpy_copy(dev2), hub2, 'merge_tt into a slice')
    out = H.zeros((T, B, 9))
    H.merge_tt(dev[:, :, 0:4], dev[:, :, 4:9], out)
    parity.assert_bits_equal(H.get_numpy_copy(out), hub[:, :, 0:9], 'merge_tt from slices')
    # split_add: accumulates the two column ranges of x into two strided outputs
    x = rs.randn(T, B, 9).astype(np.float32)
    H.split_add_tt(H.create_from_numpy(x), dev[:, :, 1:5], dev[:, :, 10:15])
    hub[:, :, 1:5] += x[:, :, :4]
    hub[:, :, 10:15] += x[:, :, 4:]
    parity.assert_elementwise_close(H.get_numpy_copy(dev), hub, 'split_add_tt')
    xs = dev2[:, :, 2:11]
    oa, ob = H.ones((T, B, 4)), H.ones((T, B, 5))
    H.split_add_tt(xs, oa, ob)
    parity.assert_elementwise_close(H.get_numpy_copy(oa), 1 + hub2[:, :, 2:6], 'split_add_tt')
    parity.assert_elementwise_close(H.get_numpy_copy(ob), 1 + hub2[:, :, 6:11], 'split_add_tt')
    # broadcast along time, batch and features into a strided destination
    for axis, shape in ((0, (1, B, 6)), (1, (T, 1, 6)), (2, (T, B, 1))):
        src = rs.randn(*shape).astype(np.float32)
        H.broadcast_t(H.create_from_numpy(src), axis, dev[:, :, 8:14])
        hub[:, :, 8:14] = np.broadcast_to(src, (T, B, 6))
        parity.assert_bits_equal(H.get_numpy_copy(dev), hub, 'broadcast_t axis %d' % axis)
    # a strided source
    H.broadcast_t(dev2[:, :, 5:6], 2, dev[:, :, 0:3])
    hub[:, :, 0:3] = np.broadcast_to(hub2[:, :, 5:6], (T, B, 3))
    parity.assert_bits_equal(H.get_numpy_copy(dev), hub, 'broadcast_t from a slice')
    # uploads into a slice on the upload stream
    part = H.pinned_empty((T, B, 5))
    part[...] = rs.randn(T, B, 5)
    H.upload_async(dev[:, :, 15:20], part)
    H.upload_join()
    hub[:, :, 15:20] = part
    parity.assert_bits_equal(H.get_numpy_copy(dev), hub, 'upload_async into a slice')
