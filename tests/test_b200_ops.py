"""GPU parity of every handler op, through the C-ABI, against (1) the stored
outputs of the reference's NumpyHandler and (2) the oracle on larger seeded
inputs.  Mirrors brainstorm/tests/test_handlers_against_reference.py:30-66: all
array arguments are compared after the call, not only `out`."""
import os

import numpy as np
import pytest

import cases as golden_cases
import parity
from oracle.numpy_oracle import OracleHandler, op_suite_inputs

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), 'golden', 'handler_ops.npz'))
CASES = golden_cases.build_cases()


@pytest.fixture(scope='module')
def H():
    from brainstorm_b200 import B200Handler
    return B200Handler(seed=4711, rng_mode='host')


def _compare(op, name, got, want, scale=None):
    if op in parity.BIT_EXACT_OPS:
        parity.assert_bits_equal(got, want, '%s.%s' % (op, name))
    elif op in parity.REDUCTION_OPS:
        parity.assert_reduction_close(got, want, scale, op, name)
    else:
        parity.assert_elementwise_close(got, want, op, name)


@pytest.mark.parametrize('idx', range(len(CASES)), ids=[c.id for c in CASES])
def test_op_against_reference_golden(H, idx):
    c = CASES[idx]
    if c.op.endswith('_deriv'):
        c.arrays['y'] = GOLDEN['%d/y' % idx]
    if c.op == 'maxpool2d_backward_batch':
        c.arrays['out'], c.arrays['argmax'] = GOLDEN['%d/out' % idx], GOLDEN['%d/argmax' % idx]
    dev = {k: H.create_from_numpy(v) for k, v in c.arrays.items()}
    getattr(H, c.op)(*c.bind(dev), **c.kwargs)
    scale = parity.reduction_scale(c.op, c.arrays, c.kwargs, c.call) \
        if c.op in parity.REDUCTION_OPS else None
    for name, d in dev.items():
        key = '%d/%s' % (idx, name)
        changed = key in GOLDEN.files and not (name == 'y' and c.op.endswith('_deriv')) and not (
            name in ('out', 'argmax') and c.op == 'maxpool2d_backward_batch')
        want = GOLDEN[key] if key in GOLDEN.files else c.arrays[name]
        got = H.get_numpy_copy(d)
        if changed:
            _compare(c.op, name, got, want, scale)
        else:  # inputs must come back untouched
            parity.assert_bits_equal(got, want, '%s.%s (input)' % (c.op, name))


def test_host_rng_mode_matches_reference(H):
    from brainstorm_b200 import B200Handler
    h = B200Handler(seed=4711, rng_mode='host')
    mask = h.allocate((6, 50))
    h.generate_probability_mask(mask, 0.3)
    gauss = h.allocate((5, 40))
    h.fill_gaussian(0.5, 2.0, gauss)
    parity.assert_bits_equal(h.get_numpy_copy(mask), GOLDEN['rng/mask'])
    parity.assert_bits_equal(h.get_numpy_copy(gauss), GOLDEN['rng/gauss'])


def test_device_rng_statistics(H):
    from brainstorm_b200 import B200Handler
    h = B200Handler(seed=99, rng_mode='device')
    mask = h.allocate((1000, 1003))
    h.generate_probability_mask(mask, 0.3)
    m = h.get_numpy_copy(mask)
    assert set(np.unique(m)) <= {0.0, 1.0}
    assert abs(m.mean() - 0.3) < 3e-3
    mask2 = h.allocate((1000, 1003))
    h.generate_probability_mask(mask2, 0.3)
    assert (h.get_numpy_copy(mask2) != m).mean() > 0.3   # a fresh stream per call
    g = h.allocate((777, 1001))
    h.fill_gaussian(1.5, 2.0, g)
    gg = h.get_numpy_copy(g)
    assert abs(gg.mean() - 1.5) < 2e-2 and abs(gg.std() - 2.0) < 2e-2
    assert np.isfinite(gg).all()


# ---- the op suite of the benchmark at its CPU-runnable size ----------------------
def _suite(H, O, rows, cols, seed):
    d = op_suite_inputs(rows, cols, seed)
    a, b, dy, row, col, div = d['a'], d['b'], d['dy'], d['row'], d['col'], d['div']
    labels = d['labels'].astype(np.float32)
    z = np.zeros_like(a)
    yield 'add_tt', (a, b, z), {}
    yield 'subtract_tt', (a, b, z), {}
    yield 'mult_tt', (a, b, z), {}
    yield 'divide_tt', (a, div, z), {}
    yield 'add_mv', (a, row, z), {}
    yield 'add_mv', (a, col, z), {}
    yield 'mult_mv', (a, row, z), {}
    yield 'mult_mv', (a, col, z), {}
    yield 'mult_st', (0.37, a, z), {}
    for act in ('sigmoid', 'tanh', 'rel', 'el'):
        yield act, (a, z), {}
        y = np.zeros_like(a)
        getattr(O, act)(a, y)
        yield act + '_deriv', (a, y, dy, z), {}
    yield 'sum_t', (a, 0, np.zeros((1, cols), np.float32)), {}
    yield 'sum_t', (a, 1, np.zeros((rows, 1), np.float32)), {}
    yield 'sum_t', (a, None, np.zeros((), np.float32)), {}
    yield 'softmax_m', (a, z), {}
    yield 'clip_t', (a, -1.0, 1.0, z), {}
    yield 'abs_t', (a, z), {}
    yield 'sign_t', (a, z), {}
    yield 'sqrt_t', (np.abs(a), z), {}
    yield 'binarize_v', (labels, z), {}
    yield 'index_m_by_v', (a, labels, np.zeros((rows, 1), np.float32)), {}


@pytest.mark.parametrize('rows,cols,seed', [(1024, 1024, 0), (515, 1030, 3), (2048, 205, 5)])
def test_op_suite_against_oracle(H, rows, cols, seed):
    O = OracleHandler(np.float32)
    for op, args, kwargs in _suite(H, O, rows, cols, seed):
        host = [x.copy() if isinstance(x, np.ndarray) else x for x in args]
        dev = [H.create_from_numpy(x) if isinstance(x, np.ndarray) else x for x in args]
        getattr(O, op)(*host, **kwargs)
        getattr(H, op)(*dev, **kwargs)
        got = H.get_numpy_copy(dev[-1])
        want = host[-1]
        if op == 'sum_t':
            axis = args[1]
            absa = np.abs(args[0].astype(np.float64))
            scale = absa.sum() if axis is None else absa.sum(axis=axis).reshape(want.shape)
            parity.assert_reduction_close(got, want, scale, op, str(axis))
            # and at least as close to the exact sum as the float32 CPU result is
            exact = args[0].astype(np.float64).sum(axis=axis).reshape(want.shape)
            assert (np.abs(got - exact) <= 1e-5 * scale + 1e-37).all()
        elif op == 'softmax_m':
            parity.assert_reduction_close(got, want, 0.0, op)
        else:
            _compare(op, 'out', got, want)


def test_bad_label_is_reported_not_read(H):
    m = H.create_from_numpy(np.arange(12, dtype=np.float32).reshape(3, 4))
    v = H.create_from_numpy(np.array([[1], [7], [2]], np.float32))
    out = H.zeros((3, 1))
    H.index_m_by_v(m, v, out)
    with pytest.raises(IndexError):
        H.get_numpy_copy(out)
    # the flag is cleared; the valid rows were still gathered
    assert H.get_numpy_copy(out).ravel().tolist() == [1.0, 0.0, 10.0]


def test_is_fully_finite(H):
    a = np.random.RandomState(0).randn(300, 70).astype(np.float32)
    assert H.is_fully_finite(H.create_from_numpy(a))
    a[299, 69] = np.inf
    assert not H.is_fully_finite(H.create_from_numpy(a))
    a[299, 69] = 0
    a[0, 0] = np.nan
    assert not H.is_fully_finite(H.create_from_numpy(a))
    assert H.is_fully_finite(H.allocate((0,)))


def test_allocate_is_zero_filled_and_ones(H):
    assert not H.get_numpy_copy(H.allocate((37, 5))).any()
    assert (H.get_numpy_copy(H.ones((3, 2, 5))) == 1).all()
    assert H.get_numpy_copy(H.zeros(())).shape == ()


def test_errors_are_exceptions(H):
    from brainstorm_b200 import B200Error
    a = H.zeros((4, 4))
    with pytest.raises(ValueError):
        H.add_tt(a, H.zeros((4, 5)), a)
    with pytest.raises(ValueError):
        H.dot_mm(a, H.zeros((5, 4)), a)
    with pytest.raises(AssertionError):
        H.set_from_numpy(a, np.zeros((3, 3)))
    from brainstorm_b200._lib import lib, check
    with pytest.raises(B200Error):
        check(lib.b200_sum_t(a.ptr, 4, 4, 4, 7, a.ptr, 0, 0))


# ---- GEMM: tensor-core path (tcgen05 + TMA, 3xTF32) and CUDA-core path ----------------
GEMM_SHAPES = [(128, 128, 64), (256, 512, 96), (300, 1000, 1000), (128, 4000, 1000),
               (100, 1200, 784), (1000, 205, 1000), (12, 1000, 12672), (1000, 1000, 2500)]


@pytest.mark.parametrize('M,N,K', GEMM_SHAPES, ids=['%dx%dx%d' % s for s in GEMM_SHAPES])
@pytest.mark.parametrize('path', [0, 1], ids=['auto', 'cuda-core'])
def test_gemm_all_transposes_against_oracle(H, M, N, K, path):
    from brainstorm_b200._lib import lib, check
    O = OracleHandler(np.float32)
    rs = np.random.RandomState(M + N + K)
    check(lib.b200_set_tuning(2, path))
    try:
        for ta in (False, True):
            for tb in (False, True):
                a = rs.randn(*((K, M) if ta else (M, K))).astype(np.float32)
                b = rs.randn(*((N, K) if tb else (K, N))).astype(np.float32)
                c0 = rs.randn(M, N).astype(np.float32)
                scale = np.abs(a.T if ta else a).astype(np.float64) @ np.abs(b.T if tb else b)
                for op in ('dot_mm', 'dot_add_mm'):
                    want = c0.copy()
                    getattr(O, op)(a, b, want, transa=ta, transb=tb)
                    dc = H.create_from_numpy(c0)
                    getattr(H, op)(H.create_from_numpy(a), H.create_from_numpy(b), dc, transa=ta, transb=tb)
                    parity.assert_reduction_close(H.get_numpy_copy(dc), want, scale + np.abs(c0), op,
                                                  '%s%s' % ('T' if ta else 'N', 'T' if tb else 'N'))
    finally:
        check(lib.b200_set_tuning(2, 0))


@pytest.mark.parametrize('K', [64, 512, 4096, 16384])
def test_gemm_same_sign_operands_keep_relative_accuracy(H, K):
    """All products positive: no cancellation hides a biased accumulation.  The
    tensor core truncates when it adds into its accumulator; the kernel's chunked
    drain must keep the bias below the 1e-5 bar for any K."""
    rs = np.random.RandomState(K)
    a = rs.uniform(0, 1, (256, K)).astype(np.float32)
    b = rs.uniform(0, 1, (192, K)).astype(np.float32)
    out = H.zeros((256, 192))
    H.dot_mm(H.create_from_numpy(a), H.create_from_numpy(b), out, transb=True)
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    rel = np.abs(H.get_numpy_copy(out) - ref) / ref
    assert rel.max() < 1e-5, rel.max()


def test_gemm_views_of_one_flat_buffer(H):
    """Operands as the memory layer hands them out: slices of one flat allocation
    at arbitrary element offsets (misaligned ones take the CUDA-core kernel)."""
    O = OracleHandler(np.float32)
    rs = np.random.RandomState(11)
    flat = rs.randn(400000).astype(np.float32)
    dflat = H.create_from_numpy(flat)
    for off in (0, 4, 3):
        a = flat[off:off + 256 * 300].reshape(256, 300)
        w = flat[100000 + off:100000 + off + 200 * 300].reshape(200, 300)
        da = dflat[off:off + 256 * 300].reshape((256, 300))
        dw = dflat[100000 + off:100000 + off + 200 * 300].reshape((200, 300))
        out = H.zeros((256, 200))
        want = np.zeros((256, 200), np.float32)
        H.dot_mm(da, dw, out, transb=True)
        O.dot_mm(a, w, want, transb=True)
        parity.assert_reduction_close(H.get_numpy_copy(out), want, np.abs(a) @ np.abs(w.T), 'dot_mm', 'offset %d' % off)


def test_overlapped_upload_orders_with_compute(H):
    """upload_async / upload_join: a batch uploaded on the second stream while
    kernels run is visible to the kernels queued after the join, and an upload into
    a buffer waits for the event of the kernels that still read it."""
    n = 1 << 22
    src0, src1 = H.pinned_empty((n,)), H.pinned_empty((n,))
    src0[:] = np.arange(n, dtype=np.float32)
    src1[:] = -np.arange(n, dtype=np.float32)
    buf, out = H.allocate((n,)), H.allocate((n,))
    H.upload_async(buf, src0)
    H.upload_join()
    H.mult_st(2.0, buf, out)                 # reads buf
    ev = H.record_event()
    H.upload_async(buf, src1, ev)            # may not overwrite buf before the kernel above is done
    first = H.get_numpy_copy(out)
    H.upload_join()
    H.mult_st(2.0, buf, out)
    second = H.get_numpy_copy(out)
    assert np.array_equal(first, 2 * src0) and np.array_equal(second, 2 * src1)
    with pytest.raises(ValueError):
        H.upload_async(buf, np.zeros(n - 1, np.float32))


def test_zero_size_operands_are_no_ops(H):
    """The memory layer first creates every time/batch-sized buffer for a 0 x 0 batch
    (buffers.py:67,108): every op must accept empty operands."""
    for shape in ((0, 5), (3, 0), (1, 0, 7)):
        a, b, out = H.zeros(shape), H.zeros(shape), H.zeros(shape)
        H.add_tt(a, b, out)
        H.mult_st(2.0, a, out)
        H.sigmoid(a, out)
        H.tanh_deriv(None, a, b, out)
        H.fill(out, 1.0)
        H.copy_to(a, out)
        assert H.get_numpy_copy(out).shape == shape
        assert H.is_fully_finite(a)
    m = H.zeros((0, 5))
    H.add_mv(m, H.ones((1, 5)), m)
    H.softmax_m(m, m)
    s = H.ones((1, 5))
    H.sum_t(m, 0, s)                       # the empty sum is 0
    assert not H.get_numpy_copy(s).any()
    tot = H.ones(())
    H.sum_t(m, None, tot)
    assert float(H.get_numpy_copy(tot)) == 0.0
    H.binarize_v(H.zeros((0, 1)), m)
    H.index_m_by_v(m, H.zeros((0, 1)), H.zeros((0, 1)))
    out = H.ones((4, 3))
    H.dot_mm(H.zeros((4, 0)), H.zeros((0, 3)), out)      # empty contraction: zeros
    assert not H.get_numpy_copy(out).any()
    H.dot_add_mm(H.zeros((4, 0)), H.zeros((0, 3)), out)
    H.dot_mm(H.zeros((0, 6)), H.zeros((6, 3)), H.zeros((0, 3)))
    H.synchronize()
