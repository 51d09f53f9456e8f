"""Tolerances of the parity tests, in one place.

Integer / index work (binarize_v, index_m_by_v, masks, copies, fills) must be
bit-exact.  fp32 elementwise ops: relative error <= 1e-6 (plus an absolute floor
of a few ulp of 1.0 where the formula itself cancels, e.g. exp(x) - 1 in `el`).
Reductions and GEMMs: |got - ref| <= 1e-5 * |ref| + 1e-5 * scale, where scale is
the sum of absolute values of the terms of that output element; the CPU
reference itself is only that accurate (its float32 sums are sequential).
"""
import numpy as np

ELEMENTWISE_RTOL = 1e-6
REDUCTION_RTOL = 1e-5

BIT_EXACT_OPS = {'binarize_v', 'index_m_by_v', 'fill', 'copy_to', 'copy_to_if', 'fill_if',
                 'broadcast_t', 'merge_tt', 'abs_t', 'sign_t', 'clip_t', 'rel', 'rel_deriv',
                 'maxpool2d_forward_batch'}
ABS_FLOOR = {'el': 5e-7, 'el_deriv': 5e-7, 'modulo_tt': 0.0}


def assert_bits_equal(got, want, what=''):
    got = np.ascontiguousarray(got, dtype=np.float32)
    want = np.ascontiguousarray(want, dtype=np.float32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    # +0.0 and -0.0 compare equal here on purpose: the sign of zero of x*(x>0) is
    # not part of the contract.
    same = (got == want) | (np.isnan(got) & np.isnan(want))
    assert same.all(), '%s: %d of %d elements differ' % (what, (~same).sum(), same.size)


def assert_elementwise_close(got, want, op='', what=''):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    atol = ABS_FLOOR.get(op, 1e-37)
    err = np.abs(got - want)
    bound = ELEMENTWISE_RTOL * np.abs(want) + atol
    bad = ~((err <= bound) | (np.isnan(got) & np.isnan(want)) | (got == want))
    assert not bad.any(), '%s %s: max rel err %.3g at %d elements' % (
        op, what, float(np.max(err[bad] / np.maximum(np.abs(want[bad]), 1e-300))), int(bad.sum()))


def assert_reduction_close(got, want, scale, op='', what=''):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = np.abs(got - want)
    bound = REDUCTION_RTOL * np.abs(want) + REDUCTION_RTOL * np.asarray(scale, dtype=np.float64) + 1e-37
    bad = ~(err <= bound)
    assert not bad.any(), '%s %s: max err/bound %.3g at %d elements' % (
        op, what, float(np.max(err[bad] / bound[bad] if np.ndim(bound) else err[bad] / bound)), int(bad.sum()))


def reduction_scale(op, arrays, kwargs, call):
    """Sum of |terms| per output element of a reduction / GEMM case."""
    if op == 'sum_t':
        axis = call[1]
        a = np.abs(arrays['a'].astype(np.float64))
        out = arrays['out']
        if axis is None:
            return a.sum()
        return a.sum(axis=axis).reshape(out.shape)
    if op in ('dot_mm', 'dot_add_mm'):
        a = np.abs(arrays['a'].astype(np.float64))
        b = np.abs(arrays['b'].astype(np.float64))
        s = np.dot(a.T if kwargs.get('transa') else a, b.T if kwargs.get('transb') else b)
        if op == 'dot_add_mm':
            s = s + np.abs(arrays['out'])
        return s
    if op == 'softmax_m':
        return 1.0
    if op.startswith(('conv2d', 'avgpool2d', 'maxpool2d')):
        # sums of a few dozen terms of order one: one scale for all outputs
        return float(max(np.abs(v).max() for v in arrays.values() if v.size) *
                     max(np.prod(arrays['w'].shape[1:]) if 'w' in arrays else 16, 16))
    raise KeyError(op)


REDUCTION_OPS = {'sum_t', 'dot_mm', 'dot_add_mm', 'softmax_m', 'conv2d_forward_batch', 'conv2d_backward_batch',
                 'avgpool2d_forward_batch', 'avgpool2d_backward_batch', 'maxpool2d_backward_batch'}
