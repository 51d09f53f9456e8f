"""Seeded handler-op cases shared by the golden-vector generator and the tests.

Every case names a ``Handler`` method, a dict of numpy input arrays and a call
template whose string entries refer to those arrays (the same name twice means
the *same* array object, i.e. an aliased call such as ``add_tt(a, b, a)``).
Inputs come from the legacy ``np.random.RandomState`` streams, which numpy keeps
frozen across versions, so only the outputs need to be stored.

The shapes start from those of the reference's own parity tests
(brainstorm/tests/test_handlers_against_reference.py:24-25) and add ragged,
odd-pitch and non-multiple-of-4 ones.
"""
from __future__ import annotations

from collections import OrderedDict

import numpy as np

F32 = np.float32

REF_2D_SHAPES = ((1, 1), (4, 1), (1, 4), (5, 5), (3, 4), (4, 3))
EXTRA_2D_SHAPES = ((7, 205), (19, 67))
SHAPES_2D = REF_2D_SHAPES + EXTRA_2D_SHAPES
SHAPES_ND = ((1, 1, 4), (1, 1, 3, 3), (3, 4, 2, 1))
GEMM_MKN = ((1, 1, 1), (4, 3, 5), (5, 5, 5), (7, 205, 12), (19, 67, 33),
            (3, 130, 64))
ACTIVATIONS = ('sigmoid', 'tanh', 'rel', 'el')


class Case(object):
    def __init__(self, op, arrays, call, kwargs=None, tag=''):
        self.op = op
        self.arrays = OrderedDict(arrays)
        self.call = list(call)
        self.kwargs = dict(kwargs or {})
        self.tag = tag

    @property
    def id(self):
        shp = 'x'.join(str(s) for s in next(iter(self.arrays.values())).shape)
        return '%s[%s%s]' % (self.op, shp, ('-' + self.tag) if self.tag else '')

    def fresh_arrays(self):
        return OrderedDict((k, v.copy()) for k, v in self.arrays.items())

    def bind(self, arrays):
        """Positional arguments for the handler call from a name->array dict."""
        return [arrays[c] if isinstance(c, str) else c for c in self.call]


def _randn(rs, shape):
    return rs.standard_normal(shape).astype(F32)


def _uniform(rs, shape, lo, hi):
    return (rs.uniform(lo, hi, shape)).astype(F32)


def _special(rs, shape):
    """Values with exact zeros, negative zeros and large magnitudes mixed in."""
    a = _randn(rs, shape) * F32(3)
    flat = a.reshape(-1)
    if flat.size >= 4:
        flat[0] = 0.0
        flat[1] = -0.0
        flat[2] = 30.0
        flat[3] = -30.0
    return a


def build_cases():
    rs = np.random.RandomState(20240607)
    cases = []
    add = cases.append

    for shape in SHAPES_2D + SHAPES_ND:
        a, b = _randn(rs, shape), _randn(rs, shape)
        div = _uniform(rs, shape, 0.5, 4.0) * np.where(
            rs.uniform(size=shape) < 0.5, F32(-1), F32(1)).astype(F32)
        acc = _randn(rs, shape)
        z = np.zeros(shape, F32)
        for op in ('add_tt', 'subtract_tt', 'mult_tt'):
            add(Case(op, [('a', a), ('b', b), ('out', z)], ['a', 'b', 'out']))
        add(Case('divide_tt', [('a', a), ('b', div), ('out', z)],
                 ['a', 'b', 'out']))
        add(Case('mult_add_tt', [('a', a), ('b', b), ('out', acc)],
                 ['a', 'b', 'out']))
        add(Case('add_tt', [('a', a), ('b', b)], ['a', 'b', 'a'], tag='alias'))
        add(Case('mult_tt', [('a', a), ('out', z)], ['a', 'a', 'out'],
                 tag='square'))
        add(Case('modulo_tt', [('a', np.round(a * 7)), ('b', np.round(div * 2)
                                                        + F32(0.0)),
                               ('out', z)], ['a', 'b', 'out']))
        for s, tag in ((0.37, 's0'), (-1, 's1'), (3, 's2')):
            add(Case('add_st', [('t', a), ('out', z)], [s, 't', 'out'], tag=tag))
            add(Case('mult_st', [('t', a), ('out', z)], [s, 't', 'out'], tag=tag))
            add(Case('mult_add_st', [('t', a), ('out', acc)], [s, 't', 'out'],
                     tag=tag))
        add(Case('mult_st', [('t', a)], [0.9, 't', 't'], tag='alias'))
        sp = _special(rs, shape)
        add(Case('abs_t', [('a', sp), ('out', z)], ['a', 'out']))
        add(Case('sign_t', [('a', sp), ('out', z)], ['a', 'out']))
        add(Case('sqrt_t', [('a', np.abs(sp)), ('out', z)], ['a', 'out']))
        add(Case('log_t', [('a', np.abs(sp) + F32(0.1)), ('out', z)],
                 ['a', 'out']))
        add(Case('clip_t', [('a', sp), ('out', z)], ['a', -1.0, 1.0, 'out']))
        add(Case('clip_t', [('a', np.abs(sp) * F32(0.2)), ('out', z)],
                 ['a', 1e-6, 1.0, 'out'], tag='ce'))
        add(Case('fill', [('mem', a)], ['mem', 0.25]))
        add(Case('copy_to', [('src', a), ('dest', z)], ['src', 'dest']))
        cond = (rs.uniform(size=shape) < 0.5).astype(F32)
        add(Case('copy_to_if', [('src', a), ('dest', b), ('cond', cond)],
                 ['src', 'dest', 'cond']))
        add(Case('fill_if', [('mem', a), ('cond', cond)], ['mem', -2.5, 'cond']))
        add(Case('add_into_if', [('a', a), ('out', b), ('cond', cond)],
                 ['a', 'out', 'cond']))
        for act in ACTIVATIONS:
            x = _special(rs, shape)
            add(Case(act, [('x', x), ('y', z)], ['x', 'y']))
            add(Case(act, [('x', x)], ['x', 'x'], tag='inplace'))
            # derivative cases get y = f(x) filled in by finalize_derivs()
            add(Case(act + '_deriv', [('x', x), ('y', z), ('dy', _randn(rs, shape)),
                                      ('dx', z)], ['x', 'y', 'dy', 'dx']))
            add(Case(act + '_deriv', [('x', x), ('y', z), ('dy', _randn(rs, shape))],
                     ['x', 'y', 'dy', 'dy'], tag='inplace'))

    for shape in SHAPES_2D:
        rows, cols = shape
        m = _randn(rs, shape)
        z = np.zeros(shape, F32)
        acc = _randn(rs, shape)
        row = _randn(rs, (1, cols))
        col = _randn(rs, (rows, 1))
        drow = _uniform(rs, (1, cols), 0.5, 4.0)
        dcol = -_uniform(rs, (rows, 1), 0.5, 4.0)
        for op in ('add_mv', 'subtract_mv', 'mult_mv', 'mult_add_mv'):
            base = acc if op == 'mult_add_mv' else z
            add(Case(op, [('m', m), ('v', row), ('out', base)],
                     ['m', 'v', 'out'], tag='row'))
            add(Case(op, [('m', m), ('v', col), ('out', base)],
                     ['m', 'v', 'out'], tag='col'))
        add(Case('divide_mv', [('m', m), ('v', drow), ('out', z)],
                 ['m', 'v', 'out'], tag='row'))
        add(Case('divide_mv', [('m', m), ('v', dcol), ('out', z)],
                 ['m', 'v', 'out'], tag='col'))
        add(Case('add_mv', [('m', m), ('v', row)], ['m', 'v', 'm'],
                 tag='row-alias'))
        add(Case('mult_mv', [('m', m), ('v', acc), ('out', z)],
                 ['m', 'v', 'out'], tag='full'))
        add(Case('sum_t', [('a', m), ('out', np.zeros((1, cols), F32))],
                 ['a', 0, 'out'], tag='ax0-keep'))
        add(Case('sum_t', [('a', m), ('out', np.zeros((cols,), F32))],
                 ['a', 0, 'out'], tag='ax0'))
        add(Case('sum_t', [('a', m), ('out', np.zeros((rows, 1), F32))],
                 ['a', 1, 'out'], tag='ax1-keep'))
        add(Case('sum_t', [('a', m), ('out', np.zeros((rows,), F32))],
                 ['a', 1, 'out'], tag='ax1'))
        add(Case('sum_t', [('a', m), ('out', np.zeros((), F32))],
                 ['a', None, 'out'], tag='all'))
        add(Case('softmax_m', [('m', m * F32(3)), ('out', z)], ['m', 'out']))
        add(Case('softmax_m', [('m', m * F32(3))], ['m', 'm'], tag='inplace'))
        labels = rs.randint(0, cols, size=(rows, 1)).astype(F32)
        add(Case('binarize_v', [('v', labels), ('out', acc)], ['v', 'out']))
        add(Case('index_m_by_v', [('m', m), ('v', labels),
                                  ('out', np.zeros((rows, 1), F32))],
                 ['m', 'v', 'out']))
        add(Case('broadcast_t', [('a', row), ('out', z)], ['a', 0, 'out'],
                 tag='ax0'))
        add(Case('broadcast_t', [('a', col), ('out', z)], ['a', 1, 'out'],
                 tag='ax1'))
        extra = _randn(rs, (rows, 3))
        add(Case('merge_tt', [('a', m), ('b', extra),
                              ('out', np.zeros((rows, cols + 3), F32))],
                 ['a', 'b', 'out']))
        add(Case('split_add_tt', [('x', _randn(rs, (rows, cols + 3))),
                                  ('out_a', m), ('out_b', extra)],
                 ['x', 'out_a', 'out_b']))

    for shape in SHAPES_ND:
        a = _randn(rs, shape)
        add(Case('sum_t', [('a', a), ('out', np.zeros((), F32))],
                 ['a', None, 'out'], tag='all-nd'))

    for (M, K, N) in GEMM_MKN:
        for ta in (False, True):
            for tb in (False, True):
                a = _randn(rs, (K, M) if ta else (M, K))
                b = _randn(rs, (N, K) if tb else (K, N))
                tag = ('T' if ta else 'N') + ('T' if tb else 'N') + \
                    '-%dx%dx%d' % (M, K, N)
                add(Case('dot_mm', [('a', a), ('b', b),
                                    ('out', np.zeros((M, N), F32))],
                         ['a', 'b', 'out'], dict(transa=ta, transb=tb), tag))
                add(Case('dot_add_mm', [('a', a), ('b', b),
                                        ('out', _randn(rs, (M, N)))],
                         ['a', 'b', 'out'], dict(transa=ta, transb=tb), tag))
    # convolution and pooling (NHWC), shapes after the reference's own tests
    # (test_handlers_against_reference.py:478-659) plus strides > 1
    def out_hw(H, W, kh, kw, pad, st):
        return (H + 2 * pad - kh) // st[0] + 1, (W + 2 * pad - kw) // st[1] + 1

    for (img, wsh, pad, st) in (((1, 3, 3, 1), (1, 1, 1), 1, (1, 1)), ((3, 8, 8, 1), (3, 3, 3), 1, (1, 1)),
                                ((2, 6, 4, 3), (6, 2, 2), 1, (1, 1)), ((1, 3, 4, 2), (2, 1, 3), 1, (1, 1)),
                                ((2, 7, 9, 4), (5, 3, 2), 2, (2, 1)), ((2, 8, 8, 3), (4, 3, 3), 0, (2, 2))):
        N, H, W, C = img
        x = _randn(rs, img)
        w = _uniform(rs, (wsh[0], wsh[1], wsh[2], C), 0.0, 1.0)
        b = _uniform(rs, (wsh[0],), 0.0, 1.0)
        oh, ow = out_hw(H, W, wsh[1], wsh[2], pad, st)
        tag = 'k%dx%d-p%d-s%dx%d' % (wsh[1], wsh[2], pad, st[0], st[1])
        add(Case('conv2d_forward_batch', [('x', x), ('w', w), ('b', b), ('out', np.zeros((N, oh, ow, wsh[0]), F32))],
                 ['x', 'w', 'b', 'out', pad, st], tag=tag))
        add(Case('conv2d_backward_batch',
                 [('x', x), ('w', w), ('in_deltas', _randn(rs, img)),
                  ('out_deltas', _uniform(rs, (N, oh, ow, wsh[0]), 0.0, 1.0)),
                  ('dw', _randn(rs, w.shape)), ('db', _randn(rs, b.shape))],
                 ['x', 'w', pad, st, 'in_deltas', 'out_deltas', 'dw', 'db'], tag=tag))

    for img in ((1, 5, 5, 1), (1, 8, 8, 3), (3, 6, 4, 2), (1, 6, 9, 2)):
        N, H, W, C = img
        x = _randn(rs, img)
        for pad, st, win in ((0, (1, 1), (2, 2)), (1, (2, 2), (3, 3)), (2, (1, 2), (4, 4)), (0, (2, 1), (2, 1)),
                             (1, (1, 1), (1, 2)), (2, (2, 2), (2, 2))):
            oh, ow = out_hw(H, W, win[0], win[1], pad, st)
            if oh <= 0 or ow <= 0:
                continue
            tag = 'w%dx%d-p%d-s%dx%d' % (win[0], win[1], pad, st[0], st[1])
            oshape = (N, oh, ow, C)
            add(Case('maxpool2d_forward_batch', [('x', x), ('out', np.zeros(oshape, F32)), ('argmax', np.zeros(oshape, F32))],
                     ['x', win, 'out', pad, st, 'argmax'], tag=tag))
            add(Case('avgpool2d_forward_batch', [('x', x), ('out', np.zeros(oshape, F32))],
                     ['x', win, 'out', pad, st], tag=tag))
            # backward cases: outputs / argmax of the forward pass are filled in by
            # finalize_derivs() (reference when generating, stored values when checking)
            add(Case('maxpool2d_backward_batch',
                     [('x', x), ('out', np.zeros(oshape, F32)), ('argmax', np.zeros(oshape, F32)),
                      ('in_deltas', _randn(rs, img)), ('out_deltas', _randn(rs, oshape))],
                     ['x', win, 'out', pad, st, 'argmax', 'in_deltas', 'out_deltas'], tag=tag))
            add(Case('avgpool2d_backward_batch',
                     [('x', x), ('out', np.zeros(oshape, F32)), ('in_deltas', _randn(rs, img)),
                      ('out_deltas', _randn(rs, oshape))],
                     ['x', win, 'out', pad, st, 'in_deltas', 'out_deltas'], tag=tag))
    return cases


def finalize_derivs(cases, handler_factory, wrap=lambda h, x: x,
                    unwrap=lambda h, x: x):
    """Fill ``y = f(x)`` of every ``*_deriv`` case using ``handler_factory()``
    (the reference handler when generating, the oracle when checking)."""
    h = handler_factory()
    for c in cases:
        if c.op.endswith('_deriv'):
            act = c.op[:-6]
            y = np.zeros_like(c.arrays['x'])
            getattr(h, act)(c.arrays['x'].copy(), y)
            c.arrays['y'] = y
        elif c.op == 'maxpool2d_backward_batch':
            x, win, _, pad, st = [c.arrays[a] if isinstance(a, str) else a for a in c.call[:5]]
            out, am = np.zeros_like(c.arrays['out']), np.zeros_like(c.arrays['argmax'])
            h.maxpool2d_forward_batch(x.copy(), win, out, pad, st, am)
            c.arrays['out'], c.arrays['argmax'] = out, am
    return cases


def inputs_digest(cases):
    """A checksum over every input array, stored beside the golden outputs to
    detect a drift of the generators."""
    import hashlib
    hsh = hashlib.sha256()
    for c in cases:
        for k, v in c.arrays.items():
            if (k == 'y' and c.op.endswith('_deriv')) or \
                    (k in ('out', 'argmax') and c.op == 'maxpool2d_backward_batch'):
                continue
            hsh.update(np.ascontiguousarray(v).tobytes())
    return hsh.hexdigest()
