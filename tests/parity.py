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
        return 0.0          # every term of the denominator is positive: a pure relative bound
    if op.startswith(('conv2d', 'avgpool2d', 'maxpool2d')):
        # sums of a few dozen terms of order one: one scale for all outputs
        return float(max(np.abs(v).max() for v in arrays.values() if v.size) *
                     max(np.prod(arrays['w'].shape[1:]) if 'w' in arrays else 16, 16))
    raise KeyError(op)


REDUCTION_OPS = {'sum_t', 'dot_mm', 'dot_add_mm', 'softmax_m', 'conv2d_forward_batch', 'conv2d_backward_batch',
                 'avgpool2d_forward_batch', 'avgpool2d_backward_batch', 'maxpool2d_backward_batch'}


def lstm_term_scales(params, x, y, internals, out_deltas, y_context=None, ca_context=None, out_delta_scale=None):
    """Per-element error scales of every buffer the LSTM layer fills
    (brainstorm/layers/lstm_layer.py:106-278), from one CPU run's own values.

    A buffer element that is a sum gets the sum of the absolute values of its terms; an
    element that is a product or a slope-<=1 function of such sums gets the scale of the
    sum times the other factor.  Scales follow the data flow by one level: the gate deltas
    enter the gradient and input-delta contractions with their own scale added to their
    magnitude, and ``out_delta_scale`` (default: |out_deltas|) is the scale the layer above
    attached to the output deltas it produced.  All arrays cover the T time steps of the
    pass (context slot stripped); ``params`` maps the fifteen parameter names to arrays.
    Returns {buffer name: scale array}, with 'y', 'dx' and 'grad.<name>' beside the internals."""
    A = lambda v: np.abs(np.asarray(v, dtype=np.float32))
    P = {k: A(v) for k, v in params.items()}
    T, B, H = y.shape
    x2 = A(x).reshape(T * B, -1)
    ya = A(y)
    y0 = np.zeros_like(ya[:1]) if y_context is None else A(y_context).reshape(1, B, H)
    y_prev = np.concatenate([y0, ya[:-1]]).reshape(T * B, H)
    I = {k: A(v) for k, v in internals.items()}
    ca = I['Ca']
    c0 = np.zeros_like(ca[:1]) if ca_context is None else A(ca_context).reshape(1, B, H)
    ca_prev = np.concatenate([c0, ca[:-1]])
    pi, pf, po = (P[k].reshape(1, 1, H) for k in ('pi', 'pf', 'po'))
    S = {}
    # forward (:117-145): the four pre-activations, then the cell and the output
    pre = {g: (x2 @ P['W' + g].T + y_prev @ P['R' + g].T).reshape(T, B, H) + P['b' + g].reshape(1, 1, H)
           for g in 'zifo'}
    pre['i'] = pre['i'] + ca_prev * pi
    pre['f'] = pre['f'] + ca_prev * pf
    pre['o'] = pre['o'] + ca * po
    for g in 'zifo':
        S[g.upper() + 'a'] = S[g.upper() + 'b'] = pre[g]
    S['Ca'] = S['Cb'] = I['Ib'] * I['Zb'] + I['Fb'] * ca_prev + pre['z'] + pre['i'] + pre['f'] * ca_prev
    S['y'] = S['Ca'] + pre['o']
    # backward (:171-205): dy = output deltas + sum over gates of dG[t+1].R; the cell delta adds five terms
    nxt = lambda a: np.concatenate([a[1:], np.zeros_like(a[:1])])
    dG = {g: I['d%sa' % g.upper()] for g in 'zifo'}
    s_out = A(out_deltas) if out_delta_scale is None else np.maximum(A(out_deltas), A(out_delta_scale))
    s_dy = s_out + sum(nxt(dG[g]).reshape(T * B, H) @ P['R' + g] for g in 'zifo').reshape(T, B, H)
    s_dca = nxt(dG['i']) * pi + nxt(dG['f']) * pf + dG['o'] * po + I['dCb'] + nxt(I['dCa']) * nxt(I['Fb'])
    s_bwd = (s_dy * (1 + ca) + s_dca) * (1 + ca_prev)
    for k in ('dZa', 'dZb', 'dIa', 'dIb', 'dFa', 'dFb', 'dOa', 'dOb', 'dCa', 'dCb'):
        S[k] = s_bwd
    # input deltas (:216-219) and gradients (:221-278)
    dGf = {g: (dG[g] + s_bwd).reshape(T * B, H) for g in 'zifo'}     # magnitude plus own scale
    S['dx'] = sum(dGf[g] @ P['W' + g] for g in 'zifo').reshape(np.shape(x))
    for g in 'zifo':
        S['grad.W' + g] = dGf[g].T @ x2
        S['grad.R' + g] = dGf[g].T @ y_prev
        S['grad.b' + g] = dGf[g].sum(0)
    extra = (ca[-1:] * (dG['i'] + s_bwd)[:1]).sum((0, 1))        # the term of :272-278
    for name, g, c in (('pi', 'i', ca_prev), ('pf', 'f', ca_prev), ('po', 'o', ca)):
        S['grad.' + name] = ((c * (dG[g] + s_bwd)).sum((0, 1)) + extra).reshape(1, H)
    return S


# ---- network-level comparisons ------------------------------------------------------------
# Every compared element must satisfy |gpu - cpu| <= RTOL * |cpu| + RTOL * scale, where scale
# is the sum of the absolute values of the terms that were added up to give that element
# (for values that are products or bounded-slope functions of such sums, the scale of the
# sum times the factor), computed from the CPU run's own buffers.  Neither side is exact:
# NumpyHandler's float32 BLAS and the GPU's split-TF32 tensor-core GEMM round differently,
# and what one rounding can move is proportional to that scale.
def absf(x):
    return np.abs(np.asarray(x, dtype=np.float32))


def bounded(got, want, scale, what, worst, rtol=REDUCTION_RTOL):
    """Records the worst err/bound ratio of one buffer in worst[what] (judged by report)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = np.abs(got - want)
    bound = rtol * np.abs(want) + rtol * np.broadcast_to(np.asarray(scale, np.float64), want.shape) + 1e-37
    worst[what] = float((err / bound).max()) if err.size else 0.0


def report(worst, title):
    """All buffers are measured first, then judged together, so that one run shows every
    buffer that leaves its bound and the observed worst ratio of each."""
    order = sorted(worst, key=worst.get, reverse=True)
    print('%s: worst err/bound %.3g at %s; next: %s' % (
        title, worst[order[0]], order[0], ', '.join('%s %.2g' % (k, worst[k]) for k in order[1:6])))
    bad = [k for k in order if not worst[k] <= 1.0]
    assert not bad, '%s: outside the bound: %s' % (title, ', '.join('%s %.3g' % (k, worst[k]) for k in bad))


def fc_layer_checks(net_cpu, net_gpu, name, worst, out_delta_scale=None, in_scale=None):
    """A FullyConnected layer (brainstorm/layers/fully_connected_layer.py:52-78): outputs
    against the sum of |terms| of x.W^T + bias (the activations have slope <= 1), weight and
    bias gradients against the sums of |terms| of their contractions over the batch, in
    which the deltas and the inputs enter with the scale their producer attached to them
    (``out_delta_scale``, ``in_scale``) where that exceeds their magnitude.
    Returns (scale of the outputs, this layer's share of the scale of its input deltas)."""
    get = lambda net, path: net.get('%s.%s' % (name, path))
    xin = get(net_cpu, 'inputs.default')
    x = absf(xin).reshape(-1, xin.shape[-1])
    W, b = absf(get(net_cpu, 'parameters.W')), absf(get(net_cpu, 'parameters.bias'))
    out = get(net_cpu, 'outputs.default')
    s_out = (x @ W.T + b).reshape(out.shape)
    bounded(get(net_gpu, 'outputs.default'), out, s_out, name + '.outputs', worst)
    dH = absf(get(net_cpu, 'output_deltas.default')).reshape(-1, W.shape[0])   # overwritten with dout * f'(y) (:73)
    if out_delta_scale is not None:
        dH = np.maximum(dH, absf(out_delta_scale).reshape(dH.shape))
    xg = x if in_scale is None else np.maximum(x, absf(in_scale).reshape(x.shape))
    bounded(get(net_gpu, 'gradients.W'), get(net_cpu, 'gradients.W'), dH.T @ xg, name + '.gradients.W', worst)
    bounded(get(net_gpu, 'gradients.bias'), get(net_cpu, 'gradients.bias'), dH.sum(0), name + '.gradients.bias', worst)
    return s_out, dH @ W


def lstm_net_checks(net_cpu, net_gpu, T, worst):
    """A stack of LSTM layers under an output projection (the 'classification' networks of
    brainstorm.tools.create_net_from_spec), after one forward/backward pass on both sides:
    all twenty internals, outputs, input deltas and gradients of every LSTM layer, element
    by element, with the scales of lstm_term_scales."""
    # scale of the deltas the output projection hands down: |dH| . |W|
    dH = absf(net_cpu.get('Output_projection.output_deltas.default'))
    above = dH.reshape(-1, dH.shape[-1]) @ absf(net_cpu.get('Output_projection.parameters.W'))
    top_scale = None
    for lname in [n for n in net_cpu.layers if n.startswith('Lstm')][::-1]:
        cut = lambda v: v[:T] if v.ndim == 3 and v.shape[0] == T + 1 else v
        get = lambda net, path: cut(net.get('%s.%s' % (lname, path)))
        names = {kind: list(net_cpu.buffer[lname][kind].keys()) for kind in ('parameters', 'internals')}
        y = get(net_cpu, 'outputs.default')
        S = lstm_term_scales({k: get(net_cpu, 'parameters.' + k) for k in names['parameters']},
                             get(net_cpu, 'inputs.default'), y,
                             {k: get(net_cpu, 'internals.' + k) for k in names['internals']},
                             get(net_cpu, 'output_deltas.default'), out_delta_scale=above.reshape(y.shape))
        above = S['dx']
        if top_scale is None:
            top_scale = S['y']
        for k in names['internals']:
            bounded(get(net_gpu, 'internals.' + k), get(net_cpu, 'internals.' + k), S[k], '%s.%s' % (lname, k), worst)
        bounded(get(net_gpu, 'outputs.default'), y, S['y'], lname + '.outputs', worst)
        bounded(get(net_gpu, 'input_deltas.default'), get(net_cpu, 'input_deltas.default'), S['dx'],
                lname + '.input_deltas', worst)
        for k in names['parameters']:
            want = get(net_cpu, 'gradients.' + k)
            bounded(get(net_gpu, 'gradients.' + k), want, S['grad.' + k].reshape(want.shape),
                    '%s.gradients.%s' % (lname, k), worst)
    fc_layer_checks(net_cpu, net_gpu, 'Output_projection', worst, in_scale=top_scale)
