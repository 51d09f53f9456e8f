"""The LSTM sequence passes against stored results of the reference's own
LstmLayerImpl: the oracle must reproduce them bit for bit (CPU), and the fused
library entry points must match them through the C-ABI (GPU) -- without the
reference being importable."""
import os

import numpy as np
import pytest

import parity  # noqa: F401
from oracle import numpy_oracle as no

G = np.load(os.path.join(os.path.dirname(__file__), 'golden', 'lstm_layer.npz'))


def _case(tag):
    get = lambda kind, name: G['%s/%s/%s' % (tag, kind, name)]
    p = {n: get('parameters', n) for n in no.LSTM_PARAMS}
    x = get('inputs', 'default')
    f_ref = {n: get('internals', n) for n in no.LSTM_FORWARD}
    f_ref['y'] = get('outputs', 'default')
    d_ref = {n: get('internals', n) for n in no.LSTM_BACKWARD}
    g_ref = {n: get('gradients', n) for n in no.LSTM_PARAMS}
    return p, x, f_ref, d_ref, g_ref, get('output_deltas', 'default'), get('input_deltas', 'default')


@pytest.mark.parametrize('tag', ['a', 'b'])
def test_oracle_lstm_reproduces_reference_layer_bits(tag):
    p, x, f_ref, d_ref, g_ref, deltas, dx_ref = _case(tag)
    O = no.OracleHandler(np.float32)
    f = {k: np.zeros_like(v) for k, v in f_ref.items()}
    no.lstm_forward(O, p, x, f)
    T = x.shape[0]
    for k in f:
        assert np.array_equal(f[k][:T], f_ref[k][:T]), k
    d = {k: np.zeros_like(v) for k, v in d_ref.items()}
    grads = {k: np.zeros_like(v) for k, v in g_ref.items()}
    dx = np.zeros_like(dx_ref)
    no.lstm_backward(O, p, x, f, deltas, d, grads, dx)
    for k in d:
        assert np.array_equal(d[k][:T], d_ref[k][:T]), k
    for k in grads:
        assert np.array_equal(grads[k], g_ref[k]), k
    # the first LSTM layer's input deltas go to the Input layer: the reference adds
    # into a buffer that other consumers may share, here there are none
    assert np.array_equal(dx, dx_ref)


@pytest.mark.gpu
@pytest.mark.parametrize('tag', ['a', 'b'])
def test_fused_lstm_entry_points_match_reference_layer(tag):
    from brainstorm_b200 import B200Handler
    from brainstorm_b200._lib import lib, check
    p, x, f_ref, d_ref, g_ref, deltas, dx_ref = _case(tag)
    H_ = B200Handler(seed=1)
    T, B, n_in = x.shape
    Hs = f_ref['y'].shape[2]
    up = H_.create_from_numpy
    Wst = up(np.concatenate([p['Wz'], p['Wi'], p['Wf'], p['Wo']], axis=0))
    Rst = up(np.concatenate([p['Rz'], p['Ri'], p['Rf'], p['Ro']], axis=0))
    bst = up(np.concatenate([p['bz'], p['bi'], p['bf'], p['bo']]))
    pst = up(np.concatenate([p['pi'].ravel(), p['pf'].ravel(), p['po'].ravel()]))
    dx_flat = up(x.reshape(T * B, n_in))
    xproj = H_.zeros((T * B, 4 * Hs))
    H_.dot_mm(dx_flat, Wst, xproj, transb=True)
    f = {k: H_.zeros((T + 1, B, Hs)) for k in f_ref}
    y_work, r_work = H_.zeros((T + 1, B, Hs)), H_.zeros((B, 4 * Hs))
    check(lib.b200_lstm_forward(xproj.ptr, Rst.ptr, bst.ptr, pst.ptr, *[f[k].ptr for k in no.LSTM_FORWARD],
                                f['y'].ptr, y_work.ptr, r_work.ptr, T, B, Hs, 1))

    internals = {k: v[:T] for k, v in list(f_ref.items()) + list(d_ref.items()) if k != 'y'}
    S = parity.lstm_term_scales(p, x, f_ref['y'][:T], internals, deltas[:T])

    def close(got, want, scale, what):      # element by element, scale = sum of |terms| of that element
        parity.assert_reduction_close(got, want, scale, 'lstm', what)

    for k in f:
        close(H_.get_numpy_copy(f[k])[:T], f_ref[k][:T], S[k], k)
    d = {k: H_.zeros((T + 1, B, Hs)) for k in d_ref}
    dG = H_.zeros((T + 1, B, 4 * Hs))
    order = ('dZa', 'dZb', 'dIa', 'dIb', 'dFa', 'dFb', 'dOa', 'dOb', 'dCa', 'dCb')
    deltas_dev = up(deltas)     # keep alive: the call only takes its address
    check(lib.b200_lstm_backward(deltas_dev.ptr, Rst.ptr, pst.ptr, f['Zb'].ptr, f['Ib'].ptr, f['Fb'].ptr,
                                 f['Ob'].ptr, f['Ca'].ptr, f['Cb'].ptr, *[d[k].ptr for k in order],
                                 dG.ptr, r_work.ptr, T, B, Hs, 1))
    for k in d:
        close(H_.get_numpy_copy(d[k])[:T], d_ref[k][:T], S[k], k)
    stacked = np.concatenate([d_ref[k][:T] for k in ('dZa', 'dIa', 'dFa', 'dOa')], axis=2)
    close(H_.get_numpy_copy(dG)[:T], stacked, np.concatenate([S['dZa']] * 4, axis=2), 'stacked gate deltas')
    # weight gradients from the stacked deltas, as the fused layer computes them
    dW = H_.zeros((4 * Hs, n_in))
    H_.dot_add_mm(dG[:T].reshape((T * B, 4 * Hs)), dx_flat, dW, transa=True)
    close(H_.get_numpy_copy(dW), np.concatenate([g_ref['Wz'], g_ref['Wi'], g_ref['Wf'], g_ref['Wo']], axis=0),
          np.concatenate([S['grad.W' + g] for g in 'zifo'], axis=0), 'dW')
