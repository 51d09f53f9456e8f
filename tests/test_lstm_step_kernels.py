"""The LSTM sequence entry points at sizes that exercise every form of the
per-timestep kernels (split-K and single-pass recurrent GEMMs, ragged tiles in both
directions, every activation) against the numpy oracle."""
import numpy as np
import pytest

import parity  # noqa: F401
from oracle import numpy_oracle as no

pytestmark = pytest.mark.gpu

ACTS = {'sigmoid': 0, 'tanh': 1, 'rel': 2, 'el': 3, 'linear': 4}


def _problem(T, B, H, n_in, seed):
    rs = np.random.RandomState(seed)
    p = {}
    for g in 'zifo':
        p['W' + g] = rs.uniform(-0.3, 0.3, (H, n_in)).astype(np.float32)
        p['R' + g] = rs.uniform(-2.0 / np.sqrt(H), 2.0 / np.sqrt(H), (H, H)).astype(np.float32)
        p['b' + g] = rs.uniform(-0.5, 0.5, (H,)).astype(np.float32)
    for g in 'ifo':
        p['p' + g] = rs.uniform(-0.5, 0.5, (1, H)).astype(np.float32)
    x = rs.randn(T, B, n_in).astype(np.float32)
    deltas = (rs.randn(T + 1, B, H) * 0.1).astype(np.float32)
    deltas[T] = 0
    return p, x, deltas


def _close(got, want, scale, what):
    """Element by element: |got - want| <= 1e-5 |want| + 1e-5 * (sum of |terms| of that element)."""
    parity.assert_reduction_close(got, want, scale, 'lstm', what)


@pytest.mark.parametrize('T,B,H,act', [
    (3, 128, 1000, 'tanh'),     # the benchmark's layer: split-K, last column tile ragged
    (3, 200, 512, 'tanh'),      # two row tiles, the second ragged
    (2, 5, 256, 'sigmoid'),
    (3, 64, 100, 'tanh'),       # K not a multiple of 32
    (2, 130, 36, 'rel'),        # a row tile with two rows
    (2, 33, 288, 'el'),
    (2, 16, 50, 'linear'),      # pitch not a multiple of 4 floats: operands staged
])
def test_sequence_passes_match_the_oracle(T, B, H, act):
    from brainstorm_b200 import B200Handler
    from brainstorm_b200._lib import lib, check
    n_in = 24
    p, x, deltas = _problem(T, B, H, n_in, seed=H + B)
    O = no.OracleHandler(np.float32)
    f_ref = {k: np.zeros((T + 1, B, H), np.float32) for k in no.LSTM_FORWARD + ('y',)}
    no.lstm_forward(O, p, x, f_ref, activation=act)
    d_ref = {k: np.zeros((T + 1, B, H), np.float32) for k in no.LSTM_BACKWARD}
    grads = {k: np.zeros_like(v) for k, v in p.items()}
    dx = np.zeros_like(x)
    no.lstm_backward(O, p, x, f_ref, deltas, d_ref, grads, dx, activation=act)

    Hd = B200Handler(seed=1)
    up = Hd.create_from_numpy
    Wst = up(np.concatenate([p['Wz'], p['Wi'], p['Wf'], p['Wo']], axis=0))
    Rst = up(np.concatenate([p['Rz'], p['Ri'], p['Rf'], p['Ro']], axis=0))
    bst = up(np.concatenate([p['bz'], p['bi'], p['bf'], p['bo']]))
    pst = up(np.concatenate([p['pi'].ravel(), p['pf'].ravel(), p['po'].ravel()]))
    xproj = Hd.zeros((T * B, 4 * H))
    Hd.dot_mm(up(x.reshape(T * B, n_in)), Wst, xproj, transb=True)
    f = {k: Hd.zeros((T + 1, B, H)) for k in f_ref}
    y_work, r_work = Hd.zeros((T + 1, B, H)), Hd.zeros((B, 4 * H))
    d = {k: Hd.zeros((T + 1, B, H)) for k in d_ref}
    dG = Hd.zeros((T + 1, B, 4 * H))
    order = ('dZa', 'dZb', 'dIa', 'dIb', 'dFa', 'dFb', 'dOa', 'dOb', 'dCa', 'dCb')
    check(lib.b200_lstm_forward(xproj.ptr, Rst.ptr, bst.ptr, pst.ptr, *[f[k].ptr for k in no.LSTM_FORWARD],
                                f['y'].ptr, y_work.ptr, r_work.ptr, T, B, H, ACTS[act]))
    deltas_dev = up(deltas)     # keep alive: the call only takes its address
    check(lib.b200_lstm_backward(deltas_dev.ptr, Rst.ptr, pst.ptr, f['Zb'].ptr, f['Ib'].ptr, f['Fb'].ptr,
                                 f['Ob'].ptr, f['Ca'].ptr, f['Cb'].ptr, *[d[k].ptr for k in order],
                                 dG.ptr, r_work.ptr, T, B, H, ACTS[act]))
    Hd.synchronize()
    internals = {k: v[:T] for k, v in list(f_ref.items()) + list(d_ref.items()) if k != 'y'}
    S = parity.lstm_term_scales(p, x, f_ref['y'][:T], internals, deltas[:T])
    for k in f:
        _close(Hd.get_numpy_copy(f[k])[:T], f_ref[k][:T], S[k], k)
    assert np.array_equal(Hd.get_numpy_copy(y_work)[:T], Hd.get_numpy_copy(f['y'])[:T])
    for k in d:
        _close(Hd.get_numpy_copy(d[k])[:T], d_ref[k][:T], S[k], k)
    stacked = np.concatenate([d_ref[k][:T] for k in ('dZa', 'dIa', 'dFa', 'dOa')], axis=2)
    _close(Hd.get_numpy_copy(dG)[:T], stacked, np.concatenate([S['dZa']] * 4, axis=2), 'stacked gate deltas')
