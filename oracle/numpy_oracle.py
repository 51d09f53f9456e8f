"""CPU oracle for the Handler hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

A numpy restatement of what the reference's CPU backend
(``brainstorm/handlers/numpy_handler.py``, class ``NumpyHandler``) computes for
every operation of the ``Handler`` API (``brainstorm/handlers/base_handler.py``)
that the B200 backend implements, plus the per-timestep LSTM gate arithmetic of
``brainstorm/layers/lstm_layer.py``.  Only the tests, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it; the
product package never does.

Parity pin: ``tests/golden/*.npz`` were produced by running the *real*
``NumpyHandler`` (and the real ``LstmLayerImpl`` on it) on seeded inputs
(``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` requires this
module to reproduce every stored output bit for bit.

Conventions follow the reference: every op writes into a pre-allocated ``out``
and returns ``None``; ``out`` may alias an input; shapes are not checked.
"""
from __future__ import annotations

import numpy as np


class OracleHandler(object):
    """Same method names, argument order and semantics as ``NumpyHandler``."""

    array_type = np.ndarray

    def __init__(self, dtype=np.float32, seed=None):
        self.dtype = np.dtype(dtype).type
        self.rnd = np.random.RandomState(seed)

    # ---- allocation / transfer: numpy_handler.py:36-65 -------------------
    def allocate(self, shape):
        # numpy_handler.py:36 -- zero-filled, although the API says "arbitrary"
        return np.zeros(shape, dtype=self.dtype)

    def zeros(self, shape):                         # numpy_handler.py:42
        return np.zeros(shape, dtype=self.dtype)

    def ones(self, shape):                          # numpy_handler.py:39
        return np.ones(shape, dtype=self.dtype)

    def create_from_numpy(self, arr):               # numpy_handler.py:54
        return np.array(arr, dtype=self.dtype)

    def set_from_numpy(self, mem, arr):             # numpy_handler.py:64
        mem[...] = np.asarray(arr).astype(self.dtype)

    def get_numpy_copy(self, mem):                  # numpy_handler.py:60
        return np.array(mem, copy=True)

    def fill(self, mem, val):                       # numpy_handler.py:57
        mem[...] = val

    def copy_to(self, src, dest):                   # numpy_handler.py:47 (src, dest)
        np.copyto(dest, src, casting='same_kind')

    def is_fully_finite(self, a):                   # numpy_handler.py:69
        return bool(np.isfinite(a).all())

    # ---- tensor (.) tensor: numpy_handler.py:86,264,245,190,233 ----------
    def add_tt(self, a, b, out):
        np.add(a, b, out=out)

    def subtract_tt(self, a, b, out):
        np.subtract(a, b, out=out)

    def mult_tt(self, a, b, out):
        np.multiply(a, b, out=out)

    def divide_tt(self, a, b, out):
        np.divide(a, b, out=out)

    def mult_add_tt(self, a, b, out):
        # numpy_handler.py:233 -- product rounded, then sum rounded (no FMA)
        prod = np.multiply(a, b)
        np.add(out, prod, out=out)

    def modulo_tt(self, a, b, out):                 # numpy_handler.py:227
        np.fmod(a, b, out=out)

    # ---- matrix (.) broadcast vector: numpy_handler.py:80,261,236,187,239 -
    def add_mv(self, m, v, out):
        np.add(m, v, out=out)

    def subtract_mv(self, m, v, out):
        np.subtract(m, v, out=out)

    def mult_mv(self, m, v, out):
        np.multiply(m, v, out=out)

    def divide_mv(self, m, v, out):
        np.divide(m, v, out=out)

    def mult_add_mv(self, m, v, out):
        prod = np.multiply(m, v)
        np.add(out, prod, out=out)

    def broadcast_t(self, a, axis, out):            # numpy_handler.py:103
        out[...] = a

    # ---- scalar (.) tensor: numpy_handler.py:83,242,230 ------------------
    def add_st(self, s, t, out):
        np.add(t, s, out=out)

    def mult_st(self, s, t, out):
        np.multiply(s, t, out=out)

    def mult_add_st(self, s, t, out):
        prod = np.multiply(s, t)
        np.add(out, prod, out=out)

    # ---- unary: numpy_handler.py:74,248,258,207,107 ----------------------
    def abs_t(self, a, out):
        np.absolute(a, out=out)

    def sign_t(self, a, out):
        np.sign(a, out=out)

    def sqrt_t(self, a, out):
        np.sqrt(a, out=out)

    def log_t(self, a, out):
        np.log(a, out=out)

    def clip_t(self, a, a_min, a_max, out):
        np.clip(a, a_min, a_max, out=out)

    # ---- predicated ops: numpy_handler.py:173,196,77 ---------------------
    def copy_to_if(self, src, dest, cond):
        sel = cond != 0
        dest[sel] = src[sel]

    def fill_if(self, mem, val, cond):
        mem[cond != 0] = val

    def add_into_if(self, a, out, cond):
        sel = cond != 0
        out[sel] += a[sel]

    # ---- concat / split on the last axis: numpy_handler.py:221,251 -------
    def merge_tt(self, a, b, out):
        na = a.shape[-1]
        o2 = out.reshape(-1, out.shape[-1])
        o2[:, :na] = a.reshape(-1, na)
        o2[:, na:] = b.reshape(-1, b.shape[-1])

    def split_add_tt(self, x, out_a, out_b):
        na = out_a.shape[-1]
        x2 = x.reshape(-1, x.shape[-1])
        oa = out_a.reshape(-1, na)
        ob = out_b.reshape(-1, out_b.shape[-1])
        oa += x2[:, :na]
        ob += x2[:, na:]

    # ---- reductions: numpy_handler.py:268,292 ----------------------------
    def sum_t(self, a, axis, out):
        keep = axis is not None and out.ndim == a.ndim
        np.sum(a, axis=axis, out=out, keepdims=keep)

    def softmax_m(self, m, out):
        shifted = m - np.amax(m, axis=1, keepdims=True)
        e = np.exp(shifted)
        np.divide(e, np.sum(e, axis=1, keepdims=True), out=out)

    # ---- label ops (bit-exact): numpy_handler.py:99,202 ------------------
    def binarize_v(self, v, out):
        labels = v.astype(np.int32).reshape(-1)
        out[...] = 0
        out[np.arange(out.shape[0]), labels] = 1

    def index_m_by_v(self, m, v, out):
        labels = v.astype(np.int32).reshape(-1)
        out[:, 0] = m[np.arange(m.shape[0]), labels]

    # ---- GEMM: numpy_handler.py:176,181 ----------------------------------
    def dot_mm(self, a, b, out, transa=False, transb=False):
        out[...] = np.dot(a.T if transa else a, b.T if transb else b)

    def dot_add_mm(self, a, b, out, transa=False, transb=False):
        out[...] += np.dot(a.T if transa else a, b.T if transb else b)

    # ---- random: numpy_handler.py:193,199 (MT19937 RandomState) ----------
    def fill_gaussian(self, mean, std, out):
        out[...] = std * self.rnd.standard_normal(out.shape) + mean

    def generate_probability_mask(self, mask, probability):
        mask[...] = self.rnd.uniform(size=mask.shape) < probability

    # ---- activations: numpy_handler.py:277-309 ---------------------------
    def sigmoid(self, x, y):
        # numpy_handler.py:283 uses two boolean-mask passes: 1/(1+exp(-x)) for
        # x >= 0 and exp(x)/(1+exp(x)) for x < 0.  exp(-|x|) equals exp(-x) on
        # the first branch and exp(x) on the second, so one pass gives the same
        # bits without overflow (and without the mask indexing cost).
        e = np.exp(-np.abs(x))
        one = self.dtype(1)
        y[...] = np.where(x >= 0, one / (one + e), e / (one + e))

    def sigmoid_deriv(self, x, y, dy, dx):
        dx[...] = dy * y * (self.dtype(1) - y)

    def tanh(self, x, y):
        np.tanh(x, out=y)

    def tanh_deriv(self, x, y, dy, dx):
        dx[...] = dy * (self.dtype(1) - y * y)

    def rel(self, x, y):
        # x * (x > 0): negatives become -0.0, NaN stays NaN
        y[...] = x * (x > 0)

    def rel_deriv(self, x, y, dy, dx):
        dx[...] = dy * (y > 0)

    def el(self, x, y):
        # note >= at zero and exp(x) - 1 (not expm1), as numpy_handler.py:305
        y[...] = x * (x >= 0) + (np.exp(x) - self.dtype(1)) * (x < 0)

    def el_deriv(self, x, y, dy, dx):
        dx[...] = dy * (y >= 0) + dy * (y + self.dtype(1)) * (y < 0)

    def act(self, name, x, y):
        """Dispatch like ``Handler.act_func`` (base_handler.py:57-63)."""
        if name == 'linear':
            self.copy_to(x, y)
        else:
            getattr(self, name)(x, y)

    def act_deriv(self, name, x, y, dy, dx):
        """Dispatch like ``Handler.act_func_deriv`` (base_handler.py:65-72)."""
        if name == 'linear':
            self.copy_to(dy, dx)
        else:
            getattr(self, name + '_deriv')(x, y, dy, dx)

    # ---- fused LSTM timestep, restated from lstm_layer.py ----------------
    def lstm_step_forward(self, Za, Ia, Fa, Oa, Ca_prev, bz, bi, bf, bo,
                          pi, pf, po, Zb, Ib, Fb, Ob, Ca, Cb, y,
                          activation='tanh'):
        """Gate math of one timestep, lstm_layer.py:117-145 minus the four
        recurrent GEMMs, which must already have been accumulated into the
        pre-activations ``Za, Ia, Fa, Oa``.  All arrays are (B, H); biases and
        peepholes are (1, H) or (H,).  Updates the pre-activations in place as
        the reference does and writes ``Zb, Ib, Fb, Ob, Ca, Cb, y``."""
        r = lambda p: p.reshape(1, -1)
        self.add_mv(Za, r(bz), Za)                      # :118
        self.act(activation, Za, Zb)                    # :119
        self.mult_add_mv(Ca_prev, r(pi), Ia)            # :123
        self.add_mv(Ia, r(bi), Ia)                      # :124
        self.sigmoid(Ia, Ib)                            # :125
        self.mult_add_mv(Ca_prev, r(pf), Fa)            # :129
        self.add_mv(Fa, r(bf), Fa)                      # :130
        self.sigmoid(Fa, Fb)                            # :131
        self.mult_tt(Ib, Zb, Ca)                        # :134
        self.mult_add_tt(Fb, Ca_prev, Ca)               # :135
        self.mult_add_mv(Ca, r(po), Oa)                 # :139
        self.add_mv(Oa, r(bo), Oa)                      # :140
        self.sigmoid(Oa, Ob)                            # :141
        self.act(activation, Ca, Cb)                    # :144
        self.mult_tt(Ob, Cb, y)                         # :145

    def lstm_step_backward(self, dy, dIa_next, dFa_next, dCa_next, Fb_next,
                           pi, pf, po, Za, Zb, Ia, Ib, Fa, Fb, Oa, Ob, Ca, Cb,
                           Ca_prev, dZa, dZb, dIa, dIb, dFa, dFb, dOa, dOb,
                           dCa, dCb, activation='tanh'):
        """Gate math of one backward timestep, lstm_layer.py:179-205.  ``dy``
        already holds the output deltas plus the four recurrent GEMM
        contributions (:173-177).  ``dCa`` is accumulated into (it starts at
        zero, :168); everything else is overwritten."""
        r = lambda p: p.reshape(1, -1)
        self.mult_add_mv(dIa_next, r(pi), dCa)          # :180
        self.mult_add_mv(dFa_next, r(pf), dCa)          # :181
        self.mult_tt(dy, Cb, dOb)                       # :184
        self.sigmoid_deriv(Oa, Ob, dOb, dOa)            # :185
        self.mult_add_mv(dOa, r(po), dCa)               # :187
        self.mult_tt(dy, Ob, dCb)                       # :190
        self.act_deriv(activation, Ca, Cb, dCb, dCb)    # :191
        self.add_tt(dCa, dCb, dCa)                      # :192
        self.mult_add_tt(dCa_next, Fb_next, dCa)        # :193
        self.mult_tt(dCa, Ca_prev, dFb)                 # :196
        self.sigmoid_deriv(Fa, Fb, dFb, dFa)            # :197
        self.mult_tt(dCa, Zb, dIb)                      # :200
        self.sigmoid_deriv(Ia, Ib, dIb, dIa)            # :201
        self.mult_tt(dCa, Ib, dZb)                      # :204
        self.act_deriv(activation, Za, Zb, dZb, dZa)    # :205


# --------------------------------------------------------------------------
# Seeded synthetic inputs of the benchmark configurations (shared by the
# parity tests and the CPU-baseline leg of the benchmark so that both sides see
# the same data).
# --------------------------------------------------------------------------
def op_suite_inputs(rows, cols, seed):
    """Inputs of the handler op suite (the workload's own seeded generator; the
    checker and the checked side must see the same arrays)."""
    from brainstorm_b200.workloads import op_suite_inputs as make
    return make(rows, cols, seed)


# --------------------------------------------------------------------------
# Whole-sequence LSTM passes, restated from lstm_layer.py with the oracle's ops
# in the reference's own order (so the results are bit-identical to running
# LstmLayerImpl on NumpyHandler).  `p` holds the fifteen parameters by name,
# `f` the ten forward internals + 'y' as (T+1, B, H) arrays (context in slot T).
# --------------------------------------------------------------------------
LSTM_PARAMS = ('Wz', 'Wi', 'Wf', 'Wo', 'pi', 'pf', 'po', 'Rz', 'Ri', 'Rf', 'Ro', 'bz', 'bi', 'bf', 'bo')
LSTM_FORWARD = ('Za', 'Zb', 'Ia', 'Ib', 'Fa', 'Fb', 'Oa', 'Ob', 'Ca', 'Cb')
LSTM_BACKWARD = ('dZa', 'dZb', 'dIa', 'dIb', 'dFa', 'dFb', 'dOa', 'dOb', 'dCa', 'dCb')


def lstm_forward(O, p, x, f, activation='tanh'):
    """lstm_layer.py:90-145."""
    T, B = x.shape[0], x.shape[1]
    flat_x = x.reshape(T * B, -1)
    for g in 'zifo':                                     # :110-113
        O.dot_mm(flat_x, p['W' + g], f[g.upper() + 'a'][:T].reshape(T * B, -1), transb=True)
    y = f['y']
    for t in range(T):
        for g in 'zifo':                                 # :117,:122,:128,:138
            O.dot_add_mm(y[t - 1], p['R' + g], f[g.upper() + 'a'][t], transb=True)
        O.lstm_step_forward(f['Za'][t], f['Ia'][t], f['Fa'][t], f['Oa'][t], f['Ca'][t - 1],
                            p['bz'], p['bi'], p['bf'], p['bo'], p['pi'], p['pf'], p['po'],
                            f['Zb'][t], f['Ib'][t], f['Fb'][t], f['Ob'][t], f['Ca'][t], f['Cb'][t],
                            y[t], activation)


def lstm_backward(O, p, x, f, deltas, d, grads, dx, activation='tanh'):
    """lstm_layer.py:147-278.  `d` holds the ten backward internals (zero-filled,
    (T+1, B, H)), `grads` the fifteen gradients (accumulated into), `dx` the input
    deltas (accumulated into)."""
    T, B = x.shape[0], x.shape[1]
    H = f['y'].shape[2]
    dy = np.zeros_like(f['y'])
    d['dCa'][...] = 0
    for t in range(T - 1, -1, -1):
        O.copy_to(deltas[t], dy[t])                                       # :173
        for g in 'ifoz':                                                  # :174-177
            O.dot_add_mm(d['d' + g.upper() + 'a'][t + 1], p['R' + g], dy[t])
        O.lstm_step_backward(dy[t], d['dIa'][t + 1], d['dFa'][t + 1], d['dCa'][t + 1], f['Fb'][t + 1],
                             p['pi'], p['pf'], p['po'], f['Za'][t], f['Zb'][t], f['Ia'][t], f['Ib'][t],
                             f['Fa'][t], f['Fb'][t], f['Oa'][t], f['Ob'][t], f['Ca'][t], f['Cb'][t],
                             f['Ca'][t - 1], d['dZa'][t], d['dZb'][t], d['dIa'][t], d['dIb'][t],
                             d['dFa'][t], d['dFb'][t], d['dOa'][t], d['dOb'][t], d['dCa'][t], d['dCb'][t],
                             activation)
    flat_x = x.reshape(T * B, -1)
    flat_dx = dx.reshape(T * B, -1)
    fl = lambda a: a.reshape(a.shape[0] * a.shape[1], -1)
    for g in 'ifoz':                                                      # :216-224
        O.dot_add_mm(fl(d['d' + g.upper() + 'a'][:T]), p['W' + g], flat_dx)
    for g in 'ifoz':
        O.dot_add_mm(fl(d['d' + g.upper() + 'a'][:T]), flat_x, grads['W' + g], transa=True)
    tmp = np.zeros((H,), x.dtype)
    for g in 'ifoz':                                                      # :226-234
        O.sum_t(fl(d['d' + g.upper() + 'a'][:T]), 0, tmp)
        O.add_tt(grads['b' + g], tmp, grads['b' + g])
    y, Ca = f['y'], f['Ca']
    big = np.zeros((T * B, H), x.dtype)
    dWc = np.zeros((1, H), x.dtype)
    O.mult_tt(fl(Ca[:T]), fl(d['dOa'][:T]), big)                          # :244-246
    O.sum_t(big, 0, dWc)
    O.add_tt(grads['po'], dWc, grads['po'])
    for g in 'ifoz':                                                      # :253-261
        O.dot_add_mm(fl(d['d' + g.upper() + 'a'][1:T]), fl(y[:T - 1]), grads['R' + g], transa=True)
        O.dot_add_mm(d['d' + g.upper() + 'a'][0], dy[-1], grads['R' + g], transa=True)
    part = np.zeros(((T - 1) * B, H), x.dtype)
    for g in 'if':                                                        # :264-270
        O.mult_tt(fl(Ca[:T - 1]), fl(d['d' + g.upper() + 'a'][1:T]), part)
        O.sum_t(part, 0, dWc)
        O.add_tt(grads['p' + g], dWc, grads['p' + g])
    one = np.zeros((B, H), x.dtype)
    for g in 'if':                                                        # :272-278 (both use dIa[0])
        O.mult_tt(d['dCa'][-1], d['dIa'][0], one)
        O.sum_t(one, 0, dWc)
        O.add_tt(grads['p' + g], dWc, grads['p' + g])


# --------------------------------------------------------------------------
# Convolution and pooling (NHWC), restated from numpy_handler.py:89-171,210-219 and
# the loops of brainstorm/handlers/_cpuop.pyx in numpy, keeping the reference's
# order of floating-point additions (per image GEMMs; window pixels scanned row by
# row; output windows visited row by row).
# --------------------------------------------------------------------------
def _im2col_one(img, kh, kw, pad, sy, sx):
    """(oh*ow, kh*kw*C) patch matrix of one (H, W, C) image, _cpuop.pyx:251-280."""
    H, W, C = img.shape
    oh = (H + 2 * pad - kh) // sy + 1
    ow = (W + 2 * pad - kw) // sx + 1
    padded = np.zeros((H + 2 * pad, W + 2 * pad, C), img.dtype)
    padded[pad:pad + H, pad:pad + W] = img
    col = np.zeros((oh, ow, kh, kw, C), img.dtype)
    for ky in range(kh):
        for kx in range(kw):
            col[:, :, ky, kx, :] = padded[ky:ky + sy * oh:sy, kx:kx + sx * ow:sx]
    return col.reshape(oh * ow, kh * kw * C), oh, ow


def _conv2d_forward_batch(self, inputs, weights, bias, outputs, padding, stride):
    F = weights.shape[0]
    w2 = weights.reshape(F, -1)
    for i in range(inputs.shape[0]):                        # numpy_handler.py:158-169
        col, oh, ow = _im2col_one(inputs[i], weights.shape[1], weights.shape[2], padding, stride[0], stride[1])
        outputs[i].reshape(oh * ow, F)[...] = np.dot(col, w2.T)
    outputs += bias.reshape((1, 1, 1, F))                   # :171


def _conv2d_backward_batch(self, inputs, params, padding, stride, in_deltas, out_deltas, dparams, dbias):
    F, kh, kw, C = params.shape
    H, W = inputs.shape[1], inputs.shape[2]
    p2 = params.reshape(F, -1)
    dparams.fill(0.0)                                       # numpy_handler.py:118-119
    dbias.fill(0.0)
    for i in range(inputs.shape[0]):
        col, oh, ow = _im2col_one(inputs[i], kh, kw, padding, stride[0], stride[1])
        od = out_deltas[i].reshape(oh * ow, F)
        dparams.reshape(F, -1)[...] += np.dot(od.T, col)    # :135
        dbias += np.sum(od, axis=0)                         # :137
        cold = np.dot(od, p2).reshape(oh, ow, kh, kw, C)    # :141
        padded = np.zeros((H + 2 * padding, W + 2 * padding, C), inputs.dtype)
        padded[padding:padding + H, padding:padding + W] = in_deltas[i]
        for oy in range(oh):                                # col2im, _cpuop.pyx:282-309
            for ox in range(ow):
                padded[oy * stride[0]:oy * stride[0] + kh, ox * stride[1]:ox * stride[1] + kw] += cold[oy, ox]
        in_deltas[i] = padded[padding:padding + H, padding:padding + W]


def _pool_geometry(inputs, window, outputs, padding, stride):
    N, H, W, C = inputs.shape
    return N, H, W, C, window[0], window[1], stride[0], stride[1], outputs.shape[1], outputs.shape[2]


def _maxpool2d_forward_batch(self, inputs, window, outputs, padding, stride, argmax):
    N, H, W, C, kh, kw, sy, sx, oh, ow = _pool_geometry(inputs, window, outputs, padding, stride)
    lowest = -np.finfo(inputs.dtype).max
    for oy in range(oh):                                    # _cpuop.pyx:27-82
        y0, y1 = max(oy * sy - padding, 0), min(oy * sy - padding + kh, H)
        for ox in range(ow):
            x0, x1 = max(ox * sx - padding, 0), min(ox * sx - padding + kw, W)
            best = np.full((N, C), lowest, inputs.dtype)
            idx = np.full((N, C), -1.0, inputs.dtype)
            for y in range(y0, y1):
                for x in range(x0, x1):
                    v = inputs[:, y, x, :]
                    better = v > best
                    best = np.where(better, v, best)
                    idx = np.where(better, ((y * W + x) * C + np.arange(C)).astype(inputs.dtype), idx)
            outputs[:, oy, ox, :] = np.where(idx < 0, 0, best)
            argmax[:, oy, ox, :] = idx


def _maxpool2d_backward_batch(self, inputs, window, outputs, padding, stride, argmax, in_deltas, out_deltas):
    N, H, W, C, kh, kw, sy, sx, oh, ow = _pool_geometry(inputs, window, outputs, padding, stride)
    flat = in_deltas.reshape(N, H * W * C)
    for oy in range(oh):                                    # _cpuop.pyx:84-117
        for ox in range(ow):
            idx = argmax[:, oy, ox, :].astype(np.int64)
            n_i, c_i = np.nonzero(idx >= 0)
            flat[n_i, idx[n_i, c_i]] += out_deltas[n_i, oy, ox, c_i]


def _avgpool2d_forward_batch(self, inputs, window, outputs, padding, stride):
    N, H, W, C, kh, kw, sy, sx, oh, ow = _pool_geometry(inputs, window, outputs, padding, stride)
    for oy in range(oh):                                    # _cpuop.pyx:120-165
        y0, y1 = max(oy * sy - padding, 0), min(oy * sy - padding + kh, H)
        for ox in range(ow):
            x0, x1 = max(ox * sx - padding, 0), min(ox * sx - padding + kw, W)
            acc = np.zeros((N, C), inputs.dtype)
            for y in range(y0, y1):
                for x in range(x0, x1):
                    acc = acc + inputs[:, y, x, :]
            outputs[:, oy, ox, :] = acc / inputs.dtype.type(max((y1 - y0) * (x1 - x0), 1))


def _avgpool2d_backward_batch(self, inputs, window, outputs, padding, stride, in_deltas, out_deltas):
    N, H, W, C, kh, kw, sy, sx, oh, ow = _pool_geometry(inputs, window, outputs, padding, stride)
    for oy in range(oh):                                    # _cpuop.pyx:167-205
        y0, y1 = max(oy * sy - padding, 0), min(oy * sy - padding + kh, H)
        for ox in range(ow):
            x0, x1 = max(ox * sx - padding, 0), min(ox * sx - padding + kw, W)
            size = (y1 - y0) * (x1 - x0)
            if size > 0:
                in_deltas[:, y0:y1, x0:x1, :] += (out_deltas[:, oy, ox, :] /
                                                  inputs.dtype.type(size))[:, None, None, :]


OracleHandler.conv2d_forward_batch = _conv2d_forward_batch
OracleHandler.conv2d_backward_batch = _conv2d_backward_batch
OracleHandler.maxpool2d_forward_batch = _maxpool2d_forward_batch
OracleHandler.maxpool2d_backward_batch = _maxpool2d_backward_batch
OracleHandler.avgpool2d_forward_batch = _avgpool2d_forward_batch
OracleHandler.avgpool2d_backward_batch = _avgpool2d_backward_batch
