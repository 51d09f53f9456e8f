"""Parity at the sizes the benchmark configurations state, not at reduced ones.

* op suite: all 27 ops on the full seed-1 draw of fp32 (65536, 4096) operands (1 GiB
  each), every output element compared with the CPU oracle (row chunks over the host's
  threads; the axis-0 and whole-array sums against the oracle's result on the whole
  matrix and against float64);
* character LSTM: time 100, batch 128, 205 symbols, two fused layers of 1000 units, one
  forward/backward pass against the reference's own LstmLayerImpl on NumpyHandler: loss,
  every gradient, all twenty internals of both layers;
* Highway + BatchNorm: batch 8192, width 4096, ten blocks, 1000 classes, one
  forward/backward pass against NumpyHandler: loss, gradients, batch statistics.

The CPU side of each costs tens of seconds of host time; tolerances are those of
tests/parity.py (the error bound of a sum or product is taken per output element from
the sum of the absolute values of its terms, never from the largest entry of a buffer).
"""
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

import parity
from conftest import needs_reference
from oracle.numpy_oracle import OracleHandler, op_suite_inputs

pytestmark = pytest.mark.gpu

ROWS, COLS, SEED = 65536, 4096, 1
CHUNK = 2048


# ------------------------------------------------------------------ op suite, (65536, 4096) seed 1
@pytest.fixture(scope='module')
def suite():
    from brainstorm_b200 import B200Handler
    H = B200Handler(seed=SEED, rng_mode='host')
    d = op_suite_inputs(ROWS, COLS, SEED)
    d['labels'] = d['labels'].astype(np.float32)
    dev = {k: H.create_from_numpy(v) for k, v in d.items()}
    dev['out'] = H.zeros((ROWS, COLS))
    dev['y'] = H.zeros((ROWS, COLS))
    pool = ThreadPoolExecutor(max_workers=os.cpu_count() or 4)
    yield H, OracleHandler(np.float32), d, dev, pool
    pool.shutdown()


def _chunks():
    return [(lo, min(ROWS, lo + CHUNK)) for lo in range(0, ROWS, CHUNK)]


def _by_rows(pool, fn):
    """fn(lo, hi) on every row chunk, on the pool's threads (numpy releases the GIL);
    assertion errors of any chunk surface here."""
    return list(pool.map(lambda c: fn(*c), _chunks()))


def _check_elementwise(op, pool, got, want_chunk):
    def one(lo, hi):
        want = want_chunk(lo, hi)
        if op in parity.BIT_EXACT_OPS:
            parity.assert_bits_equal(got[lo:hi], want, '%s rows %d..%d' % (op, lo, hi))
        else:
            parity.assert_elementwise_close(got[lo:hi], want, op, 'rows %d..%d' % (lo, hi))
    _by_rows(pool, one)


BINARY = [('add_tt', 'a', 'b'), ('subtract_tt', 'a', 'b'), ('mult_tt', 'a', 'b'), ('divide_tt', 'a', 'div')]


@pytest.mark.parametrize('op,x,y', BINARY, ids=[b[0] for b in BINARY])
def test_config2_tensor_tensor(suite, op, x, y):
    H, O, d, dev, pool = suite
    getattr(H, op)(dev[x], dev[y], dev['out'])
    got = H.get_numpy_copy(dev['out'])

    def want(lo, hi):
        z = np.empty((hi - lo, COLS), np.float32)
        getattr(O, op)(d[x][lo:hi], d[y][lo:hi], z)
        return z
    _check_elementwise(op, pool, got, want)


@pytest.mark.parametrize('op,vec', [('add_mv', 'row'), ('add_mv', 'col'), ('mult_mv', 'row'), ('mult_mv', 'col')])
def test_config2_broadcast(suite, op, vec):
    H, O, d, dev, pool = suite
    getattr(H, op)(dev['a'], dev[vec], dev['out'])
    got = H.get_numpy_copy(dev['out'])

    def want(lo, hi):
        z = np.empty((hi - lo, COLS), np.float32)
        getattr(O, op)(d['a'][lo:hi], d[vec] if vec == 'row' else d[vec][lo:hi], z)
        return z
    _check_elementwise(op, pool, got, want)


UNARY = [('mult_st', lambda h, a, z: h.mult_st(0.37, a, z)), ('clip_t', lambda h, a, z: h.clip_t(a, -1.0, 1.0, z)),
         ('abs_t', lambda h, a, z: h.abs_t(a, z)), ('sign_t', lambda h, a, z: h.sign_t(a, z))]


@pytest.mark.parametrize('op,call', UNARY, ids=[u[0] for u in UNARY])
def test_config2_unary(suite, op, call):
    H, O, d, dev, pool = suite
    call(H, dev['a'], dev['out'])
    got = H.get_numpy_copy(dev['out'])

    def want(lo, hi):
        z = np.empty((hi - lo, COLS), np.float32)
        call(O, d['a'][lo:hi], z)
        return z
    _check_elementwise(op, pool, got, want)


def test_config2_sqrt_of_absolute_values(suite):
    H, O, d, dev, pool = suite
    H.abs_t(dev['a'], dev['y'])
    H.sqrt_t(dev['y'], dev['out'])
    got = H.get_numpy_copy(dev['out'])

    def want(lo, hi):
        z = np.empty((hi - lo, COLS), np.float32)
        O.sqrt_t(np.abs(d['a'][lo:hi]), z)
        return z
    _check_elementwise('sqrt_t', pool, got, want)


@pytest.mark.parametrize('act', ['sigmoid', 'tanh', 'rel', 'el'])
def test_config2_activation_and_derivative(suite, act):
    H, O, d, dev, pool = suite
    getattr(H, act)(dev['a'], dev['out'])
    got = H.get_numpy_copy(dev['out'])
    y = np.empty((ROWS, COLS), np.float32)          # the oracle's activations: inputs of the derivative on both sides

    def fwd(lo, hi):
        getattr(O, act)(d['a'][lo:hi], y[lo:hi])
        return y[lo:hi]
    _check_elementwise(act, pool, got, fwd)
    H.set_from_numpy(dev['y'], y)
    getattr(H, act + '_deriv')(dev['a'], dev['y'], dev['dy'], dev['out'])
    got = H.get_numpy_copy(dev['out'])

    def bwd(lo, hi):
        z = np.empty((hi - lo, COLS), np.float32)
        getattr(O, act + '_deriv')(d['a'][lo:hi], y[lo:hi], d['dy'][lo:hi], z)
        return z
    _check_elementwise(act + '_deriv', pool, got, bwd)


def test_config2_sums_over_both_axes_and_everything(suite):
    H, O, d, dev, pool = suite
    a = d['a']
    s0, s1, sall = H.zeros((1, COLS)), H.zeros((ROWS, 1)), H.zeros(())
    H.sum_t(dev['a'], 0, s0)
    H.sum_t(dev['a'], 1, s1)
    H.sum_t(dev['a'], None, sall)
    g0, g1, gall = H.get_numpy_copy(s0), H.get_numpy_copy(s1), H.get_numpy_copy(sall)
    # the oracle on the whole matrix, as NumpyHandler would run it
    w0, w1, wall = np.zeros((1, COLS), np.float32), np.zeros((ROWS, 1), np.float32), np.zeros((), np.float32)
    O.sum_t(a, 0, w0)
    O.sum_t(a, 1, w1)
    O.sum_t(a, None, wall)
    # float64 sums and sums of absolute values, by row chunks
    parts = _by_rows(pool, lambda lo, hi: (a[lo:hi].astype(np.float64).sum(0),
                                           np.abs(a[lo:hi]).astype(np.float64).sum(0),
                                           a[lo:hi].astype(np.float64).sum(1),
                                           np.abs(a[lo:hi]).astype(np.float64).sum(1)))
    e0 = np.sum([p[0] for p in parts], axis=0).reshape(1, COLS)
    abs0 = np.sum([p[1] for p in parts], axis=0).reshape(1, COLS)
    e1 = np.concatenate([p[2] for p in parts]).reshape(ROWS, 1)
    abs1 = np.concatenate([p[3] for p in parts]).reshape(ROWS, 1)
    parity.assert_reduction_close(g0, w0, abs0, 'sum_t', 'axis 0 vs oracle, every column')
    parity.assert_reduction_close(g0, e0, abs0, 'sum_t', 'axis 0 vs float64')
    parity.assert_reduction_close(g1, w1, abs1, 'sum_t', 'axis 1 vs oracle, every row')
    parity.assert_reduction_close(g1, e1, abs1, 'sum_t', 'axis 1 vs float64')
    parity.assert_reduction_close(gall, wall, abs0.sum(), 'sum_t', 'all vs oracle')
    parity.assert_reduction_close(gall, e0.sum(), abs0.sum(), 'sum_t', 'all vs float64')


def test_config2_softmax(suite):
    H, O, d, dev, pool = suite
    H.softmax_m(dev['a'], dev['out'])
    got = H.get_numpy_copy(dev['out'])

    def one(lo, hi):
        z = np.empty((hi - lo, COLS), np.float32)
        O.softmax_m(d['a'][lo:hi], z)
        parity.assert_reduction_close(got[lo:hi], z, 0.0, 'softmax_m', 'rows %d..%d' % (lo, hi))
    _by_rows(pool, one)


def test_config2_labels_bit_exact(suite):
    H, O, d, dev, pool = suite
    H.binarize_v(dev['labels'], dev['out'])
    got = H.get_numpy_copy(dev['out'])

    def one(lo, hi):
        z = np.empty((hi - lo, COLS), np.float32)
        O.binarize_v(d['labels'][lo:hi], z)
        parity.assert_bits_equal(got[lo:hi], z, 'binarize_v rows %d..%d' % (lo, hi))
    _by_rows(pool, one)
    picked = H.zeros((ROWS, 1))
    H.index_m_by_v(dev['a'], dev['labels'], picked)
    want = np.zeros((ROWS, 1), np.float32)
    O.index_m_by_v(d['a'], d['labels'], want)
    parity.assert_bits_equal(H.get_numpy_copy(picked), want, 'index_m_by_v')


# ------------------------------------------------------------------ training configurations
# Bounds.  Every compared element must satisfy |gpu - cpu| <= RTOL * |cpu| + RTOL * scale,
# where scale is the sum of the absolute values of the terms that were added up to give
# that element (for values that are products or bounded-slope functions of such sums,
# the scale of the sum times the factor), computed from the CPU run's own buffers.
# Neither side is exact: NumpyHandler's float32 BLAS and the GPU's split-TF32 tensor-core
# GEMM round differently, and what one rounding can move is proportional to that scale.
RTOL = parity.REDUCTION_RTOL
_A, _bounded, _report, _fc_checks = parity.absf, parity.bounded, parity.report, parity.fc_layer_checks


def _pair(builder, fused=False, **kw):
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200 import B200Handler
    net_cpu, data, _ = builder(**kw)
    net_cpu.set_handler(NumpyHandler(np.float32, seed=77))
    net_gpu, _, _ = builder(**kw)
    net_gpu.set_handler(B200Handler(seed=77, rng_mode='host'))
    if fused:
        from brainstorm_b200.fused_lstm import fuse_lstm_layers
        assert fuse_lstm_layers(net_gpu)
    assert np.array_equal(net_cpu.get('parameters'), net_gpu.get('parameters'))
    for net in (net_cpu, net_gpu):
        net.provide_external_data(data)
        net.forward_pass(training_pass=True)
        net.backward_pass()
    l_cpu = float(net_cpu.get_loss_values()['total_loss'])
    l_gpu = float(net_gpu.get_loss_values()['total_loss'])
    assert abs(l_cpu - l_gpu) <= RTOL * abs(l_cpu), (l_cpu, l_gpu)
    return net_cpu, net_gpu


@needs_reference
def test_config4_lstm_full_size_forward_backward():
    """Time 100, batch 128, 205 symbols, two LSTM layers of 1000 units (fused on the GPU),
    SoftmaxCE: loss, every gradient and the twenty internals, outputs and input deltas of
    both layers against the reference's LstmLayerImpl on NumpyHandler."""
    from brainstorm_b200 import workloads
    T, B, H = 100, 128, 1000
    net_cpu, net_gpu = _pair(workloads.lstm, fused=True, time=T, batch=B, vocab=205, hidden=H, layers=2)
    worst = {}
    parity.lstm_net_checks(net_cpu, net_gpu, T, worst)
    _report(worst, 'config 4 (T=100, B=128, 2 x 1000)')


@needs_reference
def test_config5_highway_batchnorm_full_size_forward_backward():
    """Batch 8192, width 4096, ten Highway + BatchNorm blocks, 1000 classes: loss, every
    layer's outputs and gradients, the batch statistics and the running statistics.

    Scales follow the data flow: a buffer that combines the outputs of the two
    FullyConnected layers carries their scales (the sums of |terms| of their 4096-term dot
    products) times the factors they are multiplied with; the Highway carry path hands the
    scale of the block's input on to its output, BatchNorm divides it by the batch standard
    deviation; on the way back the deltas a block receives carry the scale the block above
    attached to them."""
    from brainstorm_b200 import workloads
    net_cpu, net_gpu = _pair(workloads.highway_bn, batch=8192, width=4096, classes=1000, blocks=10)
    worst = {}
    m = 8192.0
    g = lambda net, path: net.get(path)
    shares, s_x = {}, 0.0
    for i in range(10):
        (s_h, share_h), (s_t, share_t) = (_fc_checks(net_cpu, net_gpu, n, worst) for n in ('H%d' % i, 'T%d' % i))
        shares[i] = share_h + share_t
        s_h, s_t = s_h[0], s_t[0]
        hw, bn = 'HW%d' % i, 'BN%d' % i
        x, Hh, Tt = (_A(g(net_cpu, '%s.inputs.%s' % (hw, k)))[0] for k in ('x', 'H', 'T'))
        # Highway (highway_layer.py:52-77): y = T*(H - x) + x
        s_hw = Tt * (Hh + x) + x + Tt * s_h + (Hh + x) * s_t + (1 + Tt) * s_x
        _bounded(g(net_gpu, hw + '.outputs.default'), g(net_cpu, hw + '.outputs.default'), s_hw, hw + '.outputs', worst)
        # BatchNorm forward (batch_normalization_layer.py:54-105); its input is the Highway output
        sig = g(net_cpu, bn + '.internals.sigma_b').astype(np.float64)
        gam, bet = (_A(g(net_cpu, '%s.parameters.%s' % (bn, k))) for k in ('gamma', 'beta'))
        s_c = s_hw + s_hw.sum(0) / m                               # centered = x - mean
        cen = _A(g(net_cpu, bn + '.internals.centered'))[0]
        _bounded(g(net_gpu, bn + '.internals.sigma_b'), sig, (s_c * cen).sum(0) / m / sig, bn + '.sigma_b', worst)
        _bounded(g(net_gpu, bn + '.internals.centered'), g(net_cpu, bn + '.internals.centered'), s_c, bn + '.centered', worst)
        _bounded(g(net_gpu, bn + '.internals.x_hat'), g(net_cpu, bn + '.internals.x_hat'), s_c / sig, bn + '.x_hat', worst)
        s_x = (s_c / sig * gam + bet).astype(np.float32)           # the next block's input
        _bounded(g(net_gpu, bn + '.outputs.default'), g(net_cpu, bn + '.outputs.default'), s_x, bn + '.outputs', worst)
        for k in ('mu', 'sigma'):                                  # running statistics, updated by the forward pass
            _bounded(g(net_gpu, '%s.parameters.%s' % (bn, k)), g(net_cpu, '%s.parameters.%s' % (bn, k)),
                     s_hw.sum(0) / m, '%s.%s' % (bn, k), worst)
    _, above = _fc_checks(net_cpu, net_gpu, 'Output_projection', worst, in_scale=s_x)    # scale of the deltas it hands down
    for i in range(9, -1, -1):
        hw, bn = 'HW%d' % i, 'BN%d' % i
        # BatchNorm backward (:107-152): dgamma, dbeta, and the three-term input delta
        sig = g(net_cpu, bn + '.internals.sigma_b').astype(np.float64)
        gam = _A(g(net_cpu, bn + '.parameters.gamma'))
        dout = np.maximum(_A(g(net_cpu, bn + '.output_deltas.default'))[0], above)
        xh = _A(g(net_cpu, bn + '.internals.x_hat'))[0]
        s_dgamma, s_dbeta = (dout * xh).sum(0), dout.sum(0)
        _bounded(g(net_gpu, bn + '.gradients.gamma'), g(net_cpu, bn + '.gradients.gamma'), s_dgamma, bn + '.dgamma', worst)
        _bounded(g(net_gpu, bn + '.gradients.beta'), g(net_cpu, bn + '.gradients.beta'), s_dbeta, bn + '.dbeta', worst)
        s_bn_in = (dout + xh * s_dgamma / m + s_dbeta / m) * gam / sig
        _bounded(g(net_gpu, bn + '.input_deltas.default'), g(net_cpu, bn + '.input_deltas.default'), s_bn_in,
                 bn + '.input_deltas', worst)
        # deltas of the block's input: three sinks add into one buffer (H-FC, T-FC, Highway.x)
        Tt = _A(g(net_cpu, hw + '.inputs.T'))[0]
        above = (shares.pop(i) + (1 + Tt) * s_bn_in).astype(np.float32)
        _bounded(g(net_gpu, hw + '.input_deltas.x'), g(net_cpu, hw + '.input_deltas.x'), above, hw + '.input_deltas.x', worst)
    _report(worst, 'config 5 (8192 x 4096, 10 blocks)')
