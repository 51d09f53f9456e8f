"""Convolution and pooling with channel counts that take the 128-bit forms of the kernels
(multiples of 4), against the reference's NumpyHandler (its Cython loops), and the reference's
CIFAR-10 network (examples/cifar10_cnn.py) trained on both handlers."""
import numpy as np
import pytest

from conftest import needs_reference

pytestmark = [pytest.mark.gpu, needs_reference]


def _handlers():
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200 import B200Handler
    return NumpyHandler(np.float32), B200Handler()


def _out_hw(H, W, kh, kw, pad, st):
    return (H + 2 * pad - kh) // st[0] + 1, (W + 2 * pad - kw) // st[1] + 1


def _close(got, want, scale, what):
    err = np.abs(got - want).max() if got.size else 0.0
    assert err <= 1e-5 * scale, '%s: max error %.3g against scale %.3g' % (what, err, scale)


@pytest.mark.parametrize('img,filters,k,pad,st', [((3, 15, 15, 32), 32, (5, 5), 2, (1, 1)), ((2, 9, 7, 8), 5, (3, 3), 1, (2, 2)),
                                                   ((2, 8, 8, 4), 8, (3, 2), 0, (1, 2)), ((1, 7, 7, 64), 64, (5, 5), 2, (1, 1)),
                                                   ((4, 6, 5, 12), 7, (2, 2), 1, (1, 1))])
def test_convolution_with_wide_channels(img, filters, k, pad, st):
    cpu, gpu = _handlers()
    rs = np.random.RandomState(sum(img) + filters)
    N, H, W, C = img
    oh, ow = _out_hw(H, W, k[0], k[1], pad, st)
    x = rs.randn(*img).astype(np.float32)
    w = rs.uniform(-1, 1, (filters, k[0], k[1], C)).astype(np.float32)
    b = rs.uniform(-1, 1, (filters,)).astype(np.float32)
    od = rs.randn(N, oh, ow, filters).astype(np.float32)
    ind = rs.randn(*img).astype(np.float32)
    res = []
    for h in (cpu, gpu):
        X, Wt, Bs = h.create_from_numpy(x), h.create_from_numpy(w), h.create_from_numpy(b)
        out = h.zeros((N, oh, ow, filters))
        h.conv2d_forward_batch(X, Wt, Bs, out, pad, st)
        ID, OD = h.create_from_numpy(ind), h.create_from_numpy(od)
        dW, dB = h.zeros(w.shape), h.zeros(b.shape)
        h.conv2d_backward_batch(X, Wt, pad, st, ID, OD, dW, dB)
        res.append([h.get_numpy_copy(a) for a in (out, ID, dW, dB)])
    taps = k[0] * k[1] * C
    _close(res[1][0], res[0][0], np.abs(x).max() * np.abs(w).max() * taps + 1, 'outputs')
    _close(res[1][1], res[0][1], np.abs(od).max() * np.abs(w).max() * k[0] * k[1] * filters + np.abs(ind).max(), 'in_deltas')
    _close(res[1][2], res[0][2], np.abs(od).max() * np.abs(x).max() * N * oh * ow, 'dW')
    _close(res[1][3], res[0][3], np.abs(od).sum(axis=(0, 1, 2)).max(), 'dbias')


@pytest.mark.parametrize('img,win,pad,st', [((3, 32, 32, 32), (3, 3), 0, (2, 2)), ((2, 9, 7, 8), (2, 2), 1, (1, 1)),
                                            ((2, 6, 6, 4), (4, 4), 2, (1, 2)), ((5, 7, 7, 64), (3, 3), 0, (2, 2))])
def test_pooling_with_wide_channels(img, win, pad, st):
    cpu, gpu = _handlers()
    rs = np.random.RandomState(sum(img))
    N, H, W, C = img
    oh, ow = _out_hw(H, W, win[0], win[1], pad, st)
    x = rs.randn(*img).astype(np.float32)
    od = rs.randn(N, oh, ow, C).astype(np.float32)
    ind = rs.randn(*img).astype(np.float32)
    res = []
    for h in (cpu, gpu):
        X = h.create_from_numpy(x)
        out, am = h.zeros((N, oh, ow, C)), h.zeros((N, oh, ow, C))
        h.maxpool2d_forward_batch(X, win, out, pad, st, am)
        ID, OD = h.create_from_numpy(ind), h.create_from_numpy(od)
        h.maxpool2d_backward_batch(X, win, out, pad, st, am, ID, OD)
        aout = h.zeros((N, oh, ow, C))
        h.avgpool2d_forward_batch(X, win, aout, pad, st)
        AID = h.create_from_numpy(ind)
        h.avgpool2d_backward_batch(X, win, aout, pad, st, AID, OD)
        res.append([h.get_numpy_copy(a) for a in (out, am, ID, aout, AID)])
    assert np.array_equal(res[1][0], res[0][0]), 'max pooling outputs'
    assert np.array_equal(res[1][1], res[0][1]), 'argmax'
    _close(res[1][2], res[0][2], np.abs(od).max() * win[0] * win[1] + np.abs(ind).max(), 'max pooling in_deltas')
    _close(res[1][3], res[0][3], np.abs(x).max(), 'average pooling outputs')
    _close(res[1][4], res[0][4], np.abs(od).max() * win[0] * win[1] + np.abs(ind).max(), 'average pooling in_deltas')


def test_cifar10_network_trains_like_on_numpy_handler():
    from brainstorm_b200 import workloads
    from test_b200_networks import _check_training
    _check_training(workloads.cifar10_cnn, steps=2, batch=12)
