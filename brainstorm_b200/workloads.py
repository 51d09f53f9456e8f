"""Builders of the training workloads the backend is measured on.

They only assemble networks out of the reference's own, unchanged layers,
``Network`` and steppers (the callers of the handler); nothing here computes.
brainstorm must be importable (see oracle/install_reference.sh).

Shapes follow the reference's examples: ``mlp`` is examples/mnist_pi.py:28-37 with
MomentumStepper(0.1, 0.9) (:46); ``lstm`` is examples/hutter_lstm.py:24-32 with two
LSTM layers of 1000 units on 205 symbols; ``highway_bn`` is a stack of Highway
layers (tanh transform, sigmoid gate) each followed by BatchNorm.  Datasets are
not available, so inputs are seeded synthetic arrays of the same shapes.
"""
from __future__ import annotations

import numpy as np


def _bs():
    import brainstorm as bs
    return bs


def op_suite_inputs(rows, cols, seed, alloc=None):
    """Inputs of the handler op suite: fp32 (rows, cols) operands ``a``, ``b``, ``dy``
    uniform[-4, 4], a (1, cols) row vector, a (rows, 1) column vector, divisors ``div``
    uniform[0.5, 4] with a random sign, and int32 ``labels`` uniform in [0, cols), all
    from ``RandomState(seed)``.  The draw runs in row blocks (a few hundred MB of
    float64 at a time), which consumes the generator's stream exactly as one draw per
    array would; ``alloc(shape)`` may supply the float32 arrays (e.g. page-locked)."""
    rs = np.random.RandomState(seed)
    f32 = np.float32
    alloc = alloc or (lambda shape: np.empty(shape, f32))
    block = max(1, (1 << 25) // max(cols, 1))          # rows per block: 32 Mi samples

    def u(shape, lo=-4.0, hi=4.0, out=None):
        out = alloc(shape) if out is None else out
        for r0 in range(0, shape[0], block):
            r1 = min(shape[0], r0 + block)
            out[r0:r1] = rs.random_sample((r1 - r0,) + tuple(shape[1:])).astype(f32) * f32(hi - lo) + f32(lo)
        return out

    d = {}
    d['a'] = u((rows, cols))
    d['b'] = u((rows, cols))
    d['dy'] = u((rows, cols))
    d['row'] = u((1, cols))
    d['col'] = u((rows, 1))
    sign = np.empty((rows, cols), f32)
    for r0 in range(0, rows, block):
        r1 = min(rows, r0 + block)
        sign[r0:r1] = np.where(rs.random_sample((r1 - r0, cols)) < 0.5, f32(-1), f32(1))
    d['div'] = u((rows, cols), 0.5, 4.0)
    d['div'] *= sign
    d['labels'] = rs.randint(0, cols, size=(rows, 1)).astype(np.int32)
    return d


def mlp(batch=100, hidden=1200, n_in=784, n_out=10, seed=42, data_seed=0):
    bs = _bs()
    bs.global_rnd.set_seed(seed)
    inp, fc = bs.tools.get_in_out_layers('classification', (n_in,), n_out, projection_name='FC')
    net = bs.Network.from_layer(
        inp >> bs.layers.Dropout(drop_prob=0.2) >>
        bs.layers.FullyConnected(hidden, name='Hid1', activation='rel') >>
        bs.layers.Dropout(drop_prob=0.5) >>
        bs.layers.FullyConnected(hidden, name='Hid2', activation='rel') >>
        bs.layers.Dropout(drop_prob=0.5) >> fc)
    net.initialize(bs.initializers.Gaussian(0.01))
    rs = np.random.RandomState(data_seed)
    data = {'default': rs.uniform(0, 1, (1, batch, n_in)).astype(np.float32),
            'targets': rs.randint(0, n_out, (1, batch, 1)).astype(np.int32)}
    stepper = lambda: bs.training.MomentumStepper(learning_rate=0.1, momentum=0.9)
    return net, data, stepper


def lstm(time=100, batch=128, vocab=205, hidden=1000, layers=2, seed=42, data_seed=0):
    bs = _bs()
    bs.global_rnd.set_seed(seed)
    net = bs.tools.create_net_from_spec('classification', vocab, vocab,
                                        ' '.join(['L%d' % hidden] * layers))
    net.initialize(bs.initializers.Uniform(0.1))
    rs = np.random.RandomState(data_seed)
    idx = rs.randint(0, vocab, (time, batch))
    data = {'default': np.eye(vocab, dtype=np.float32)[idx],
            'targets': rs.randint(0, vocab, (time, batch, 1)).astype(np.int32)}
    stepper = lambda: bs.training.SgdStepper(learning_rate=0.1)
    return net, data, stepper


def highway_bn(batch=8192, width=4096, classes=1000, blocks=10, seed=42, data_seed=0):
    bs = _bs()
    bs.global_rnd.set_seed(seed)
    inp, fc = bs.tools.get_in_out_layers('classification', (width,), classes)
    cur = inp
    for i in range(blocks):
        h = bs.layers.FullyConnected(width, activation='tanh', name='H%d' % i)
        t = bs.layers.FullyConnected(width, activation='sigmoid', name='T%d' % i)
        hw = bs.layers.Highway(name='HW%d' % i)
        cur >> h >> 'H' - hw
        cur >> t >> 'T' - hw
        cur >> 'x' - hw
        cur = hw >> bs.layers.BatchNorm(name='BN%d' % i)
    net = bs.Network.from_layer(cur >> fc)
    net.initialize({'default': bs.initializers.Gaussian(0.02),
                    'BN*': {'gamma': 1, 'beta': 0, 'mu': 0, 'sigma': 1}})
    rs = np.random.RandomState(data_seed)
    data = {'default': rs.randn(1, batch, width).astype(np.float32),
            'targets': rs.randint(0, classes, (1, batch, 1)).astype(np.int32)}
    stepper = lambda: bs.training.SgdStepper(learning_rate=0.01)
    return net, data, stepper


def cifar10_cnn(batch=100, seed=42, data_seed=0):
    """The convolutional network of the reference's examples/cifar10_cnn.py:28-46 (three 5x5
    convolutions with 3x3 / stride-2 max pooling, two FullyConnected layers, momentum SGD,
    minibatches of 100) on seeded stand-ins for normalised 32 x 32 x 3 images."""
    bs = _bs()
    bs.global_rnd.set_seed(seed)
    inp, fc = bs.tools.get_in_out_layers('classification', (32, 32, 3), 10)
    (inp >>
     bs.layers.Convolution2D(32, kernel_size=(5, 5), padding=2, name='Conv1') >>
     bs.layers.Pooling2D(type='max', kernel_size=(3, 3), stride=(2, 2)) >>
     bs.layers.Convolution2D(32, kernel_size=(5, 5), padding=2, name='Conv2') >>
     bs.layers.Pooling2D(type='max', kernel_size=(3, 3), stride=(2, 2)) >>
     bs.layers.Convolution2D(64, kernel_size=(5, 5), padding=2, name='Conv3') >>
     bs.layers.Pooling2D(type='max', kernel_size=(3, 3), stride=(2, 2)) >>
     bs.layers.FullyConnected(64, name='FC') >> fc)
    net = bs.Network.from_layer(fc)
    net.initialize({'Conv*': {'W': bs.initializers.Gaussian(0.01), 'bias': 0},
                    'FC': {'W': bs.initializers.Gaussian(0.1), 'bias': 0},
                    'Output_projection': {'W': bs.initializers.Gaussian(0.1), 'bias': 0}})
    rs = np.random.RandomState(data_seed)
    data = {'default': rs.randn(1, batch, 32, 32, 3).astype(np.float32),
            'targets': rs.randint(0, 10, (1, batch, 1)).astype(np.int32)}
    stepper = lambda: bs.training.MomentumStepper(learning_rate=0.01, momentum=0.9)
    return net, data, stepper


def train_steps(net, data, stepper, steps):
    """Runs `steps` updates exactly as Trainer does per minibatch
    (training/trainer.py:96-101): provide data, stepper.run, read the loss."""
    stepper.start(net)
    losses = []
    for _ in range(steps):
        net.provide_external_data(data)
        stepper.run()
        losses.append(float(net.get_loss_values()['total_loss']))
        net.apply_weight_modifiers()
    return losses
