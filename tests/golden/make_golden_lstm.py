"""Generate tests/golden/lstm_layer.npz from the REAL reference LSTM layer.

Runs the reference's own network stack (two LstmLayerImpl layers + SoftmaxCE, built by
tools.create_net_from_spec) on NumpyHandler(float32) for one forward and backward pass
and stores, for the first LSTM layer, its parameters, inputs, every internal buffer,
outputs, output deltas, input deltas and gradients.

usage:  oracle/install_reference.sh && python tests/golden/make_golden_lstm.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, 'baseline', '_ref'))
sys.path.insert(0, ROOT)

from brainstorm.handlers import NumpyHandler  # noqa: E402
from brainstorm_b200 import workloads  # noqa: E402


def main():
    store = {}
    for tag, kw in (('a', dict(time=5, batch=3, vocab=6, hidden=4)),
                    ('b', dict(time=9, batch=16, vocab=12, hidden=24))):
        net, data, _ = workloads.lstm(seed=7, data_seed=8, **kw)
        net.set_handler(NumpyHandler(np.float32))
        net.provide_external_data(data)
        net.forward_pass(training_pass=True)
        net.backward_pass()
        L = 'Lstm_1'
        for kind in ('parameters', 'internals', 'gradients', 'inputs', 'outputs', 'input_deltas', 'output_deltas'):
            for name in net.buffer[L][kind].keys():
                store['%s/%s/%s' % (tag, kind, name)] = net.get('%s.%s.%s' % (L, kind, name))
    out = os.path.join(HERE, 'lstm_layer.npz')
    np.savez_compressed(out, **store)
    print('%d arrays, %.1f KiB -> %s' % (len(store), os.path.getsize(out) / 1024.0, out))


if __name__ == '__main__':
    main()
