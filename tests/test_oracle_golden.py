"""The oracle must reproduce the reference's stored outputs bit for bit."""
import os

import numpy as np
import pytest

import cases as golden_cases
from oracle.numpy_oracle import OracleHandler

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), 'golden',
                              'handler_ops.npz'))
CASES = golden_cases.build_cases()


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def test_generator_inputs_unchanged():
    assert int(GOLDEN['__count__']) == len(CASES)
    assert str(GOLDEN['__digest__']) == golden_cases.inputs_digest(CASES)


@pytest.mark.parametrize('idx', range(len(CASES)), ids=[c.id for c in CASES])
def test_oracle_matches_reference_bits(idx):
    c = CASES[idx]
    if c.op.endswith('_deriv'):
        c.arrays['y'] = GOLDEN['%d/y' % idx]
    if c.op == 'maxpool2d_backward_batch':
        c.arrays['out'], c.arrays['argmax'] = GOLDEN['%d/out' % idx], GOLDEN['%d/argmax' % idx]
    arrays = c.fresh_arrays()
    getattr(OracleHandler(np.float32), c.op)(*c.bind(arrays), **c.kwargs)
    for name, got in arrays.items():
        key = '%d/%s' % (idx, name)
        want = GOLDEN[key] if key in GOLDEN.files else c.arrays[name]
        assert got.shape == want.shape
        assert np.array_equal(_bits(got), _bits(want)), (c.id, name)


def test_host_rng_matches_reference():
    h = OracleHandler(np.float32, seed=4711)
    mask = np.zeros((6, 50), np.float32)
    h.generate_probability_mask(mask, 0.3)
    gauss = np.zeros((5, 40), np.float32)
    h.fill_gaussian(0.5, 2.0, gauss)
    assert np.array_equal(mask, GOLDEN['rng/mask'])
    assert np.array_equal(_bits(gauss), _bits(GOLDEN['rng/gauss']))
