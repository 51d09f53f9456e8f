"""Generate tests/golden/handler_ops.npz from the REAL reference backend.

Runs every case of ``cases.build_cases()`` on the reference's own
``NumpyHandler(np.float32)`` (brainstorm/handlers/numpy_handler.py:13), imported
from the install that ``oracle/install_reference.sh`` makes out of the
reference checkout, and stores every array argument that the call changed
(plus the ``y = f(x)`` input of the derivative cases).  The reference is only
needed to *generate* the file; the tests read the stored vectors.

usage:  oracle/install_reference.sh && python tests/golden/make_golden.py
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, 'baseline', '_ref'))
sys.path.insert(0, HERE)

import cases as golden_cases  # noqa: E402
from brainstorm.handlers.numpy_handler import NumpyHandler  # noqa: E402


def main():
    ref = NumpyHandler(np.float32)
    cases = golden_cases.build_cases()
    golden_cases.finalize_derivs(cases, lambda: NumpyHandler(np.float32))
    store = {'__digest__': np.array(golden_cases.inputs_digest(cases)),
             '__count__': np.array(len(cases))}
    for i, c in enumerate(cases):
        arrays = c.fresh_arrays()
        getattr(ref, c.op)(*c.bind(arrays), **c.kwargs)
        for name, after in arrays.items():
            before = c.arrays[name]
            changed = not np.array_equal(before.view(np.uint32),
                                         after.view(np.uint32))
            derived_input = (name == 'y' and c.op.endswith('_deriv')) or \
                (name in ('out', 'argmax') and c.op == 'maxpool2d_backward_batch')
            if changed or derived_input:
                store['%d/%s' % (i, name)] = after
    # host-RNG parity mode: masks / gaussians drawn from a seeded RandomState
    # exactly as numpy_handler.py:193-200 does.
    rng = NumpyHandler(np.float32, seed=4711)
    mask = np.zeros((6, 50), np.float32)
    rng.generate_probability_mask(mask, 0.3)
    gauss = np.zeros((5, 40), np.float32)
    rng.fill_gaussian(0.5, 2.0, gauss)
    store['rng/mask'] = mask
    store['rng/gauss'] = gauss
    out = os.path.join(HERE, 'handler_ops.npz')
    np.savez_compressed(out, **store)
    print('%d cases, %d stored arrays, %.1f KiB -> %s' % (
        len(cases), len(store), os.path.getsize(out) / 1024.0, out))


if __name__ == '__main__':
    main()
