"""Every layer the reference tests itself with (brainstorm/tests/test_layers.py:
31 layer factories x 4 (time, batch, activation) specs), set up exactly as the
reference's own helper does (tests/helpers.py:45-76), run forward and backward on
B200Handler and on NumpyHandler(float32) with identical values, all buffers
compared, convolution and pooling layers included."""
import numpy as np
import pytest

from conftest import needs_reference, has_reference

pytestmark = [pytest.mark.gpu, needs_reference]

if has_reference():
    from brainstorm.tests import test_layers as ref_tests
    FACTORIES = ref_tests.layers_to_test
    SPECS = ref_tests.spec_list
else:                                                   # collected, then skipped
    FACTORIES, SPECS = [], []


def _set_up(layer, spec, handler, seed):
    from brainstorm.structure.layout import create_layout
    from brainstorm.structure.buffers import get_total_size_slices_and_shapes
    from brainstorm.structure.buffer_views import BufferView  # noqa: F401
    from brainstorm.structure.buffers import create_buffer_views_from_layout
    layer.set_handler(handler)
    T, B = spec.get('time_steps', 3), spec.get('batch_size', 2)
    hubs, layout = create_layout({'test_layer': layer})
    total, slices, shapes = get_total_size_slices_and_shapes(hubs, T, B)
    full = handler.allocate((total,))
    buffers = [full[s].reshape(sh) for s, sh in zip(slices, shapes)]
    view = create_buffer_views_from_layout(layout, buffers, hubs)
    rs = np.random.RandomState(seed)
    handler.set_from_numpy(view.parameters, rs.randn(view.parameters.size))
    for name, value in spec.get('inits', {}).items():
        handler.set_from_numpy(view.test_layer.parameters[name], value)
    lb = view.test_layer
    for key in lb.inputs.keys():
        value = spec[key] if key in spec else rs.randn(*lb.inputs[key].shape)
        handler.set_from_numpy(lb.inputs[key], value)
    return lb, rs


def _run(factory, spec_tuple, handler):
    np.random.seed(4321)                 # the factories draw targets from the global generator
    spec = dict(zip(('time_steps', 'batch_size', 'activation'), spec_tuple))
    layer, spec = factory(spec)
    lb, rs = _set_up(layer, spec, handler, seed=99)
    layer.forward_pass(lb)
    for key in lb.output_deltas.keys():
        handler.set_from_numpy(lb.output_deltas[key], rs.randn(*lb.output_deltas[key].shape))
    layer.backward_pass(lb)
    out = {}
    for kind in ('outputs', 'input_deltas', 'gradients', 'internals'):
        for key in lb[kind].keys():
            out['%s.%s' % (kind, key)] = handler.get_numpy_copy(lb[kind][key])
    return out


@pytest.mark.parametrize('spec', SPECS, ids=['%d-%d-%s' % s for s in SPECS])
@pytest.mark.parametrize('factory', FACTORIES, ids=[f.__name__ for f in FACTORIES])
def test_layer_forward_backward_matches_numpy_handler(factory, spec):
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200 import B200Handler
    gpu = B200Handler(seed=3, rng_mode='host')
    want = _run(factory, spec, NumpyHandler(np.float32, seed=3))
    got = _run(factory, spec, gpu)
    assert set(got) == set(want)
    for key in want:
        w, g = want[key], got[key]
        assert g.shape == w.shape, key
        scale = max(float(np.abs(w).max()), 1e-30) if w.size else 1.0
        err = float(np.abs(g - w).max()) if w.size else 0.0
        assert err <= 2e-5 * scale, '%s: max err %.3g at scale %.3g' % (key, err, scale)
