"""The fused Highway / BatchNorm / FullyConnected layers (brainstorm_b200/fused_layers.py) against the
reference's own layer code on the same handler (bit for bit) and on NumpyHandler (to rounding)."""
import numpy as np
import pytest

from conftest import needs_reference

pytestmark = [needs_reference]


def _snapshot(net):
    """Every buffer the layers leave behind, as host copies."""
    out = {'parameters': net.get('parameters'), 'gradients': net.get('gradients')}
    for name, layer in net.layers.items():
        buffers = net.buffer[name]
        for kind in ('outputs', 'internals', 'input_deltas'):
            group = buffers[kind]
            for key in group.keys():
                out['%s.%s.%s' % (name, kind, key)] = net.handler.get_numpy_copy(group[key])
    return out


def _nets(**kw):
    from brainstorm_b200 import B200Handler, workloads
    from brainstorm_b200.fused_layers import fuse_layers
    plain, data, stepper = workloads.highway_bn(**kw)
    plain.set_handler(B200Handler(seed=5, rng_mode='host'))
    fused, _, _ = workloads.highway_bn(**kw)
    fused.set_handler(B200Handler(seed=5, rng_mode='host'))
    swapped = fuse_layers(fused)
    assert len(swapped) == 4 * kw['blocks'] + 1
    return plain, fused, data, stepper


def test_fuse_layers_swaps_classes_and_keeps_the_layout():
    import brainstorm as bs
    from brainstorm_b200 import workloads
    from brainstorm_b200.fused_layers import (fuse_layers, FusedHighwayLayerImpl, FusedBatchNormLayerImpl,
                                              FusedFullyConnectedLayerImpl)
    net, data, stepper = workloads.highway_bn(batch=8, width=8, classes=3, blocks=2)
    before = {n: (l.parameter_shapes, l.internal_shapes, l.out_shapes) for n, l in net.layers.items()}
    from brainstorm.describable import get_description
    described = get_description(net)
    names = fuse_layers(net)
    assert get_description(net) == described       # a saved network does not tell which classes ran it
    assert sorted(names) == sorted(n for n in net.layers if n[0] in 'HTB' or n == 'Output_projection')
    kinds = {type(l) for l in net.layers.values()}
    assert {FusedHighwayLayerImpl, FusedBatchNormLayerImpl, FusedFullyConnectedLayerImpl} <= kinds
    assert before == {n: (l.parameter_shapes, l.internal_shapes, l.out_shapes) for n, l in net.layers.items()}
    assert fuse_layers(net) == []          # nothing left to swap
    # on another handler the fused classes run the reference's own code
    ref, _, _ = workloads.highway_bn(batch=8, width=8, classes=3, blocks=2)
    for n in (net, ref):
        n.provide_external_data(data)
        n.forward_pass(training_pass=True)
        n.backward_pass()
    assert np.array_equal(net.get('gradients'), ref.get('gradients'))


@pytest.mark.gpu
@pytest.mark.parametrize('batch,width,blocks', [(96, 64, 3), (4, 4, 1), (300, 128, 2), (6000, 256, 1), (24, 30, 2), (8192, 4096, 2)])
def test_fused_layers_give_the_bits_of_the_handler_call_chains(batch, width, blocks):
    from brainstorm_b200.workloads import train_steps
    plain, fused, data, stepper = _nets(batch=batch, width=width, classes=10, blocks=blocks)
    for training in (True, False):
        for net in (plain, fused):
            net.provide_external_data(data)
            net.forward_pass(training_pass=training)
            if training:
                net.backward_pass()
        a, b = _snapshot(plain), _snapshot(fused)
        assert a.keys() == b.keys()
        for key in a:
            if not training and ('deltas' in key or key == 'gradients'):
                continue
            assert np.array_equal(a[key], b[key], equal_nan=True), '%s differs (training_pass=%s)' % (key, training)
    la = train_steps(plain, data, stepper(), 3)
    lb = train_steps(fused, data, stepper(), 3)
    assert la == lb
    assert np.array_equal(plain.get('parameters'), fused.get('parameters'))


@pytest.mark.gpu
def test_fused_layers_against_numpy_handler():
    from brainstorm_b200 import workloads
    from brainstorm_b200.fused_layers import fuse_layers
    from test_b200_networks import _check_training
    _check_training(workloads.highway_bn, steps=2, grad_tol=5e-6, prepare=fuse_layers,
                    batch=96, width=64, classes=10, blocks=3)


@pytest.mark.gpu
def test_fused_layers_in_a_recorded_step():
    """A step with fused layers replayed from a recording follows the eager steps bit for bit."""
    from brainstorm_b200 import GraphedStepper
    from brainstorm_b200.workloads import train_steps
    import brainstorm as bs
    plain, fused, data, stepper = _nets(batch=64, width=64, classes=10, blocks=2)
    want = train_steps(plain, data, stepper(), 5)
    got = train_steps(fused, data, GraphedStepper(bs.training.SgdStepper(learning_rate=0.01)), 5)
    assert want == got
    assert np.array_equal(plain.get('parameters'), fused.get('parameters'))


@pytest.mark.gpu
@pytest.mark.parametrize('act', ['sigmoid', 'tanh', 'rel', 'el', 'linear'])
@pytest.mark.parametrize('rows,cols,ld', [(1, 4, 4), (37, 64, 64), (37, 64, 72), (513, 1028, 1028), (300, 12, 40)])
def test_bias_act_gives_the_bits_of_add_mv_then_the_activation(act, rows, cols, ld):
    """b200_bias_act against the two handler calls it replaces (fully_connected_layer.py:61-62),
    on rows with and without a pitch."""
    from brainstorm_b200 import B200Handler
    from brainstorm_b200._lib import lib, check
    from brainstorm_b200.fused_layers import _ACT
    H = B200Handler()
    rs = np.random.RandomState(rows * 131 + cols)
    x = (3 * rs.randn(rows, ld)).astype(np.float32)
    bias = rs.randn(cols).astype(np.float32)
    want = H.create_from_numpy(x)[:, :cols]
    H.add_mv(want, H.create_from_numpy(bias.reshape(1, cols)), want)
    H.inplace_act_func[act](want)
    got = H.create_from_numpy(x)
    check(lib.b200_bias_act(got.ptr, H.create_from_numpy(bias).ptr, rows, cols, ld, _ACT[act]))
    got = H.get_numpy_copy(got)
    assert np.array_equal(got[:, :cols], H.get_numpy_copy(want))
    assert np.array_equal(got[:, cols:], x[:, cols:])            # the padding of pitched rows is untouched


def _sgd_pair(make_handler):
    import brainstorm as bs
    from brainstorm_b200 import workloads
    from brainstorm_b200.steppers import FusedSgdStepper
    from brainstorm_b200.workloads import train_steps
    out = []
    for cls in (bs.training.SgdStepper, FusedSgdStepper):
        net, data, _ = workloads.highway_bn(batch=24, width=16, classes=5, blocks=2)
        net.set_handler(make_handler())
        losses = train_steps(net, data, cls(learning_rate=0.07), 4)
        out.append((losses, net.get('parameters')))
    assert out[0][0] == out[1][0]
    assert np.array_equal(out[0][1], out[1][1])


def test_fused_sgd_stepper_gives_the_bits_of_sgd_stepper_on_numpy_handler():
    from brainstorm.handlers import NumpyHandler
    _sgd_pair(lambda: NumpyHandler(np.float32))


@pytest.mark.gpu
def test_fused_sgd_stepper_gives_the_bits_of_sgd_stepper():
    from brainstorm_b200 import B200Handler
    _sgd_pair(lambda: B200Handler())
