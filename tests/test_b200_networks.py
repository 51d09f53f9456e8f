"""The reference's own layers, Network and steppers, unchanged, on B200Handler
(installed through Network.set_handler) against the same stack on NumpyHandler."""
import numpy as np
import pytest

import parity
from conftest import needs_reference

pytestmark = [pytest.mark.gpu, needs_reference]


def _pair(builder, fused=False, prepare=None, **kw):
    import brainstorm as bs
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200 import B200Handler
    net_cpu, data, stepper = builder(**kw)
    net_cpu.set_handler(NumpyHandler(np.float32, seed=77))
    net_gpu, _, _ = builder(**kw)
    net_gpu.set_handler(B200Handler(seed=77, rng_mode='host'))
    if fused:
        from brainstorm_b200.fused_lstm import fuse_lstm_layers
        assert len(fuse_lstm_layers(net_gpu)) == kw.get('layers', 2)
    if prepare is not None:
        prepare(net_gpu)
    p_cpu = net_cpu.get('parameters')
    p_gpu = net_gpu.get('parameters')
    assert np.array_equal(p_cpu, p_gpu)
    return net_cpu, net_gpu, data, stepper


def _close(got, want, rtol, what):
    scale = np.abs(want).max() + 1e-30
    err = np.abs(got - want).max()
    assert err <= rtol * scale, '%s: max err %.3g vs scale %.3g' % (what, err, scale)


def _close_l2(got, want, rtol, what):
    err = np.linalg.norm((got - want).ravel())
    ref = np.linalg.norm(want.ravel()) + 1e-30
    assert err <= rtol * ref, '%s: L2 err %.3g vs norm %.3g' % (what, err, ref)


def _relu_flips(net_cpu, net_gpu):
    """Units of the ReLU layers that are switched on on one backend and off on the other:
    a pre-activation within rounding distance of zero may fall on either side."""
    flips = 0
    for lname, layer in net_cpu.layers.items():
        if getattr(layer, 'activation', None) == 'rel':
            path = lname + '.outputs.default'
            flips += int(((net_cpu.get(path) > 0) != (net_gpu.get(path) > 0)).sum())
    return flips


# Observed on B200 (max error over max magnitude): gradients 1e-7 .. 1.7e-6, parameters after
# the optimiser steps 4e-8 .. 2.1e-7, losses 0 .. 1.8e-7.  The bounds are ten times that.
GRAD_TOL, PARAM_TOL, LOSS_TOL = 2e-5, 2e-6, 2e-6


def _check_training(builder, steps, grad_tol=GRAD_TOL, param_tol=PARAM_TOL, compare=None, fused=False,
                    after_first_pass=None, prepare=None, **kw):
    compare = compare or _close
    from brainstorm_b200.workloads import train_steps
    net_cpu, net_gpu, data, stepper = _pair(builder, fused=fused, prepare=prepare, **kw)
    # one forward/backward: loss, every gradient
    for net in (net_cpu, net_gpu):
        net.provide_external_data(data)
        net.forward_pass(training_pass=True)
        net.backward_pass()
    l_cpu = float(net_cpu.get_loss_values()['total_loss'])
    l_gpu = float(net_gpu.get_loss_values()['total_loss'])
    assert abs(l_cpu - l_gpu) <= 1e-5 * abs(l_cpu), (l_cpu, l_gpu)
    compare(net_gpu.get('gradients'), net_cpu.get('gradients'), grad_tol, 'gradients')
    if after_first_pass is not None:     # buffer-by-buffer checks while both sides still hold the same parameters
        after_first_pass(net_cpu, net_gpu)
    # a few optimiser steps: losses and parameters stay together
    lc = train_steps(net_cpu, data, stepper(), steps)
    lg = train_steps(net_gpu, data, stepper(), steps)
    np.testing.assert_allclose(lg, lc, rtol=LOSS_TOL)
    compare(net_gpu.get('parameters'), net_cpu.get('parameters'), param_tol, 'parameters')
    return net_cpu, net_gpu


def _lstm_buffers(T):
    """Every internal, output, input delta and gradient of the LSTM layers, element by
    element, against sums of |terms| (parity.lstm_net_checks)."""
    def check(net_cpu, net_gpu):
        worst = {}
        parity.lstm_net_checks(net_cpu, net_gpu, T, worst)
        parity.report(worst, 'LSTM buffers')
    return check


def test_mlp_dropout_fc_softmax_momentum():
    """The ReLU network has kinks: where a pre-activation lies within rounding distance of
    zero the two backends may disagree on which side, and the unit's whole delta then
    appears in, or vanishes from, the gradient (observed: one unit of 240 000, moving the
    gradient by 2.3e-3 of its norm).  So the flipped units are counted, and the gradient
    bound allows for them and for nothing else; parameters and losses must agree closely
    either way (the masks come from the same host generator on both sides)."""
    from brainstorm_b200 import workloads
    seen = {}

    def count(net_cpu, net_gpu):
        seen['flips'] = _relu_flips(net_cpu, net_gpu)
        assert seen['flips'] <= 4, seen

    def gradients(got, want, tol, what):
        if what == 'gradients':
            flips = _relu_flips(*seen['nets'])
            tol = tol + 3e-3 * flips
        _close_l2(got, want, tol, what)

    net_cpu, net_gpu, data, stepper = _pair(workloads.mlp, batch=100)
    seen['nets'] = (net_cpu, net_gpu)
    for net in (net_cpu, net_gpu):
        net.provide_external_data(data)
        net.forward_pass(training_pass=True)
        net.backward_pass()
    count(net_cpu, net_gpu)
    gradients(net_gpu.get('gradients'), net_cpu.get('gradients'), GRAD_TOL, 'gradients')
    from brainstorm_b200.workloads import train_steps
    lc = train_steps(net_cpu, data, stepper(), 3)
    lg = train_steps(net_gpu, data, stepper(), 3)
    np.testing.assert_allclose(lg, lc, rtol=LOSS_TOL)
    _close_l2(net_gpu.get('parameters'), net_cpu.get('parameters'), 1e-6, 'parameters')


def test_lstm_two_layers_sgd():
    from brainstorm_b200 import workloads
    _check_training(workloads.lstm, steps=2, after_first_pass=_lstm_buffers(7), time=7, batch=9, vocab=23, hidden=32)


def test_lstm_aligned_sizes_use_tensor_cores():
    from brainstorm_b200 import workloads
    _check_training(workloads.lstm, steps=2, after_first_pass=_lstm_buffers(6), time=6, batch=64, vocab=48, hidden=128)


@pytest.mark.parametrize('shape', [dict(time=7, batch=9, vocab=23, hidden=32),
                                   dict(time=6, batch=64, vocab=48, hidden=128),
                                   dict(time=1, batch=5, vocab=7, hidden=12),
                                   dict(time=12, batch=128, vocab=205, hidden=200),
                                   dict(time=4, batch=3, vocab=5, hidden=5)],
                         ids=['ragged', 'aligned', 'one-step', 'wide', 'odd'])
def test_fused_lstm_layer_matches_reference_layer(shape):
    """The fused layer on the GPU against the reference's own LstmLayerImpl on
    NumpyHandler: loss, every gradient, parameters after SGD steps -- and every
    one of the twenty internal buffers plus outputs and input deltas."""
    from brainstorm_b200 import workloads
    _check_training(workloads.lstm, steps=2, fused=True, after_first_pass=_lstm_buffers(shape['time']), **shape)


@pytest.mark.parametrize('piece,shape', [(2, dict(time=7, batch=9, vocab=23, hidden=32)),
                                         (3, dict(time=12, batch=128, vocab=205, hidden=200)),
                                         (2, dict(time=6, batch=64, vocab=48, hidden=128, layers=3))],
                         ids=['ragged', 'wide', 'three-layers'])
def test_stacked_fused_lstm_layers_side_by_side(piece, shape, monkeypatch):
    """With pieces shorter than the sequence the second LSTM layer runs on the second
    stream, piece by piece behind the first one (forward) and ahead of it (backward).
    Same checks as above, and the overlap must really have been taken."""
    from brainstorm_b200 import fused_lstm, workloads
    from brainstorm_b200._lib import lib
    monkeypatch.setattr(fused_lstm, 'PIECE', piece)
    used = []
    real = lib.b200_use_stream
    monkeypatch.setattr(lib, 'b200_use_stream', lambda i: (used.append(i), real(i))[1])
    _check_training(workloads.lstm, steps=2, fused=True, after_first_pass=_lstm_buffers(shape['time']), **shape)
    assert used.count(1) >= 2 * 3            # forward and backward of (at least) three passes


def test_fused_lstm_carries_context_between_calls():
    """Truncated BPTT: forward passes with context hand y and the cell state from
    one chunk to the next (network.py:405-428); the fused layer must read them."""
    from brainstorm_b200 import workloads
    net_cpu, net_gpu, data, _ = _pair(workloads.lstm, fused=True, time=5, batch=6, vocab=11, hidden=16)
    outs = []
    for net in (net_cpu, net_gpu):
        net.provide_external_data(data)
        net.forward_pass(training_pass=True)
        ctx = net.get_context()
        net.forward_pass(training_pass=True, context=ctx)
        outs.append(net.get('Output_projection.outputs.default'))
    _close(outs[1], outs[0], 2e-6, 'outputs of the second chunk')


def test_highway_batchnorm_stack():
    from brainstorm_b200 import workloads
    _check_training(workloads.highway_bn, steps=2, grad_tol=5e-6, batch=96, width=64, classes=10, blocks=3)


def _two_sources(batch=6, time=3, n_in=12, n_out=5, seed=42, data_seed=0):
    """Two layers feeding one input: their outputs (and output deltas) are feature
    slices of one hub, i.e. row-pitched views (buffer_structure.py:232-245)."""
    import brainstorm as bs
    bs.global_rnd.set_seed(seed)
    inp, fc = bs.tools.get_in_out_layers('classification', (n_in,), n_out)
    inp >> bs.layers.FullyConnected(7, name='A', activation='tanh') >> fc
    inp >> bs.layers.FullyConnected(9, name='B', activation='sigmoid') >> fc
    net = bs.Network.from_layer(fc)
    net.initialize(bs.initializers.Gaussian(0.1))
    rs = np.random.RandomState(data_seed)
    data = {'default': rs.randn(time, batch, n_in).astype(np.float32),
            'targets': rs.randint(0, n_out, (time, batch, 1)).astype(np.int32)}
    return net, data, lambda: bs.training.SgdStepper(learning_rate=0.1)


def test_hub_with_two_sources_hands_out_strided_views():
    net_cpu, net_gpu = _check_training(_two_sources, steps=3, grad_tol=2e-6, param_tol=1e-6)
    assert not net_gpu.buffer['A'].outputs.default.is_contiguous
    assert not net_gpu.buffer['B'].output_deltas.default.is_contiguous
    for path in ('A.outputs.default', 'B.outputs.default', 'A.output_deltas.default', 'B.output_deltas.default'):
        _close(net_gpu.get(path), net_cpu.get(path), 2e-6, path)


def test_handler_is_describable_and_weight_modifier_runs():
    import brainstorm as bs
    from brainstorm.describable import get_description, create_from_description
    from brainstorm_b200 import B200Handler, workloads
    h = B200Handler(seed=5)
    d = get_description(h)
    assert d == {'@type': 'B200Handler'}
    assert isinstance(create_from_description(d), B200Handler)
    net_cpu, net_gpu, data, stepper = _pair(workloads.mlp, batch=20, hidden=64)
    for net in (net_cpu, net_gpu):   # examples/mnist_pi.py:42
        net.set_weight_modifiers({'FC': {'W': bs.value_modifiers.ConstrainL2Norm(0.5)}})
        net.apply_weight_modifiers()
    _close(net_gpu.get('parameters'), net_cpu.get('parameters'), 1e-5, 'constrained parameters')


def test_reference_debug_handler_wraps_b200_handler():
    """The reference's DebugHandler (shape / finite checks around every op,
    brainstorm/handlers/debug_handler.py:61) on top of B200Handler: the array
    contract it relies on (shape, size, reshape, indexing) must hold."""
    from brainstorm.handlers.debug_handler import DebugHandler
    from brainstorm_b200 import B200Handler, workloads
    from brainstorm_b200.workloads import train_steps
    net, data, stepper = workloads.lstm(time=4, batch=3, vocab=6, hidden=5)
    net.set_handler(DebugHandler(B200Handler(seed=1, rng_mode='host')))
    losses = train_steps(net, data, stepper(), 2)
    assert np.isfinite(losses).all() and losses[1] < losses[0]
    net2, data2, stepper2 = workloads.highway_bn(batch=12, width=8, classes=3, blocks=1)
    net2.set_handler(DebugHandler(B200Handler(seed=1, rng_mode='host')))
    assert np.isfinite(train_steps(net2, data2, stepper2(), 2)).all()


def test_reference_trainer_with_iterators_and_hooks():
    """The reference's Trainer loop, Minibatches iterator, momentum stepper and
    hooks (MonitorLoss on a validation iterator, StopOnNan -> is_fully_finite,
    StopAfterEpoch), unchanged, on B200Handler vs NumpyHandler."""
    import brainstorm as bs
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200 import B200Handler, workloads
    rs = np.random.RandomState(4)
    x = rs.uniform(0, 1, (1, 64, 20)).astype(np.float32)
    t = rs.randint(0, 4, (1, 64, 1)).astype(np.int32)
    logs = []
    for handler in (NumpyHandler(np.float32, seed=9), B200Handler(seed=9, rng_mode='host')):
        bs.global_rnd.set_seed(11)
        net, _, _ = workloads.mlp(batch=16, hidden=24, n_in=20, n_out=4)
        net.set_handler(handler)
        trainer = bs.Trainer(bs.training.MomentumStepper(learning_rate=0.1, momentum=0.9), verbose=False)
        trainer.add_hook(bs.hooks.MonitorLoss('valid', name='valid_loss', verbose=False))
        trainer.add_hook(bs.hooks.StopOnNan())
        trainer.add_hook(bs.hooks.StopAfterEpoch(3))
        trainer.train(net, bs.data_iterators.Minibatches(16, shuffle=False, default=x, targets=t),
                      valid=bs.data_iterators.Minibatches(32, shuffle=False, default=x, targets=t))
        logs.append((trainer.logs['rolling_training']['total_loss'], trainer.logs['valid_loss']['total_loss'],
                     net.get('parameters')))
        assert trainer.current_epoch_nr == 3 and trainer.current_update_nr == 12
    np.testing.assert_allclose(logs[1][0], logs[0][0], rtol=2e-6)
    np.testing.assert_allclose(logs[1][1], logs[0][1], rtol=2e-6)
    _close_l2(logs[1][2], logs[0][2], 2e-6, 'parameters after 3 epochs')


def test_device_one_hot_iterator_matches_host_one_hot():
    """Trainer + DeviceOneHot (indices uploaded, one-hot rows written on the GPU)
    against Trainer + the reference's host OneHot on NumpyHandler."""
    import brainstorm as bs
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200 import B200Handler, workloads
    from brainstorm_b200.iterators import DeviceOneHot
    rs = np.random.RandomState(2)
    T, B, V = 5, 8, 9
    idx = rs.randint(0, V, (T, 2 * B, 1))
    tgt = rs.randint(0, V, (T, 2 * B, 1)).astype(np.int32)
    results = []
    for handler, onehot in ((NumpyHandler(np.float32), bs.data_iterators.OneHot),
                            (B200Handler(seed=1), DeviceOneHot)):
        net, _, _ = workloads.lstm(time=T, batch=B, vocab=V, hidden=12, layers=1)
        net.set_handler(handler)
        trainer = bs.Trainer(bs.training.SgdStepper(learning_rate=0.1), verbose=False)
        trainer.add_hook(bs.hooks.StopAfterEpoch(2))
        it = onehot(bs.data_iterators.Minibatches(B, shuffle=False, default=idx, targets=tgt), {'default': V})
        trainer.train(net, it)
        results.append((trainer.logs['rolling_training']['total_loss'], net.get('parameters')))
    np.testing.assert_allclose(results[1][0], results[0][0], rtol=2e-6)
    _close(results[1][1], results[0][1], 2e-6, 'parameters')
