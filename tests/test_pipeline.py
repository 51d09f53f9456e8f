"""PrefetchingIterator and defer_loss_readback under the reference's unchanged Trainer
(brainstorm/training/trainer.py:96-110): the same updates as with the plain iterator and
the blocking loss read, with the host round trips off the critical path."""
import numpy as np
import pytest

from conftest import needs_reference

pytestmark = [pytest.mark.gpu, needs_reference]


def _train(wrap_iter, defer, epochs=3):
    import brainstorm as bs
    from brainstorm_b200 import B200Handler, workloads
    from brainstorm_b200.pipeline import defer_loss_readback
    rs = np.random.RandomState(2)
    T, B, V = 5, 8, 9
    x = np.eye(V, dtype=np.float32)[rs.randint(0, V, (T, 5 * B))]
    tgt = rs.randint(0, V, (T, 5 * B, 1)).astype(np.int32)
    net, _, _ = workloads.lstm(time=T, batch=B, vocab=V, hidden=12, layers=1)
    net.set_handler(B200Handler(seed=1))
    deferred = defer_loss_readback(net) if defer else None
    per_update = []
    if not defer:                                   # the blocking read, update by update
        plain = net.get_loss_values

        def recording():
            v = plain()
            per_update.append(v['total_loss'])
            return v
        net.get_loss_values = recording
    trainer = bs.Trainer(bs.training.SgdStepper(learning_rate=0.1), verbose=False)
    trainer.add_hook(bs.hooks.StopOnNan())
    trainer.add_hook(bs.hooks.StopAfterEpoch(epochs))
    it = bs.data_iterators.Minibatches(B, shuffle=False, default=x, targets=tgt)
    trainer.train(net, wrap_iter(it))
    assert trainer.current_update_nr == 5 * epochs
    if defer:
        deferred.flush()
        per_update = list(deferred.history)
    return net.get('parameters'), per_update, list(trainer.logs['rolling_training']['total_loss'])


def test_prefetching_iterator_trains_bit_for_bit_like_the_plain_iterator():
    from brainstorm_b200.pipeline import PrefetchingIterator
    p0, l0, logs0 = _train(lambda it: it, False)
    p1, l1, logs1 = _train(PrefetchingIterator, False)
    assert np.array_equal(p0, p1)
    assert l0 == l1 and logs0 == logs1
    assert len(l0) >= 15


def test_deferred_loss_reports_every_update_one_call_late():
    from brainstorm_b200.pipeline import PrefetchingIterator
    p0, l0, logs0 = _train(lambda it: it, False)
    p1, l1, logs1 = _train(PrefetchingIterator, True)
    assert np.array_equal(p0, p1)                   # the updates themselves are untouched
    assert l1 == l0                                 # every call's true value, in the order of the calls
    assert logs1 != logs0 or len(set(l0)) <= 1      # what the Trainer saw while running was one call late


def test_prefetching_iterator_needs_the_device_handler_and_passes_shapes_through():
    import brainstorm as bs
    from brainstorm_b200.pipeline import PrefetchingIterator
    x = np.zeros((3, 4, 2), np.float32)
    it = PrefetchingIterator(bs.data_iterators.Minibatches(2, shuffle=False, default=x))
    assert it.data_shapes == {'default': (3, 4, 2)} and it.length == 2
    with pytest.raises(ValueError):
        next(it(handler=None))
