"""Recorded steps (B200Handler.record / GraphedStepper): a replay must do exactly
what the same handler calls do one by one."""
import numpy as np
import pytest

from conftest import needs_reference


# ------------------------------------------------------------------ no GPU needed
def test_graph_end_without_begin_is_an_error_not_a_crash():
    from brainstorm_b200._lib import lib
    assert lib.b200_graph_end(None) != 0
    assert b'no graph is being recorded' in lib.b200_last_error()


def test_graph_launch_needs_an_initialised_library_or_a_handle():
    from brainstorm_b200._lib import lib
    assert lib.b200_graph_launch(0) != 0
    assert lib.b200_graph_destroy(0) == 0


# ------------------------------------------------------------------ GPU
@pytest.fixture(scope='module')
def H():
    from brainstorm_b200 import B200Handler
    return B200Handler(seed=5)


@pytest.mark.gpu
def test_replay_matches_the_same_calls_issued_one_by_one(H):
    rs = np.random.RandomState(0)
    x0 = rs.randn(96, 160).astype(np.float32)
    x1 = rs.randn(96, 160).astype(np.float32)
    w = H.create_from_numpy(rs.randn(160, 64).astype(np.float32))
    row = H.create_from_numpy(rs.randn(1, 64).astype(np.float32))
    x = H.create_from_numpy(x0)
    tmp, out = H.zeros((96, 160)), H.zeros((96, 64))
    total = H.zeros((1, 64))

    def calls():
        H.tanh(x, tmp)
        H.dot_mm(tmp, w, out)
        H.add_mv(out, row, out)
        H.sigmoid(out, out)
        H.sum_t(out, 0, total)

    calls()                                   # the ordinary way (also sizes work buffers)
    want0 = (H.get_numpy_copy(out), H.get_numpy_copy(total))
    H.set_from_numpy(x, x1)
    calls()
    want1 = (H.get_numpy_copy(out), H.get_numpy_copy(total))

    step = H.record(calls)
    assert step.kernels >= 5
    H.fill(out, -1.0)                         # nothing ran during the recording
    assert np.all(H.get_numpy_copy(out) == -1.0)
    for data, want in ((x0, want0), (x1, want1), (x0, want0)):
        H.set_from_numpy(x, data)
        H.fill(out, 0.0)
        step.launch()
        assert np.array_equal(H.get_numpy_copy(out), want[0])
        assert np.array_equal(H.get_numpy_copy(total), want[1])
    step.release()
    with pytest.raises(ValueError):
        step.launch()


@pytest.mark.gpu
def test_launch_counter_counts_the_replayed_kernels(H):
    from brainstorm_b200._lib import lib
    a, b = H.ones((8, 8)), H.zeros((8, 8))

    def calls():
        H.add_tt(a, b, b)
        H.mult_st(0.5, b, b)

    before = lib.b200_launch_count()
    step = H.record(calls)
    assert lib.b200_launch_count() == before          # recorded, not launched
    assert step.kernels == 2
    step.launch()
    assert lib.b200_launch_count() == before + 2 + 1   # + the replay-counter kernel
    assert np.all(H.get_numpy_copy(b) == 0.5)


@pytest.mark.gpu
def test_calls_that_wait_or_transfer_are_refused_and_the_handler_stays_usable(H):
    from brainstorm_b200 import B200Error
    a = H.ones((4, 4))

    for bad in (lambda: H.get_numpy_copy(a),
                lambda: H.set_from_numpy(a, np.zeros((4, 4), np.float32)),
                lambda: H.synchronize()):
        def calls():
            H.mult_st(2.0, a, a)
            bad()
        with pytest.raises(B200Error, match='being recorded'):
            H.record(calls)
        # the recording was discarded: nothing ran, ordinary calls work again
        assert np.all(H.get_numpy_copy(a) == 1.0)
    H.mult_st(2.0, a, a)
    assert np.all(H.get_numpy_copy(a) == 2.0)


@pytest.mark.gpu
def test_python_exception_inside_the_recorded_function_discards_the_recording(H):
    a = H.ones((4, 4))

    def calls():
        H.mult_st(3.0, a, a)
        raise KeyError('boom')

    with pytest.raises(KeyError):
        H.record(calls)
    assert np.all(H.get_numpy_copy(a) == 1.0)
    step = H.record(lambda: H.mult_st(3.0, a, a))     # a new recording can start
    step.launch()
    assert np.all(H.get_numpy_copy(a) == 3.0)


@pytest.mark.gpu
def test_temporaries_made_and_dropped_while_recording_survive_for_the_replays(H):
    rs = np.random.RandomState(1)
    x = H.create_from_numpy(rs.randn(300, 70).astype(np.float32))
    out = H.zeros((300, 70))

    def calls():
        t = H.zeros((300, 70))          # allocated inside the recording ...
        H.mult_tt(x, x, t)
        H.add_tt(t, x, out)
        del t                           # ... and released inside it

    step = H.record(calls)
    xs = H.get_numpy_copy(x)
    want = xs * xs + xs
    junk = [H.ones((300, 70)) for _ in range(8)]      # would reuse the temporary's memory if it had been freed
    for _ in range(3):
        H.fill(out, 0.0)
        step.launch()
        assert np.array_equal(H.get_numpy_copy(out), want)
    assert all(np.all(H.get_numpy_copy(j) == 1.0) for j in junk)


@pytest.mark.gpu
def test_every_replay_draws_a_new_dropout_mask(H):
    mask = H.zeros((512, 512))
    step = H.record(lambda: H.generate_probability_mask(mask, 0.3))
    seen = []
    for _ in range(3):
        step.launch()
        m = H.get_numpy_copy(mask)
        assert set(np.unique(m)) <= {0.0, 1.0}
        assert abs(m.mean() - 0.3) < 0.01
        seen.append(m)
    assert not np.array_equal(seen[0], seen[1])
    assert not np.array_equal(seen[1], seen[2])
    # and the ordinary call after the replays is a different stream again
    H.generate_probability_mask(mask, 0.3)
    assert not any(np.array_equal(H.get_numpy_copy(mask), s) for s in seen)


def _train(builder, wrap, steps, fused=False, **kw):
    from brainstorm_b200 import B200Handler
    net, data, stepper = builder(**kw)
    net.set_handler(B200Handler(seed=3))
    if fused:
        from brainstorm_b200.fused_lstm import fuse_lstm_layers
        fuse_lstm_layers(net)
    st = wrap(stepper())
    st.start(net)
    losses = []
    for i in range(steps):
        batch = {k: np.roll(v, i, axis=1) for k, v in data.items()}   # a new batch every step
        net.provide_external_data(batch)
        st.run()
        losses.append(float(net.get_loss_values()['total_loss']))
    return net.get('parameters'), losses, st


@pytest.mark.gpu
@needs_reference
@pytest.mark.parametrize('fused', [False, True])
def test_graphed_stepper_trains_the_lstm_bit_for_bit_like_the_plain_stepper(fused):
    from brainstorm_b200 import GraphedStepper, workloads
    kw = dict(time=6, batch=64, vocab=48, hidden=128)
    p_plain, l_plain, _ = _train(workloads.lstm, lambda s: s, 5, fused=fused, **kw)
    p_graph, l_graph, st = _train(workloads.lstm, GraphedStepper, 5, fused=fused, **kw)
    assert st._step is not None and st._step.kernels > 10     # steps 3.. were replays
    assert l_plain == l_graph
    assert np.array_equal(p_plain, p_graph)


@pytest.mark.gpu
@needs_reference
def test_recording_a_step_whose_lstm_layers_run_on_two_streams(monkeypatch):
    """The second LSTM layer of a stack runs on the library's side stream; a recording
    has to follow the fork and the join."""
    from brainstorm_b200 import GraphedStepper, fused_lstm, workloads
    monkeypatch.setattr(fused_lstm, 'PIECE', 2)
    kw = dict(time=6, batch=64, vocab=48, hidden=128)
    p_plain, l_plain, _ = _train(workloads.lstm, lambda s: s, 5, fused=True, **kw)
    p_graph, l_graph, st = _train(workloads.lstm, GraphedStepper, 5, fused=True, **kw)
    assert st._step is not None
    assert l_plain == l_graph
    assert np.array_equal(p_plain, p_graph)


@pytest.mark.gpu
@needs_reference
def test_graphed_stepper_records_again_when_a_frozen_scalar_or_the_batch_shape_changes():
    import brainstorm as bs
    from brainstorm_b200 import B200Handler, GraphedStepper, workloads
    net, data, _ = workloads.lstm(time=5, batch=16, vocab=20, hidden=32)
    ref, _, _ = workloads.lstm(time=5, batch=16, vocab=20, hidden=32)
    net.set_handler(B200Handler(seed=3))
    ref.set_handler(B200Handler(seed=3))
    plain = bs.training.SgdStepper(learning_rate=0.1)
    graphed = GraphedStepper(bs.training.SgdStepper(learning_rate=0.1))
    plain.start(ref)
    graphed.start(net)
    half = {k: v[:, :8] for k, v in data.items()}
    schedule = [(data, 0.1)] * 3 + [(data, 0.05)] * 3 + [(half, 0.05)] * 3 + [(data, 0.05)] * 2
    recordings = []
    for batch, lr in schedule:
        plain.learning_rate = lr
        graphed.stepper.learning_rate = lr
        for n, s in ((ref, plain), (net, graphed)):
            n.provide_external_data(batch)
            s.run()
        if graphed._step is not None and not any(r is graphed._step for r in recordings):
            recordings.append(graphed._step)
    assert len(recordings) >= 3
    assert np.array_equal(net.get('parameters'), ref.get('parameters'))


@pytest.mark.gpu
@needs_reference
def test_graphed_mlp_with_dropout_learns_and_uses_fresh_masks():
    from brainstorm_b200 import GraphedStepper, workloads
    _, losses, st = _train(workloads.mlp, GraphedStepper, 30, batch=100)
    assert st._step is not None
    assert np.isfinite(losses).all()
    assert np.mean(losses[-5:]) < np.mean(losses[:5])
    # the masks of the replayed steps differ from step to step
    net, data, stepper = workloads.mlp(batch=100)
    from brainstorm_b200 import B200Handler
    net.set_handler(B200Handler(seed=3))
    gs = GraphedStepper(stepper())
    gs.start(net)
    masks = []
    name = [n for n in net.layers if 'ropout' in n][0]
    for _ in range(5):
        net.provide_external_data(data)
        gs.run()
        masks.append(net.get('%s.internals.mask' % name))
    assert not np.array_equal(masks[-1], masks[-2])


@pytest.mark.gpu
@needs_reference
def test_reference_trainer_runs_on_a_graphed_stepper():
    """The reference's Trainer with hooks and a Minibatches iterator, its stepper wrapped in
    GraphedStepper: same logs and parameters as with the plain stepper, bit for bit, and
    the wrapper survives the Trainer's description machinery."""
    import brainstorm as bs
    from brainstorm.describable import get_description
    from brainstorm_b200 import B200Handler, GraphedStepper, workloads
    rs = np.random.RandomState(2)
    T, B, V = 5, 8, 9
    x = np.eye(V, dtype=np.float32)[rs.randint(0, V, (T, 4 * B))]
    tgt = rs.randint(0, V, (T, 4 * B, 1)).astype(np.int32)
    results = []
    for wrap in (lambda s: s, GraphedStepper):
        net, _, _ = workloads.lstm(time=T, batch=B, vocab=V, hidden=12, layers=1)
        net.set_handler(B200Handler(seed=1))
        stepper = wrap(bs.training.SgdStepper(learning_rate=0.1))
        trainer = bs.Trainer(stepper, verbose=False)
        trainer.add_hook(bs.hooks.StopOnNan())
        trainer.add_hook(bs.hooks.StopAfterEpoch(3))
        trainer.train(net, bs.data_iterators.Minibatches(B, shuffle=False, default=x, targets=tgt))
        assert trainer.current_update_nr == 12
        results.append((list(trainer.logs['rolling_training']['total_loss']), net.get('parameters')))
    assert stepper._step is not None and stepper._step.kernels > 10
    assert get_description(stepper)['@type'] == 'GraphedStepper'
    assert results[0][0] == results[1][0]
    assert np.array_equal(results[0][1], results[1][1])


@pytest.mark.gpu
@needs_reference
def test_eager_work_between_replays_does_not_pull_memory_from_under_the_recording():
    """A recording bakes in the addresses of work arrays it did not get from the caller: the
    split-K partials of the GEMMs, the handler's reduction scratch, the arrays one fused
    LSTM layer hands to the next.  A Trainer with a validation monitor runs ordinary
    forward passes between replays, and any other ordinary call may need a larger work
    array.  None of that may free memory a replay still writes."""
    from brainstorm_b200 import B200Handler, GraphedStepper, workloads
    from brainstorm_b200.fused_lstm import fuse_lstm_layers
    kw = dict(time=64, batch=16, vocab=20, hidden=32)      # 64 timesteps: two pieces, so layers hand work arrays over
    results = []
    for wrap in (lambda s: s, GraphedStepper):
        net, data, stepper = workloads.lstm(**kw)
        H = B200Handler(seed=3)
        net.set_handler(H)
        fuse_lstm_layers(net)
        st = wrap(stepper())
        st.start(net)
        rs = np.random.RandomState(9)
        big_a = H.create_from_numpy(rs.randn(128, 4096).astype(np.float32))
        big_b = H.create_from_numpy(rs.randn(256, 4096).astype(np.float32))
        tall = H.create_from_numpy(rs.randn(4096, 3000).astype(np.float32))
        losses = []
        for i in range(6):
            batch = {k: np.roll(v, i, axis=1) for k, v in data.items()}
            net.provide_external_data(batch)
            st.run()
            losses.append(float(net.get_loss_values()['total_loss']))
            if i == 2:        # steps 1 and 2 were the recording and its first replay
                net.forward_pass(training_pass=False)          # takes and drops the handed-over arrays
                out = H.zeros((128, 256))
                H.dot_mm(big_a, big_b, out, transb=True)       # split-K: a much larger partial buffer
                col = H.zeros((1, 3000))
                H.sum_t(tall, 0, col)                          # needs more scratch than the step did
                junk = [H.allocate((1 << 18,)) for _ in range(24)]
                for j in junk:                                 # whatever was freed is reused and poisoned
                    H.fill(j, float('nan'))
                H.synchronize()
                del junk
        results.append((net.get('parameters'), losses))
        if wrap is GraphedStepper:
            assert st._step is not None and len(st._step._keep) >= 1
    assert results[0][1] == results[1][1]
    assert np.isfinite(results[1][0]).all()
    assert np.array_equal(results[0][0], results[1][0])


# ------------------------------------------------------------------ GraphedStepper logic, no GPU
class _FakeStep(object):
    def __init__(self):
        self.launches, self.released = 0, False

    def launch(self):
        assert not self.released
        self.launches += 1

    def release(self):
        self.released = True


class _FakeArray(object):
    def __init__(self, ptr):
        self.ptr = ptr


class _FakeManager(object):
    def __init__(self):
        self.full_buffer, self.time_size, self.batch_size = _FakeArray(4096), 5, 16


class _FakeNet(object):
    def __init__(self):
        self._buffer_manager = _FakeManager()
        self.handler = type('H', (), {'_comm': None})()


class _FakeStepper(object):
    def __init__(self):
        self.learning_rate, self._runs, self.net = 0.1, 0, None   # scalars without '_' are part of the key

    def start(self, net):
        self.net = net

    def run(self):
        self._runs += 1


def _graphed(monkeypatch):
    from brainstorm_b200 import graph
    made = []

    def fake_record(fn, *a, **k):
        k.pop('handler', None)           # whose work arrays the recording keeps alive
        fn(*a, **k)                      # a recording runs the calls once (without executing them)
        made.append(_FakeStep())
        return made[-1]

    monkeypatch.setattr(graph, 'record', fake_record)
    inner = _FakeStepper()
    gs = graph.GraphedStepper(inner, eager_steps=1)
    net = _FakeNet()
    gs.start(net)
    return gs, inner, net, made


def test_graphed_stepper_runs_once_eagerly_then_records_then_replays(monkeypatch):
    gs, inner, net, made = _graphed(monkeypatch)
    for _ in range(5):
        gs.run()
    assert inner._runs == 2               # the eager step and the recorded one
    assert len(made) == 1 and made[0].launches == 4


def test_graphed_stepper_records_again_after_a_change_of_scalar_shape_or_buffer(monkeypatch):
    gs, inner, net, made = _graphed(monkeypatch)
    for _ in range(3):
        gs.run()
    inner.learning_rate = 0.05
    for _ in range(3):
        gs.run()
    net._buffer_manager.batch_size = 8
    for _ in range(3):
        gs.run()
    net._buffer_manager.full_buffer = _FakeArray(8192)
    for _ in range(3):
        gs.run()
    assert len(made) == 4
    assert [m.released for m in made] == [True, True, True, False]
    assert all(m.launches == 2 for m in made)       # per setting: eager, record + launch, launch
    assert inner._runs == 8


def test_graphed_stepper_passes_through_under_data_parallelism(monkeypatch):
    gs, inner, net, made = _graphed(monkeypatch)
    net.handler._comm = object()
    for _ in range(4):
        gs.run()
    assert inner._runs == 4 and not made
