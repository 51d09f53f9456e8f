"""align_buffers: every hub of the reference's flat buffer on a 16-byte boundary, nothing
else changed (brainstorm/structure/buffers.py:48-55,69-96)."""
import numpy as np
import pytest

from conftest import needs_reference


def _offsets(net, base_of, addr_of):
    base = base_of(net._buffer_manager.full_buffer)
    return [(addr_of(b) - base) // 4 for b in net._buffer_manager.buffers]


@needs_reference
def test_aligned_hubs_train_exactly_like_packed_hubs_on_the_cpu_handler():
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200 import workloads
    from brainstorm_b200.layout import align_buffers, aligned_slices
    total, slices = aligned_slices([(3,), (5, 2), (1,), (0, 4), (7,)])
    assert [s.start for s in slices] == [0, 4, 16, 20, 20] and total == 27
    addr = lambda a: a.__array_interface__['data'][0]
    results = []
    for align in (False, True):
        net, data, stepper = workloads.highway_bn(batch=24, width=12, classes=5, blocks=2)
        net.set_handler(NumpyHandler(np.float32))
        if align:
            align_buffers(net)
        losses = workloads.train_steps(net, data, stepper(), 3)
        offs = _offsets(net, addr, addr)
        assert (set(o % 4 for o in offs) == {0}) == align or not align
        if not align:
            assert any(o % 4 for o in offs)           # the packed layout really is misaligned
        params = net.get('parameters')
        net.provide_external_data({k: v[:, :12] for k, v in data.items()})   # a resize keeps the parameters
        net.forward_pass()
        assert np.array_equal(net.get('parameters'), params)
        results.append((losses, params))
    assert results[0][0] == results[1][0]
    assert np.array_equal(results[0][1], results[1][1])


@pytest.mark.gpu
@needs_reference
@pytest.mark.parametrize('which', ['highway_bn', 'lstm', 'mlp'])
def test_aligned_hubs_train_like_packed_hubs_on_the_gpu(which):
    """Aligned operands take the 128-bit kernels and go to TMA without a staging copy.  The
    arithmetic per element is the same; only the order in which a softmax row or a column
    sum is added up depends on the kernel form, so results agree to rounding."""
    from brainstorm_b200 import B200Handler, workloads
    from brainstorm_b200.fused_lstm import fuse_lstm_layers
    from brainstorm_b200.layout import align_buffers
    build = {'highway_bn': lambda: workloads.highway_bn(batch=96, width=64, classes=10, blocks=3),
             'lstm': lambda: workloads.lstm(time=6, batch=64, vocab=45, hidden=128),
             'mlp': lambda: workloads.mlp(batch=100, hidden=256)}[which]
    results = []
    for align in (False, True):
        net, data, stepper = build()
        net.set_handler(B200Handler(seed=7, rng_mode='host', align_hubs=False))
        if which == 'lstm':
            fuse_lstm_layers(net)
        if align:
            align_buffers(net)
        losses = workloads.train_steps(net, data, stepper(), 3)
        if align:
            assert all(b.ptr % 16 == 0 for b in net._buffer_manager.buffers)
        results.append((losses, net.get('parameters'), net.get('gradients')))
    np.testing.assert_allclose(results[1][0], results[0][0], rtol=1e-6)
    for k in (1, 2):
        err = np.abs(results[1][k] - results[0][k]).max()
        assert err <= 2e-6 * np.abs(results[0][k]).max(), (k, err)


@pytest.mark.gpu
@needs_reference
def test_set_handler_alone_gives_aligned_hubs():
    """B200Handler(align_hubs=True), the default: the BufferManager gets the aligned resize
    when it asks the handler for its flat buffer inside net.set_handler; nothing else to call."""
    from brainstorm_b200 import B200Handler, workloads
    for align in (True, False):
        net, data, stepper = workloads.highway_bn(batch=24, width=12, classes=5, blocks=2)
        net.set_handler(B200Handler(seed=7, align_hubs=align))
        losses = workloads.train_steps(net, data, stepper(), 2)
        assert np.isfinite(losses).all()
        aligned = all(b.ptr % 16 == 0 for b in net._buffer_manager.buffers)
        assert aligned == align
        assert bool(getattr(net._buffer_manager, '_b200_aligned', False)) == align
