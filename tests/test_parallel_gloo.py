"""Host logic of the batch-sharded path on CPU: two gloo ranks, each running the
unchanged reference stack on its half of the batch with the sharded-sum mixin, must
reproduce the single-process run on the whole batch."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import needs_reference, ROOT

WORLD = 2


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _init(rank, port):
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    for p in (ROOT, os.path.join(ROOT, 'baseline', '_ref'), os.path.join(ROOT, 'tests')):
        if p not in sys.path:
            sys.path.insert(0, p)
    dist.init_process_group('gloo', rank=rank, world_size=WORLD)
    return dist


def _spawn(fn, *args):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(fn, args=(port,) + args, nprocs=WORLD, join=True)


# ---------------------------------------------------------------- op level
def _rank_sum_axis0(rank, port, out_dir):
    dist = _init(rank, port)
    from brainstorm_b200.parallel import Comm, AxisZeroAllReduce
    from oracle.numpy_oracle import OracleHandler, op_suite_inputs

    class Sharded(AxisZeroAllReduce, OracleHandler):
        pass

    h = Sharded(np.float32)
    h.set_comm(Comm(), 'sum')
    a = op_suite_inputs(64, 48, seed=9)['a']
    mine = a[rank * 32:(rank + 1) * 32]
    out = np.zeros((1, 48), np.float32)
    h.sum_t(mine, 0, out)
    other = np.zeros((32, 1), np.float32)
    h.sum_t(mine, 1, other)            # axis 1 stays local
    h.set_comm(Comm(), 'avg')
    avg = np.zeros((48,), np.float32)
    h.sum_t(mine, 0, avg)
    np.savez(os.path.join(out_dir, 'r%d.npz' % rank), s=out, row=other, avg=avg)
    dist.destroy_process_group()


def test_axis0_sum_is_completed_across_ranks(tmp_path):
    from oracle.numpy_oracle import op_suite_inputs
    _spawn(_rank_sum_axis0, str(tmp_path))
    a = op_suite_inputs(64, 48, seed=9)['a']
    for rank in range(WORLD):
        r = np.load(str(tmp_path / ('r%d.npz' % rank)))
        np.testing.assert_allclose(r['s'], a.sum(0, keepdims=True), rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(r['avg'], a.sum(0) / 2, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(r['row'], a[rank * 32:(rank + 1) * 32].sum(1, keepdims=True), rtol=1e-5, atol=1e-5)


# ---------------------------------------------------------------- network level
def _build(which):
    from brainstorm_b200 import workloads
    if which in ('highway_bn', 'highway_bn_fused_classes'):
        return workloads.highway_bn(batch=24, width=12, classes=5, blocks=2)
    if which == 'lstm':
        return workloads.lstm(time=4, batch=8, vocab=9, hidden=10)
    return workloads.mlp(batch=16, hidden=24, n_in=20, n_out=4)


def _rank_train(rank, port, which, out_dir, per_layer=True):
    dist = _init(rank, port)
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200 import parallel
    from brainstorm_b200.parallel import Comm, AxisZeroAllReduce, data_parallel, shard_batch
    # per layer (the form large networks get) or one all-reduce over the whole vector
    parallel.OVERLAP_MIN_BYTES = 0 if per_layer else (1 << 40)
    from brainstorm_b200.workloads import train_steps

    class ShardedNumpyHandler(AxisZeroAllReduce, NumpyHandler):
        pass

    net, data, stepper = _build(which)
    net.set_handler(ShardedNumpyHandler(np.float64))
    if which == 'highway_bn_fused_classes':
        # the fused layer classes and stepper on a handler that is not theirs: they run the reference's own chains,
        # whose column sums the mixin completes across the shards
        from brainstorm_b200.fused_layers import fuse_layers
        from brainstorm_b200.steppers import FusedSgdStepper
        assert len(fuse_layers(net)) == 9
        stepper = lambda: FusedSgdStepper(learning_rate=0.01)
    data_parallel(net, Comm(), axis0_reduce='avg' if which.startswith('highway_bn') else 'local')
    losses = train_steps(net, shard_batch(data, rank, WORLD), stepper(), 3)
    np.savez(os.path.join(out_dir, 'r%d.npz' % rank), p=net.get('parameters'),
             g=net.get('gradients'), losses=np.array(losses))
    dist.destroy_process_group()


@needs_reference
@pytest.mark.parametrize('per_layer', [True, False], ids=['per-layer', 'one-piece'])
@pytest.mark.parametrize('which', ['lstm', 'highway_bn', 'highway_bn_fused_classes'])
def test_sharded_training_equals_global_batch(tmp_path, which, per_layer):
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200.workloads import train_steps
    _spawn(_rank_train, which, str(tmp_path), per_layer)
    net, data, stepper = _build(which)
    net.set_handler(NumpyHandler(np.float64))
    losses = train_steps(net, data, stepper(), 3)
    ranks = [np.load(str(tmp_path / ('r%d.npz' % r))) for r in range(WORLD)]
    np.testing.assert_allclose(ranks[0]['p'], ranks[1]['p'], rtol=0, atol=0)   # replicas stay identical
    np.testing.assert_allclose(ranks[0]['p'], net.get('parameters'), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(ranks[0]['g'], net.get('gradients'), rtol=1e-8, atol=1e-11)
    # the global loss is the mean of the shard losses
    np.testing.assert_allclose((ranks[0]['losses'] + ranks[1]['losses']) / 2, losses, rtol=1e-9)
