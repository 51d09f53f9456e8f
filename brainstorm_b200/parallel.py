"""Batch-axis data parallelism for networks that run on a handler.

The reference has no distributed code at all; this module adds the one strategy
the handler path shards on: every activation buffer is (time, batch, features), so
each rank (one process per GPU) runs the unchanged network on its own slice of the
batch, and only the contractions over the batch axis need an exchange:

* **Gradients** -- one all-reduce (average) of the single contiguous gradient
  vector (``net.buffer.gradients``) after every backward pass.  The local Loss
  layer scales deltas by 1/B_local (brainstorm/layers/loss_layer.py:56), so the
  average of the local gradients is the gradient of the global batch.
* **Batch statistics** -- with ``axis0_reduce='avg'`` every ``sum_t(a, axis=0)`` is
  completed by an all-reduce (average) of its small result.  BatchNorm divides its
  sums by the *local* batch size (batch_normalization_layer.py:63,117), so averaged
  sums give exactly the global mean / variance, also where the backward pass reuses
  them inside the delta formula (:130-151).  ``'sum'`` gives the plain global sum
  (the op-suite benchmark); ``'local'`` (default) exchanges nothing.

The rules are pure arithmetic and backend independent: ``AxisZeroAllReduce`` is a
mixin for any handler class and ``Comm`` works on numpy arrays over ``gloo`` (used
by the CPU tests with world size 2) and on device arrays over NCCL.
"""
from __future__ import annotations

import numpy as np


class Comm(object):
    """All-reduce over ``torch.distributed`` (initialised by the caller)."""

    def __init__(self):
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError('torch.distributed is not initialised')
        self.dist = dist
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self._stream = None

    def _device_stream(self):
        # NCCL work is ordered after, and the library's later kernels after it, by
        # presenting the library stream to torch as the current stream: no host sync.
        if self._stream is None:
            import torch
            from ._lib import lib
            self._stream = torch.cuda.ExternalStream(lib.b200_stream())
        return self._stream

    def allreduce(self, arr, op='sum'):
        """In-place all-reduce of a numpy array (gloo) or a device array (NCCL)."""
        import torch
        if self.world == 1:
            return
        if isinstance(arr, np.ndarray):
            if arr.ndim == 0:
                buf = arr.reshape(1)
            else:
                buf = arr
            if not buf.flags.c_contiguous:
                tmp = np.ascontiguousarray(buf)
                self.allreduce(tmp, op)
                buf[...] = tmp
                return
            t = torch.from_numpy(buf)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
            if op == 'avg':
                buf /= buf.dtype.type(self.world)
            return
        if not arr.is_contiguous:
            raise NotImplementedError('all-reduce of a strided device view')
        if arr.size == 0:
            return
        flat = arr.reshape((arr.size,))
        with torch.cuda.stream(self._device_stream()):
            t = torch.as_tensor(flat, device='cuda')
            self.dist.all_reduce(t, op=self.dist.ReduceOp.AVG if op == 'avg' else self.dist.ReduceOp.SUM)


class AxisZeroAllReduce(object):
    """Handler mixin: completes ``sum_t(axis=0)`` across the batch shards.

        class ShardedNumpyHandler(AxisZeroAllReduce, NumpyHandler): pass

    ``B200Handler`` has the same hook built in (``set_comm``)."""
    comm = None
    axis0_reduce = 'local'

    def set_comm(self, comm, axis0_reduce='local'):
        if axis0_reduce not in ('local', 'sum', 'avg'):
            raise ValueError("axis0_reduce must be 'local', 'sum' or 'avg'")
        self.comm = comm
        self.axis0_reduce = axis0_reduce

    def sum_t(self, a, axis, out):
        super(AxisZeroAllReduce, self).sum_t(a, axis, out)
        if axis == 0 and self.comm is not None and self.axis0_reduce != 'local':
            self.comm.allreduce(out, self.axis0_reduce)


def shard_batch(data, rank, world):
    """This rank's slice of the batch axis (axis 1) of every array in ``data``."""
    out = {}
    for k, v in data.items():
        b = v.shape[1]
        if b % world:
            raise ValueError('batch %d is not divisible by %d ranks' % (b, world))
        n = b // world
        out[k] = np.ascontiguousarray(v[:, rank * n:(rank + 1) * n])
    return out


def data_parallel(net, comm, axis0_reduce='local'):
    """Make ``net`` (already on its handler) train data-parallel over ``comm``.

    Wraps ``net.backward_pass`` of this instance so that the flat gradient vector
    is averaged over the ranks before the stepper reads it (steppers.py:61-69), and
    switches the handler's axis-0 sums to ``axis0_reduce``.  The Trainer, steppers
    and layers stay unchanged."""
    handler = net.handler
    if not hasattr(handler, 'set_comm'):
        raise TypeError('handler %r cannot complete sums across ranks' % (handler,))
    handler.set_comm(comm, axis0_reduce)
    local_backward = net.backward_pass

    def backward_pass():
        local_backward()
        comm.allreduce(net.buffer.gradients, 'avg')

    net.backward_pass = backward_pass
    return net
