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
    """All-reduce over the ranks of a ``torch.distributed`` group (initialised by the
    caller; it is the rendezvous and carries host arrays).  Device arrays go through the
    library's own entry points: ``b200_comm_allreduce`` (NCCL on the library's stream,
    recordable into graphs) and, for small arrays after ``enable_peer``,
    ``b200_peer_allreduce`` (one kernel over NVLink peer memory).  If the library cannot
    find NCCL, device arrays fall back to the group's NCCL backend."""

    def __init__(self, library_nccl=True):
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError('torch.distributed is not initialised')
        self.dist = dist
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self._stream = None
        self._lib_nccl = False    # device arrays go through b200_comm_allreduce
        if library_nccl and self.world > 1:
            self._join_library_communicator()
        self._peer_max = 0        # > 0: device arrays up to this many floats go over peer memory
        self._peer_windows = False   # this Comm registered peer windows that close() must release

    def _join_library_communicator(self):
        """Collective.  Rank 0 draws an NCCL id inside the library, the group hands it
        round, every rank joins.  One communicator per process: a second ``Comm`` reuses it."""
        import ctypes
        import torch
        from ._lib import lib
        if not torch.cuda.is_available() or not lib.b200_stream():
            return                                   # CPU ranks (gloo) or no handler yet
        if lib.b200_comm_world() == self.world:
            self._lib_nccl = True
            return
        # The collectives run beside compute kernels that want (almost) every SM for themselves:
        # a tensor-core GEMM CTA cannot share an SM with a collective's CTA (registers), so every
        # SM the collective holds is one the next GEMM wave does not get.  Sixteen CTAs carry the
        # gradient traffic of a step many times over; NCCL's default may take twice as many.
        import os
        os.environ.setdefault('NCCL_MAX_CTAS', '16')
        ident = ctypes.create_string_buffer(128)
        box = [ident.raw if (self.rank == 0 and lib.b200_comm_unique_id(ident) == 0) else None]
        self.dist.broadcast_object_list(box, src=0)
        ok = box[0] is not None and lib.b200_comm_init(self.rank, self.world, box[0]) == 0
        agreed = [None] * self.world
        self.dist.all_gather_object(agreed, ok)
        if all(agreed):
            self._lib_nccl = True
        elif ok:
            lib.b200_comm_destroy()

    @property
    def capturable(self):
        """True if every device all-reduce of this object can be part of a recorded step."""
        return self.world == 1 or self._lib_nccl

    def enable_peer(self):
        """Set up the library's all-reduce over NVLink peer memory for small device
        arrays (``b200_peer_allreduce``: one single-CTA kernel per call instead of a
        library collective; the sums that complete ``sum_t(axis=0)`` across batch shards
        are a few thousand floats).  Collective: every rank calls it.  Needs one process
        per GPU on one node and CUDA IPC between them; returns False, and leaves
        everything on NCCL, if any rank cannot set it up."""
        import ctypes
        from ._lib import lib
        if self.world == 1 or (self._peer_max and lib.b200_peer_enabled()):
            return bool(self._peer_max)
        if self.world > 16:
            return False
        # windows of an earlier Comm of this process (collectively: nobody uses them any more)
        lib.b200_sync()
        self.dist.barrier()
        lib.b200_peer_teardown()
        handle = ctypes.create_string_buffer(64)
        mine = ctypes.c_uint64()
        ok = lib.b200_peer_window_alloc(ctypes.byref(mine), handle) == 0
        gathered = [None] * self.world
        self.dist.all_gather_object(gathered, (ok, handle.raw if ok else None))
        ok = all(g[0] for g in gathered)
        windows = (ctypes.c_uint64 * self.world)()
        opened = []
        registered = False
        if ok:
            for r, (_, raw) in enumerate(gathered):
                if r == self.rank:
                    windows[r] = mine.value
                    continue
                p = ctypes.c_uint64()
                if lib.b200_peer_window_open(raw, ctypes.byref(p)) != 0:
                    ok = False
                    break
                opened.append(p.value)
                windows[r] = p.value
            if ok:
                registered = ok = lib.b200_peer_setup(self.rank, self.world, windows) == 0
        agreed = [None] * self.world
        self.dist.all_gather_object(agreed, ok)
        if not all(agreed):
            if registered:
                lib.b200_peer_teardown()          # frees this rank's window and unmaps the others
            else:                                 # never registered: give the pieces back one by one
                for p in opened:
                    lib.b200_peer_window_release(p, 0)
                lib.b200_peer_window_release(mine.value, 1)
            return False
        self.dist.barrier()               # every window is mapped and cleared everywhere before the first call
        self._peer_max = int(lib.b200_peer_max_floats())
        self._peer_windows = True
        return True

    def close(self):
        """Release the peer-memory windows (collective; after the last all-reduce)."""
        if self._peer_windows:
            from ._lib import lib, check
            lib.b200_sync()               # an error flagged earlier has been reported already
            self.dist.barrier()
            self._peer_max = 0
            self._peer_windows = False
            check(lib.b200_peer_teardown())

    def _peer_ok(self, arr):
        """True if ``arr`` goes over peer memory.  After a wait ran out (a rank never
        arrived; the library reported it at a synchronising call) the ranks' call counters
        no longer agree and the library has switched the path off: everything goes back to
        NCCL until ``enable_peer`` is called again."""
        if not self._peer_max or arr.size > self._peer_max:
            return False
        from ._lib import lib
        if not lib.b200_peer_enabled():
            self._peer_max = 0
            return False
        return True

    def peer_wait_stats(self):
        """(calls, seconds): the peer all-reduces of this rank since ``enable_peer`` and the time
        their kernels spent waiting for the other ranks' values.  Synchronises."""
        import ctypes
        from ._lib import lib, check
        calls, waited = ctypes.c_uint64(), ctypes.c_uint64()
        check(lib.b200_peer_wait_stats(ctypes.byref(calls), ctypes.byref(waited)))
        return calls.value, waited.value * 1e-9

    def _peer_allreduce(self, arr, op):
        from ._lib import lib, check
        check(lib.b200_peer_allreduce(arr.ptr, arr.ptr, arr.size, 1 if op == 'avg' else 0))

    def _device_stream(self):
        # NCCL work is ordered after, and the library's later kernels after it, by
        # presenting the library stream to torch as the current stream: no host sync.
        if self._stream is None:
            import torch
            from ._lib import lib
            self._stream = torch.cuda.ExternalStream(lib.b200_stream())
        return self._stream

    def allreduce_async(self, arr, op='sum'):
        """Start an in-place all-reduce and return a handle for ``wait``.  On the GPU
        the collective is ordered after the kernels queued so far, and kernels queued
        after this call do NOT wait for it until ``wait(handle)``."""
        import torch
        if self.world == 1 or arr.size == 0:
            return None
        if isinstance(arr, np.ndarray):
            if not arr.flags.c_contiguous:
                raise NotImplementedError('asynchronous all-reduce of a strided host view')
            buf = arr.reshape(-1)
            work = self.dist.all_reduce(torch.from_numpy(buf), op=self.dist.ReduceOp.SUM, async_op=True)
            return (work, buf if op == 'avg' else None)
        if not arr.is_contiguous:
            raise NotImplementedError('asynchronous all-reduce of a strided device view')
        if self._peer_ok(arr):
            self._peer_allreduce(arr, op)     # a kernel on the library stream: nothing to wait for
            return None
        if self._lib_nccl:
            from ._lib import lib, check
            check(lib.b200_comm_allreduce_async(arr.ptr, arr.size, 1 if op == 'avg' else 0))
            return 'library'
        flat = arr.reshape((arr.size,))
        with torch.cuda.stream(self._device_stream()):
            t = torch.as_tensor(flat, device='cuda')
            work = self.dist.all_reduce(
                t, op=self.dist.ReduceOp.AVG if op == 'avg' else self.dist.ReduceOp.SUM, async_op=True)
        return (work, None)

    def wait(self, handle):
        if handle is None:
            return
        if handle == 'library':             # the library stream waits for its communication stream
            from ._lib import lib, check
            check(lib.b200_comm_join())
            return
        work, host_avg = handle
        if host_avg is not None:
            work.wait()
            host_avg /= host_avg.dtype.type(self.world)
            return
        import torch
        if torch.cuda.is_available() and self._stream is not None:
            with torch.cuda.stream(self._device_stream()):
                work.wait()          # the library stream waits; the host does not
        else:
            work.wait()

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
        if arr.size == 0:
            return
        if not arr.is_contiguous:           # a strided view: through a contiguous temporary
            from .handler import _any_handler
            h = _any_handler()
            tmp = h._contiguous_copy(arr)
            self.allreduce(tmp, op)
            h.copy_to(tmp, arr)
            return
        if self._peer_ok(arr):
            self._peer_allreduce(arr, op)
            return
        if self._lib_nccl:
            from ._lib import lib, check
            check(lib.b200_comm_allreduce(arr.ptr, arr.size, 1 if op == 'avg' else 0))
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


def _element_offset(view, flat):
    """Offset of ``view`` inside ``flat`` in elements (numpy or device arrays)."""
    if isinstance(view, np.ndarray):
        return (view.__array_interface__['data'][0] - flat.__array_interface__['data'][0]) // flat.itemsize
    return (view.ptr - flat.ptr) // 4


OVERLAP_MIN_BYTES = 32 << 20     # gradient vectors below this are all-reduced in one piece


def data_parallel(net, comm, axis0_reduce='local', overlap=True, peer=True, on_phase=None):
    """Make ``net`` (already on its handler) train data-parallel over ``comm``.

    Wraps ``net.backward_pass`` of this instance so that the flat gradient vector
    is averaged over the ranks before the stepper reads it (steppers.py:61-69), and
    switches the handler's axis-0 sums to ``axis0_reduce``.  The Trainer, steppers
    and layers stay unchanged.

    With ``overlap`` the all-reduce is issued per layer, as soon as that layer's
    backward pass has been queued (the gradients of one layer are one contiguous
    block of the flat vector, brainstorm/structure/layout.py:149-157), so the
    collective of layer k runs while the layers before it are still computing.
    Networks with gradient modifiers fall back to one all-reduce at the end, since
    the modifiers run inside the reference's backward_pass (network.py:445).

    With ``peer`` (the default, and a ``B200Handler``) all-reduces of small device arrays,
    i.e. the batch statistics, use the library's kernel over NVLink peer memory instead of a
    library collective (``Comm.enable_peer``; stays on NCCL if the ranks cannot map each
    other's memory).

    ``on_phase`` (for measurements): called with ``'backward_queued'`` when the local
    backward pass has been queued and with ``'reduced'`` when the work queued next will
    see the averaged gradients."""
    handler = net.handler
    if not hasattr(handler, 'set_comm'):
        raise TypeError('handler %r cannot complete sums across ranks' % (handler,))
    if axis0_reduce == 'sum':
        # every sum over the batch axis would be summed over the ranks, the bias and BatchNorm
        # gradients among them, and the gradient average that follows would leave those `world`
        # times too large next to the weight gradients
        raise ValueError("axis0_reduce='sum' is for plain op sequences (the op-suite benchmark); "
                         "training needs 'avg' (global batch statistics) or 'local'")
    handler.set_comm(comm, axis0_reduce)
    if peer and hasattr(comm, 'enable_peer') and type(handler).__name__ == 'B200Handler':
        comm.enable_peer()                # small all-reduces over NVLink peer memory, if the node allows it
    local_backward = net.backward_pass
    pending = []

    def backward_pass():
        del pending[:]
        if axis0_reduce == 'avg' and hasattr(handler, '_axis0_skip') and hasattr(net.buffer.gradients, 'ptr'):
            # Sums over the batch axis that land in the gradient vector (bias gradients) are averaged
            # with it below; completing each of them across the ranks first would be a second,
            # redundant exchange.  (In 'avg' mode both give the same values.)
            g = net.buffer.gradients
            handler._axis0_skip = (g.ptr, g.ptr + 4 * g.size)
        local_backward()
        if on_phase is not None:
            on_phase('backward_queued')
        if pending:
            for h in pending:
                comm.wait(h)
            del pending[:]
        else:
            comm.allreduce(net.buffer.gradients, 'avg')
        if on_phase is not None:
            on_phase('reduced')

    net.backward_pass = backward_pass

    # Small networks are bound by the host: one collective over the whole vector costs fewer
    # calls than one per layer, and there is nothing worth overlapping.
    big_enough = net.buffer.gradients.size * 4 >= OVERLAP_MIN_BYTES
    if overlap and big_enough and hasattr(comm, 'allreduce_async') and not getattr(net, 'gradient_modifiers', None):
        def wrap(name, layer):
            layer_backward = layer.backward_pass

            def layer_backward_then_reduce(buffers):
                layer_backward(buffers)
                flat = net.buffer.gradients
                views = list(net.buffer[name].gradients)
                lo = min(_element_offset(v, flat) for v in views)
                hi = max(_element_offset(v, flat) + v.size for v in views)
                pending.append(comm.allreduce_async(flat[lo:hi], 'avg'))

            layer.backward_pass = layer_backward_then_reduce

        for name, layer in net.layers.items():
            if 'gradients' in net.buffer[name] and len(net.buffer[name].gradients):
                wrap(name, layer)
    return net
