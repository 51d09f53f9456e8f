"""The two host round trips of a training update, taken off the critical path.

The reference's training loop (brainstorm/training/trainer.py:96-101) does, per update:
``provide_external_data`` (network.py:381-403: a blocking host-to-device copy of the batch),
``stepper.run()``, and ``get_loss_values`` (network.py:466: a device-to-host read of the
loss that waits for the whole step).  On a B200 both are as long as a small network's
step.  Two drop-ins, used with the unchanged ``Trainer``:

* ``PrefetchingIterator(iter)`` wraps any data iterator of the reference.  While step k
  runs, batch k+1 is copied into page-locked memory and uploaded on the library's
  upload stream into one of two sets of device arrays; the iterator yields device arrays,
  so ``provide_external_data`` takes its device-to-device branch (network.py:399-400).
* ``defer_loss_readback(net)`` makes ``net.get_loss_values()`` queue an asynchronous copy
  of the loss into page-locked memory and return the value of the previous update, which
  has arrived by then; ``history`` holds every update's true loss after ``flush()``.
"""
from __future__ import annotations

import ctypes
from collections import OrderedDict

import numpy as np

from brainstorm.data_iterators import DataIterator

from ._lib import lib, check
from .array import B200Array


class PrefetchingIterator(DataIterator):
    """Yields the batches of ``iter`` as device arrays, each uploaded while the previous
    step was running.  Needs the network's ``B200Handler`` at iteration time (the Trainer
    passes it, training/trainer.py:96)."""

    def __init__(self, iter):
        DataIterator.__init__(self, iter.data_shapes, iter.length)
        self.iter = iter

    def __call__(self, handler=None):
        if handler is None or getattr(handler, 'array_type', None) is not B200Array:
            raise ValueError('PrefetchingIterator needs the B200Handler of the network')
        slots = [{}, {}]             # name -> (page-locked host array, device array)
        free_after = [0, 0]          # event behind the last reader of each slot's device arrays

        def stage(batch, which):
            out = OrderedDict()
            for name, value in batch.items():
                if isinstance(value, B200Array):        # already on the device (e.g. DeviceOneHot upstream)
                    out[name] = value
                    continue
                value = np.asarray(value)
                have = slots[which].get(name)
                if have is None or have[0].shape != value.shape:
                    have = (handler.pinned_empty(value.shape), B200Array.empty(value.shape, zero=False))
                    slots[which][name] = have
                host, dev = have
                host[...] = value                        # cast to float32 like set_from_numpy
                handler.upload_async(dev, host, free_after[which])
                out[name] = dev
            return out

        source = iter(self.iter(handler))
        try:
            first = next(source)
        except StopIteration:
            return
        which = 0
        current = stage(first, which)
        while current is not None:
            handler.upload_join()                        # work queued from here on sees `current`
            try:
                following = next(source)
            except StopIteration:
                following = None
            # The other slot was last read by the update before this one; the event recorded when
            # that update had been queued (below) orders the new upload behind it.  The upload
            # then runs beside the update the caller starts after this yield.
            nxt = stage(following, which ^ 1) if following is not None else None
            yield current
            # the caller has queued the update that reads this slot: later uploads into it wait for that
            free_after[which] = handler.record_event(free_after[which] or None)
            current = nxt
            which ^= 1


class DeferredLoss(object):
    """Installed by ``defer_loss_readback``.  ``history`` lists the loss of every update in
    order (complete after ``flush()``); ``restore()`` gives the network its own
    ``get_loss_values`` back."""

    def __init__(self, net):
        self.net = net
        self.history = []
        self._original = net.get_loss_values
        self._inflight = []          # [event, host slot, loss layer names, values or None], oldest first
        self._slots = []
        self._events = [0, 0]
        self._count = 0

    def _resolve(self, entry):
        if entry[3] is None:
            event, host, names = entry[:3]
            check(lib.b200_event_wait(event))
            values = OrderedDict()
            if len(names) == 1:
                values['total_loss'] = float(host[0])
            else:
                for i, name in enumerate(names):
                    values[name] = float(host[i])
                values['total_loss'] = sum(values[name] for name in names)
            entry[3] = values
        return entry[3]

    def _retire_oldest(self):
        entry = self._inflight.pop(0)
        values = self._resolve(entry)
        self.history.append(values['total_loss'])
        return values

    def get_loss_values(self):
        net = self.net
        handler = net.handler
        names = list(net.loss_layers)
        while len(self._slots) < 2:
            self._slots.append(handler.pinned_empty((max(len(names), 1),)))
        k = self._count % 2
        self._count += 1
        host = self._slots[k]
        for i, name in enumerate(names):
            view = net.buffer[name].outputs.loss
            check(lib.b200_memcpy_d2h_async(host.ctypes.data + 4 * i, view.ptr, 4))
        self._events[k] = handler.record_event(self._events[k] or None)
        self._inflight.append([self._events[k], host, names, None])
        if len(self._inflight) >= 2:
            return self._retire_oldest()       # the previous update's loss: it has arrived by now
        return self._resolve(self._inflight[0])   # the very first update: nothing earlier to report

    def flush(self):
        """Waits for the newest update's loss; afterwards ``history`` is complete.  Returns
        the newest values."""
        values = None
        while self._inflight:
            values = self._retire_oldest()
        return values

    def restore(self):
        self.flush()
        self.net.get_loss_values = self._original


def defer_loss_readback(net):
    """Make ``net.get_loss_values()`` (network.py:455-475) return the loss of the previous
    update instead of waiting for the current one.  Returns the ``DeferredLoss`` that now
    serves the calls."""
    deferred = DeferredLoss(net)
    net.get_loss_values = deferred.get_loss_values
    return deferred
