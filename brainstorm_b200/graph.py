"""Recorded training steps: one replay call instead of one launch per kernel.

A training step of the reference (``TrainingStepper.run``,
brainstorm/training/steppers.py:61-70 for SGD, :103-121 with momentum) is a fixed
sequence of handler calls on the fixed views of one flat buffer
(brainstorm/structure/buffers.py:79-99).  For small networks the step is bound by
the host: the 85 kernels of the MNIST MLP step take less time on the device than
Python and the driver need to launch them.  ``B200Handler.record`` runs such a
sequence once with the library stream in capture mode and returns a
``RecordedStep``; ``launch()`` replays all of it with one call.

``GraphedStepper`` wraps any stepper of the reference so that a ``Trainer`` uses
this without changes::

    trainer = bs.Trainer(GraphedStepper(bs.training.MomentumStepper(0.1, 0.9)))

What a recording freezes: every address, shape and scalar argument (learning rate,
momentum, dropout probability).  What it does not freeze: the contents of the
buffers (new batches are copied into the same input views between replays) and the
random masks (every replay draws from a new Philox stream).  ``GraphedStepper``
records again when the buffer layout, the batch shape or a scalar attribute of
the wrapped stepper changes.
"""
from __future__ import annotations

import ctypes

from ._lib import lib, check

try:  # the reference's base class keeps the wrapper describable for checkpoints
    from brainstorm.training.steppers import TrainingStepper as _StepperBase
except Exception:  # brainstorm is not importable: stand-alone use
    class _StepperBase(object):
        def __init__(self):
            self.net = None

        def start(self, net):
            self.net = net

        def run(self):
            pass


class RecordedStep(object):
    """Handle of a recorded sequence of handler calls (see ``B200Handler.record``).

    Arrays that the recorded calls touch must stay alive for as long as the step is
    replayed; arrays released *during* the recording are kept alive by the
    recording itself, and so are the work arrays the handler and the fused layers
    lent to the recorded calls (``keep``)."""

    def __init__(self, handle, keep=()):
        self._handle = int(handle)
        self._keep = list(keep)
        n = ctypes.c_uint64()
        check(lib.b200_graph_kernel_count(self._handle, ctypes.byref(n)))
        self.kernels = int(n.value)

    def launch(self):
        if not self._handle:
            raise ValueError('this recorded step has been released')
        check(lib.b200_graph_launch(self._handle))

    __call__ = launch

    def release(self):
        handle, self._handle = self._handle, 0
        if handle:
            check(lib.b200_graph_destroy(handle))
        self._keep = []

    def __del__(self):
        try:
            self.release()
        except Exception:  # interpreter shutdown
            pass


def _release_handover_slots():
    """The fused LSTM layers leave work arrays for the layer that is called next
    (fused_lstm._handover).  Emptied while a recording is still open, the arrays are
    released inside it, and the library keeps such memory until the recording is
    destroyed; left in place, the next ordinary pass would free memory that every
    replay still writes."""
    import sys
    mod = sys.modules.get('brainstorm_b200.fused_lstm')
    if mod is not None:
        for k in mod._handover:
            mod._handover[k] = None


def record(fn, *args, **kwargs):
    """Run ``fn(*args, **kwargs)`` with the library stream in capture mode.

    Nothing executes during the call: the handler calls ``fn`` makes are recorded.
    Calls that wait for the device or cross PCIe (``get_numpy_copy``,
    ``set_from_numpy``, ``synchronize`` ...) raise ``B200Error`` and the recording
    is discarded.  Run ``fn`` once the ordinary way first: work buffers that grow on
    first use cannot grow inside a recording.

    ``handler`` (keyword, optional): the handler whose calls are recorded.  Its
    reduction scratch array is baked into the recording, so the recording keeps a
    reference to it: a later ordinary ``sum_t`` that needs a larger one allocates a
    new array without freeing the one replays still use."""
    handler = kwargs.pop('handler', None)
    check(lib.b200_graph_begin())
    try:
        fn(*args, **kwargs)
        _release_handover_slots()
    except BaseException:
        lib.b200_graph_end(None)   # discard; the original exception is the one to report
        raise
    handle = ctypes.c_uint64()
    check(lib.b200_graph_end(ctypes.byref(handle)))
    keep = []
    scratch = getattr(handler, '_scratch', None)
    if scratch is not None:
        keep.append(scratch)
    return RecordedStep(handle.value, keep)


def _scalars(obj):
    return tuple(sorted((k, v) for k, v in vars(obj).items()
                        if isinstance(v, (bool, int, float)) and not k.startswith('_')))


class GraphedStepper(_StepperBase):
    """Wraps a stepper of the reference; replays its ``run()`` from a recording.

    The first ``eager_steps`` runs (and the first runs after anything the
    recording depends on has changed) go through the wrapped stepper the
    ordinary way, which also sizes every work buffer; the next one is recorded;
    all later ones are replays."""
    __undescribed__ = {'net', '_step', '_key', '_eager_left'}
    __default_values__ = {'eager_steps': 1}

    def __init__(self, stepper, eager_steps=1):
        super(GraphedStepper, self).__init__()
        self.stepper = stepper
        self.eager_steps = int(eager_steps)
        self._step = None
        self._key = None
        self._eager_left = self.eager_steps

    def start(self, net):
        super(GraphedStepper, self).start(net)
        self.stepper.start(net)
        self.invalidate()

    def invalidate(self):
        """Forget the recording (after changing something it froze)."""
        if self._step is not None:
            self._step.release()
        self._step = None
        self._key = None
        self._eager_left = self.eager_steps

    def _state_key(self):
        manager = self.net._buffer_manager
        full = manager.full_buffer
        return (getattr(full, 'ptr', id(full)), manager.time_size, manager.batch_size,
                type(self.stepper).__name__, _scalars(self.stepper))

    def run(self):
        comm = getattr(self.net.handler, '_comm', None)
        if comm is not None and not getattr(comm, 'capturable', False):
            return self.stepper.run()       # data parallel over collectives that cannot be recorded: run as usual
        key = self._state_key()
        if key != self._key:
            self.invalidate()
            self._key = key
        if self._step is None:
            if self._eager_left > 0:
                self._eager_left -= 1
                return self.stepper.run()
            self._step = record(self.stepper.run, handler=self.net.handler)
        self._step.launch()
