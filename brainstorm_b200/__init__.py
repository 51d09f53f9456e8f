"""brainstorm_b200: an NVIDIA B200 (sm_100a) backend for the brainstorm Handler API.

    from brainstorm_b200 import B200Handler
    net.set_handler(B200Handler())

The first use of any name below loads ``libb200handler.so`` (build it with
``python -m brainstorm_b200.build``); there is no CPU fallback.  The names are
resolved lazily so that the build module can be run before the library exists.
"""
__all__ = ['B200Handler', 'B200Array', 'B200Error', 'GraphedStepper', 'RecordedStep', 'lib',
           'align_buffers', 'fuse_lstm_layers', 'fuse_layers', 'FusedSgdStepper', 'PrefetchingIterator', 'defer_loss_readback', 'data_parallel', 'Comm']

_HOME = {'B200Handler': 'handler', 'B200Array': 'array', 'B200Error': '_lib', 'lib': '_lib',
         'GraphedStepper': 'graph', 'RecordedStep': 'graph',
         # drop-ins for networks of the reference (these need brainstorm to be importable)
         'align_buffers': 'layout', 'fuse_lstm_layers': 'fused_lstm', 'fuse_layers': 'fused_layers', 'FusedSgdStepper': 'steppers', 'PrefetchingIterator': 'pipeline',
         'defer_loss_readback': 'pipeline', 'data_parallel': 'parallel', 'Comm': 'parallel'}


def __getattr__(name):
    if name in _HOME:
        import importlib
        value = getattr(importlib.import_module('.' + _HOME[name], __name__), name)
        globals()[name] = value
        return value
    raise AttributeError('module %r has no attribute %r' % (__name__, name))
