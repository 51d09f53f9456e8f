"""Device-side counterparts of host data iterators for networks on B200Handler.

``DeviceOneHot`` replaces the reference's ``OneHot`` iterator
(brainstorm/data_iterators.py:188-231), which expands index arrays to one-hot
vectors on the host (``np.eye(V)[idx]``) and then uploads V floats per symbol.
Here only the indices are uploaded and ``binarize_v`` writes the one-hot rows on
the GPU; the iterator yields device arrays, which
``Network.provide_external_data`` copies device-to-device (network.py:399-400).
"""
from __future__ import annotations

import numpy as np

from brainstorm.data_iterators import DataIterator
from brainstorm.utils import IteratorValidationError

from .array import B200Array


class DeviceOneHot(DataIterator):
    """Same arguments and validation as ``OneHot``; needs the network's
    ``B200Handler`` at iteration time (the Trainer passes it,
    training/trainer.py:96)."""

    def __init__(self, iter, vocab_size_dict):
        DataIterator.__init__(self, iter.data_shapes, iter.length)
        for key, size in vocab_size_dict.items():
            if key not in iter.data_shapes:
                raise IteratorValidationError(
                    'key {} is not present in iterator. Available keys: {}'.format(
                        key, iter.data_shapes.keys()))
            if not isinstance(size, int):
                raise IteratorValidationError('Vocabulary size must be int')
            shape = iter.data_shapes[key]
            if not (shape[-1] == 1 and len(shape) == 3):
                raise IteratorValidationError('Only 3D data is supported')
        self.vocab_size_dict = vocab_size_dict
        self.iter = iter

    def __call__(self, handler=None):
        if handler is None or getattr(handler, 'array_type', None) is not B200Array:
            raise IteratorValidationError('DeviceOneHot needs the B200Handler of the network')
        for data in self.iter(handler):
            for name, vocab in self.vocab_size_dict.items():
                idx = np.asarray(data[name])
                t, b = idx.shape[0], idx.shape[1]
                labels = handler.create_from_numpy(idx.reshape(t * b, 1))
                hot = B200Array.empty((t * b, vocab), zero=False)
                handler.binarize_v(labels, hot)
                data[name] = hot.reshape((t, b, vocab))
            yield data
