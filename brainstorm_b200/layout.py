"""16-byte aligned hubs for networks that run on ``B200Handler``.

The reference's memory layer packs every hub of a network back to back into one flat
allocation (brainstorm/structure/buffers.py:48-55,79-83).  One hub of odd size -- the
scalar loss, a (batch, 1) target column -- leaves every hub behind it at an odd element
offset, and the kernels then cannot use 128-bit accesses or hand the arrays to TMA as they
are (GEMM operands are copied into an aligned temporary first).

``align_buffers(net)`` makes the network's ``BufferManager`` start every hub on a multiple
of four floats.  Only the slicing of the flat buffer changes: hub shapes, the layout, the
views, parameter handling on a resize and everything else are the reference's own.  Call
it after ``net.set_handler(B200Handler())``, like ``fuse_lstm_layers``.
"""
from __future__ import annotations

import numpy as np


def aligned_slices(shapes, floats=4):
    """(total size, [slice per hub]) with every slice starting on a multiple of `floats`."""
    slices, pos = [], 0
    for shape in shapes:
        pos = -(-pos // floats) * floats
        n = int(np.prod(shape))
        slices.append(slice(pos, pos + n))
        pos += n
    return pos, slices


def align_buffers(net, floats=4):
    """Re-lay the hubs of ``net`` on `floats`-element boundaries, now and on every later
    resize.  Parameters are carried over.  Returns ``net``."""
    from brainstorm.structure.buffers import create_buffer_views_from_layout
    manager = net._buffer_manager

    def resize(time_size, batch_size):
        # BufferManager.resize (buffers.py:69-96) with padded hub starts
        if time_size == manager.time_size and batch_size == manager.batch_size:
            return manager.views
        manager.time_size = time_size
        manager.batch_size = batch_size
        shapes = [h.get_shape(time_size, batch_size) for h in manager.hubs]
        total_size, slices = aligned_slices(shapes, floats)
        if total_size > manager.size:
            manager.full_buffer = manager.handler.allocate((total_size,))
            manager.size = total_size
        manager.buffers = [manager.full_buffer[slices[i]].reshape(shapes[i]) for i in range(len(manager.hubs))]
        parameters = None
        if manager.views is not None:
            parameters = manager.handler.get_numpy_copy(manager.views.parameters)
        manager.views = create_buffer_views_from_layout(manager.layout, manager.buffers, manager.hubs,
                                                        existing_view=manager.views)
        if parameters is not None:
            manager.handler.set_from_numpy(manager.views.parameters, parameters)
        return manager.views

    manager.resize = resize
    # lay the current buffers out again (the padded total may exceed what is allocated)
    time_size, batch_size = manager.time_size, manager.batch_size
    manager.time_size = manager.batch_size = -1
    manager.size = -1
    net.buffer = resize(max(time_size, 0), max(batch_size, 0))
    return net
