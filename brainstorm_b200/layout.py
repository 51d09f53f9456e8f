"""16-byte aligned hubs for networks that run on ``B200Handler``.

The reference's memory layer packs every hub of a network back to back into one flat
allocation (brainstorm/structure/buffers.py:48-55,79-83).  One hub of odd size -- the
scalar loss, a (batch, 1) target column -- leaves every hub behind it at an odd element
offset, and the kernels then cannot use 128-bit accesses or hand the arrays to TMA as they
are (GEMM operands are copied into an aligned temporary first).

``align_buffers(net)`` makes the network's ``BufferManager`` start every hub on a multiple
of four floats.  Only the slicing of the flat buffer changes: hub shapes, the layout, the
views, parameter handling on a resize and everything else are the reference's own.
``B200Handler(align_hubs=True)`` (the default) arranges the same by itself the first time a
``BufferManager`` asks it for its flat buffer, i.e. inside ``net.set_handler(handler)``; an
explicit ``align_buffers(net)`` is only needed for a handler created with
``align_hubs=False`` or to re-lay buffers that exist already.
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


def install_aligned_resize(manager, floats=4):
    """Give this ``BufferManager`` instance a ``resize`` that starts every hub on a multiple
    of `floats` elements; takes effect at its next resize.  Returns the new method."""
    from brainstorm.structure.buffers import create_buffer_views_from_layout

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
    manager._b200_aligned = True
    return resize


def align_buffers(net, floats=4):
    """Re-lay the hubs of ``net`` on `floats`-element boundaries, now and on every later
    resize.  Parameters are carried over.  Returns ``net``."""
    manager = net._buffer_manager
    resize = install_aligned_resize(manager, floats)
    # lay the current buffers out again (the padded total may exceed what is allocated)
    time_size, batch_size = manager.time_size, manager.batch_size
    manager.time_size = manager.batch_size = -1
    manager.size = -1
    net.buffer = resize(max(time_size, 0), max(batch_size, 0))
    return net


def align_calling_buffer_manager(depth=2):
    """Called by ``B200Handler.allocate``: if the caller `depth` frames up is
    ``BufferManager.resize`` asking for its one flat buffer (structure/buffers.py:79), give
    that manager the aligned ``resize`` for all later calls.  This is how a network gets
    aligned hubs from ``net.set_handler(B200Handler())`` alone: ``set_handler`` makes the
    manager resize to (0, 0) (buffers.py:98-108), which asks the new handler for memory."""
    import sys
    manager = None
    for up in range(depth, depth + 3):      # a wrapping handler (DebugHandler) adds a frame or two
        try:
            frame = sys._getframe(up)
        except ValueError:
            return False
        candidate = frame.f_locals.get('self')
        if frame.f_code.co_name == 'resize' and type(candidate).__name__ == 'BufferManager':
            manager = candidate
            break
    if manager is None:
        return False
    if getattr(manager, '_b200_aligned', False):
        return True
    try:
        install_aligned_resize(manager)
    except Exception:            # brainstorm is not importable or differs: leave the manager alone
        return False
    return True
