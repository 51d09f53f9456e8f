"""Drop-in fused LSTM layer for networks that run on ``B200Handler``.

``FusedLstmLayerImpl`` subclasses the reference's ``LstmLayerImpl``
(brainstorm/layers/lstm_layer.py:21) and keeps its ``setup`` untouched, so
parameter names, order and shapes (:38-55), the twenty internal buffers (:57-87),
memory layout, initialisers and saved networks are interchangeable with the
reference layer.  Only ``forward_pass`` / ``backward_pass`` differ: the four input
projections are one stacked GEMM, and the loop over time is one library call that
runs, per timestep, one stacked recurrent GEMM and one gate kernel
(``b200_lstm_forward`` / ``b200_lstm_backward``) instead of 19 / 20 handler calls.

    net.set_handler(B200Handler())
    fuse_lstm_layers(net)            # swaps the class of every LSTM layer in place

Every buffer the reference layer fills is filled with the same values (to
rounding: the recurrent contributions of the four gates are summed inside one
GEMM instead of one after the other).

Stacked LSTM layers run side by side.  The reference walks a network layer by
layer (brainstorm/structure/network.py:429-430, :441-444), but layer l+1 at time t
needs layer l only up to time t, and a timestep is latency-bound (it leaves most
of the GPU idle).  A fused layer therefore marks the stream after every piece of
about ``PIECE`` timesteps; a fused layer called directly after the layer that produced
its input (forward) or its output deltas (backward) walks the same pieces on the
library's second stream, each piece as soon as the other layer has finished it,
and the main stream joins it before the call returns.
"""
from __future__ import annotations

import ctypes

from brainstorm.layers.lstm_layer import LstmLayerImpl
from brainstorm.utils import flatten_time, flatten_time_and_features

from ._lib import lib, check
from .array import B200Array
from .handler import B200Handler

_ACT = {'sigmoid': 0, 'tanh': 1, 'rel': 2, 'el': 3, 'linear': 4}

PIECE = 32            # about this many timesteps per piece when stacked layers overlap (0 = never overlap)
# What the fused layer that ran last left behind, per direction: (address of the array it
# filled, _Pieces).  Only the layer called directly afterwards may take it, so one slot each.
_handover = {'forward': None, 'backward': None}


def _take(direction, address):
    """The pieces left for the array at `address`, if the last fused layer left any; the
    slot is emptied either way."""
    left, _handover[direction] = _handover[direction], None
    return left[1] if left is not None and left[0] == address else None


class _Pieces(object):
    """What a fused layer leaves behind for the fused layer that is called next."""

    def __init__(self, layer, ranges, marks, start, stream, launches, y_work=None):
        self.layer = layer          # the layer that ran them
        self.ranges = ranges        # [(t0, t1), ...] in the order they were run
        self.marks = marks          # marks[i] is reached when piece i is complete
        self.start = start          # mark on the producer's stream from before its first piece
        self.stream = stream        # 0 = main, 1 = side
        self.launches = launches    # library launch counter when the producer returned
        self.y_work = y_work        # forward: aligned copy of the output sequence


def _ranges(T):
    """The sequence cut into about T / PIECE pieces of equal length."""
    n = int(round(T / float(PIECE))) if PIECE > 0 else 1
    if n < 2:
        return [(0, T)]
    cuts = [(T * i) // n for i in range(n + 1)]
    return [(cuts[i], cuts[i + 1]) for i in range(n)]


def _share(i, n, follows, followed):
    """Split-K plan of piece i of n: while two layers' loops run at the same time their
    recurrent GEMMs plan for half of the SMs each, so that both are resident together
    (two loops finish in 2.43 ms instead of 2.77 ms); a loop that runs alone plans for
    all of them.  The layer that follows another one runs alone in its last piece, the
    layer that is followed in its first."""
    if follows:
        return 2 if i < n - 1 else 1
    return 2 if followed and i >= 1 else 1


def _new_mark():
    m = ctypes.c_uint64()
    check(lib.b200_mark_create(ctypes.byref(m)))
    return m.value


def _stack(views, shape):
    """One array over parameter views that lie back to back in memory, or None."""
    for a, b in zip(views[:-1], views[1:]):
        if not (a.is_contiguous and b.is_contiguous and a.ptr + 4 * a.size == b.ptr):
            return None
    return B200Array(views[0].base, views[0].ptr, shape)


def _aligned(h, arr):
    """arr itself if it starts on a 16-byte boundary, else an aligned copy."""
    if arr.ptr % 16 == 0:
        return arr
    c = B200Array.empty(arr.shape, zero=False)
    h.copy_to(arr, c)
    return c


class FusedLstmLayerImpl(LstmLayerImpl):

    def _stacks(self, views, in_size):
        H = self.size
        (Wz, Wi, Wf, Wo, pi, pf, po, Rz, Ri, Rf, Ro, bz, bi, bf, bo) = views
        return (_stack([Wz, Wi, Wf, Wo], (4 * H, in_size)), _stack([Rz, Ri, Rf, Ro], (4 * H, H)),
                _stack([bz, bi, bf, bo], (4 * H,)), _stack([pi, pf, po], (3 * H,)))

    def _marks(self, n):
        marks = self.__dict__.setdefault('_mark_pool', [])
        while len(marks) < n + 2:
            marks.append(_new_mark())
        return marks[2:n + 2], marks[0], marks[1]      # piece marks, start mark, done mark

    def forward_pass(self, buffers, training_pass=True):
        h = self.handler
        x = buffers.inputs.default
        y = buffers.outputs.default
        T, B = x.shape[0], x.shape[1]
        H = self.size
        self._fused = None
        prod = _take('forward', x.ptr)      # the layer that has just produced x, if it left pieces to follow
        flat_x = flatten_time_and_features(x)
        stacks = self._stacks(buffers.parameters, flat_x.shape[1])
        hubs = list(buffers.internals)[:10] + [y]
        if (not isinstance(h, B200Handler) or any(s is None for s in stacks) or
                not all(a.is_contiguous for a in hubs) or T == 0):
            return LstmLayerImpl.forward_pass(self, buffers, training_pass)
        Wst, Rst, bst, pst = stacks
        (Za, Zb, Ia, Ib, Fa, Fb, Oa, Ob, Ca, Cb) = hubs[:10]
        ranges = _ranges(T)
        marks, start, done = self._marks(len(ranges))
        if prod is not None and not (prod.ranges == ranges and len(ranges) > 1 and prod.stream == 0 and
                                     prod.y_work.shape == (T + 1,) + tuple(x.shape[1:]) and
                                     prod.launches == lib.b200_launch_count()):
            prod = None
        # was this layer followed in the last pass?  Then it will be in this one (a guess that costs
        # little when wrong and corrects itself in the next pass)
        followed, self._followed_fwd = getattr(self, '_followed_fwd', False), False
        if prod is not None:
            prod.layer._followed_fwd = True
        stream = 0 if prod is None else 1
        if stream:
            check(lib.b200_use_stream(1))
        try:
            if stream:
                check(lib.b200_wait_mark(prod.start))       # everything queued before the producer's pieces
            else:
                check(lib.b200_mark(start))
            xproj = B200Array.empty((T * B, 4 * H), zero=False)
            Rw = _aligned(h, Rst)
            y_work = B200Array.empty((T + 1, B, H), zero=False)
            h.copy_to(y[T], y_work[T])                          # context: y[t-1] at t = 0
            r_work = B200Array.empty((B, 4 * H), zero=False)
            if prod is None:
                h.dot_mm(flat_x, Wst, xproj, transb=True)       # lstm_layer.py:110-113, stacked
            else:
                Ww = _aligned(h, Wst)
                src = flatten_time_and_features(prod.y_work[:T])   # the same values as x, 16-byte aligned
            for i, (t0, t1) in enumerate(ranges):
                if prod is not None:
                    check(lib.b200_wait_mark(prod.marks[i]))
                    h.dot_mm(src[t0 * B:t1 * B], Ww, xproj[t0 * B:t1 * B], transb=True)
                check(lib.b200_set_tuning(6, _share(i, len(ranges), prod is not None, followed)))
                check(lib.b200_lstm_forward_steps(xproj.ptr, Rw.ptr, bst.ptr, pst.ptr, Za.ptr, Zb.ptr, Ia.ptr,
                                                  Ib.ptr, Fa.ptr, Fb.ptr, Oa.ptr, Ob.ptr, Ca.ptr, Cb.ptr, y.ptr,
                                                  y_work.ptr, r_work.ptr, T, B, H, _ACT[self.activation], t0, t1))
                if len(ranges) > 1:
                    check(lib.b200_mark(marks[i]))
            if stream:
                check(lib.b200_mark(done))
        finally:
            lib.b200_set_tuning(6, 1)
            if stream:
                check(lib.b200_use_stream(0))
        if stream:
            check(lib.b200_wait_mark(done))                     # the main stream joins
        self._fused = (Rw, y_work, r_work, prod is not None, prod.y_work if prod is not None else None)
        if len(ranges) > 1:
            _handover['forward'] = (y.ptr, _Pieces(self, ranges, marks, start if not stream else done, stream,
                                                   lib.b200_launch_count(), y_work))

    def backward_pass(self, buffers):
        fused = getattr(self, '_fused', None)
        dx = buffers.input_deltas.default
        deltas = buffers.output_deltas.default
        # the layer that has just added its input deltas to `deltas`, if it left pieces to follow
        prod = _take('backward', deltas.ptr)
        if fused is None:
            return LstmLayerImpl.backward_pass(self, buffers)
        h = self.handler
        Rw, y_work, r_work, fed_by_lstm, x_work = fused
        x = buffers.inputs.default
        T, B = x.shape[0], x.shape[1]
        H = self.size
        flat_x = flatten_time_and_features(x) if x_work is None else flatten_time_and_features(x_work[:T])
        Wst, _, _, pst = self._stacks(buffers.parameters, flat_x.shape[1])
        dWst, dRst, dbst, _ = self._stacks(buffers.gradients, flat_x.shape[1])
        (dpi, dpf, dpo) = list(buffers.gradients)[4:7]
        (Za, Zb, Ia, Ib, Fa, Fb, Oa, Ob, Ca, Cb,
         dZa, dZb, dIa, dIb, dFa, dFb, dOa, dOb, dCa, dCb) = buffers.internals
        if dWst is None or dRst is None or dbst is None or not deltas.is_contiguous:
            return LstmLayerImpl.backward_pass(self, buffers)

        ranges = _ranges(T)[::-1]                               # from the end of the sequence backwards
        marks, start, done = self._marks(len(ranges))
        flat_dx = flatten_time_and_features(dx)
        if prod is not None and not (prod.ranges == ranges and len(ranges) > 1 and prod.stream == 0 and
                                     prod.launches == lib.b200_launch_count()):
            prod = None
        # a layer fed by a fused LSTM layer hands its input deltas over piece by piece
        by_piece = fed_by_lstm and len(ranges) > 1
        followed, self._followed_bwd = getattr(self, '_followed_bwd', False), False
        if prod is not None:
            prod.layer._followed_bwd = True
        stream = 0 if prod is None else 1
        if stream:
            check(lib.b200_use_stream(1))
        try:
            if stream:
                check(lib.b200_wait_mark(prod.start))
            else:
                check(lib.b200_mark(start))
            dG = B200Array.empty((T + 1, B, 4 * H), zero=False)
            h.fill(dG[T], 0.0)
            h.fill(dCa, 0.0)                                    # lstm_layer.py:168
            Ww = _aligned(h, Wst) if by_piece else Wst
            for i, (t0, t1) in enumerate(ranges):
                if prod is not None:
                    check(lib.b200_wait_mark(prod.marks[i]))
                check(lib.b200_set_tuning(6, _share(i, len(ranges), prod is not None, followed and by_piece)))
                check(lib.b200_lstm_backward_steps(deltas.ptr, Rw.ptr, pst.ptr, Zb.ptr, Ib.ptr, Fb.ptr, Ob.ptr,
                                                   Ca.ptr, Cb.ptr, dZa.ptr, dZb.ptr, dIa.ptr, dIb.ptr, dFa.ptr,
                                                   dFb.ptr, dOa.ptr, dOb.ptr, dCa.ptr, dCb.ptr, dG.ptr,
                                                   r_work.ptr, T, B, H, _ACT[self.activation], t0, t1))
                if by_piece:                                    # input deltas of this piece (:216-219)
                    h.dot_add_mm(dG[t0:t1].reshape(((t1 - t0) * B, 4 * H)), Ww, flat_dx[t0 * B:t1 * B])
                    check(lib.b200_mark(marks[i]))
            if stream:
                check(lib.b200_mark(done))
        finally:
            lib.b200_set_tuning(6, 1)
            if stream:
                check(lib.b200_use_stream(0))
        if stream:
            check(lib.b200_wait_mark(done))                     # the main stream joins
        handed_over = _Pieces(self, ranges, marks, start if not stream else done, stream, 0) if by_piece else None
        dGf = dG[:T].reshape((T * B, 4 * H))
        # input deltas and input-weight gradients (:216-224), four gates at once
        if not by_piece:
            h.dot_add_mm(dGf, Wst, flat_dx)
        h.dot_add_mm(dGf, flat_x, dWst, transa=True)
        # biases (:226-234)
        tmp = B200Array.empty((4 * H,), zero=False)
        h.sum_t(dGf, axis=0, out=tmp)
        h.add_tt(dbst, tmp, dbst)
        # recurrent-weight gradients (:253-256); the extra term of :258-261 multiplies
        # a slice of the reference's temporary that is never written, i.e. zeros
        if T > 1:
            h.dot_add_mm(dG[1:T].reshape(((T - 1) * B, 4 * H)),
                         y_work[:T - 1].reshape(((T - 1) * B, H)), dRst, transa=True)
        # peepholes (:236-278)
        dWc = B200Array.empty(dpo.shape, zero=False)
        products = B200Array.empty((T * B, H), zero=False)
        h.mult_tt(flatten_time(Ca[:T]), flatten_time(dOa[:T]), products)
        h.sum_t(products, axis=0, out=dWc)
        h.add_tt(dpo, dWc, dpo)
        for d_gate, d_peep in ((dIa, dpi), (dFa, dpf)):
            if T > 1:
                p1 = products[:(T - 1) * B]
                h.mult_tt(flatten_time(Ca[:T - 1]), flatten_time(d_gate[1:T]), p1)
                h.sum_t(p1, axis=0, out=dWc)
                h.add_tt(d_peep, dWc, d_peep)
            p0 = products[:B]
            h.mult_tt(dCa[T], dIa[0], p0)                        # :273-278 (both use dIa[0])
            h.sum_t(p0, axis=0, out=dWc)
            h.add_tt(d_peep, dWc, d_peep)
        self._fused = None
        if handed_over is not None:
            handed_over.launches = lib.b200_launch_count()
            _handover['backward'] = (dx.ptr, handed_over)


def fuse_lstm_layers(net):
    """Swap every LSTM layer of ``net`` for the fused implementation, in place.
    Returns the names of the layers that were swapped."""
    swapped = []
    for name, layer in net.layers.items():
        if type(layer) is LstmLayerImpl:
            layer.__class__ = FusedLstmLayerImpl
            layer._fused = None
            swapped.append(name)
    return swapped
