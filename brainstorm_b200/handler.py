"""B200Handler: the brainstorm ``Handler`` API on one NVIDIA B200.

A third backend beside the reference's ``NumpyHandler``
(brainstorm/handlers/numpy_handler.py:13) and ``PyCudaHandler``
(brainstorm/handlers/pycuda_handler.py:26).  It is installed like them::

    net.set_handler(B200Handler())         # brainstorm/structure/network.py:359

Every method implements the abstract method of the same name in
brainstorm/handlers/base_handler.py and must agree with ``NumpyHandler`` on the
same inputs.  All arithmetic runs in hand-written sm_100a kernels behind the
C-ABI of ``include/b200_handler.h``; this file only translates array views into
pointers and extents.  There is no CPU or library fallback: without the shared
library the import fails, and without a B200 the constructor raises.
"""
from __future__ import annotations

import ctypes

import numpy as np

from ._lib import lib, check, B200Error  # noqa: F401
from .array import B200Array
from .handler_api import Handler, new_random_state

_f32 = np.float32
_byref = ctypes.byref


def _sizes_match(*arrs):
    n = arrs[0].size
    for a in arrs[1:]:
        if a.size != n:
            raise ValueError('operands differ in size: %r' % ([x.shape for x in arrs],))
    return n


def _views(*arrs):
    """(rows, cols, [ld per operand]) of equally sized elementwise operands."""
    n = _sizes_match(*arrs)
    contig = True
    for a in arrs:
        if not a._contig:
            contig = False
            break
    if contig:
        return 1, n, [n] * len(arrs)
    forms = [a.as_2d() for a in arrs]
    rc = None
    for a, f in zip(arrs, forms):
        if f is None:
            raise NotImplementedError('view with strides %r has no row-pitched form' % (a.strides,))
        if not a._contig:
            if rc is None:
                rc = (f[0], f[1])
            elif rc != (f[0], f[1]):
                raise NotImplementedError('strided operands with different row structure')
    rows, cols = rc
    lds = [cols if a._contig else f[2] for a, f in zip(arrs, forms)]
    return rows, cols, lds


def _matrix(a):
    """(rows, cols, ld) of a 2-D array whose rows are contiguous."""
    if len(a.shape) != 2:
        raise ValueError('expected a 2-D array, got shape %r' % (a.shape,))
    rows, cols = a.shape
    if a._contig:
        return rows, cols, cols
    if cols > 1 and a.strides[1] != 1:
        raise NotImplementedError('matrix view with a non-unit column stride')
    return rows, cols, a.strides[0] if rows > 1 else cols


class B200Handler(Handler):
    """Handler backend for one B200 GPU (one process per GPU).

    Args:
        seed: seed of ``self.rnd`` (host ``RandomState``) and of the device
            Philox streams.
        device: CUDA device ordinal; defaults to ``LOCAL_RANK`` or 0.
        rng_mode: ``'device'`` draws dropout masks / gaussians with the
            in-kernel Philox generator; ``'host'`` draws them from ``self.rnd``
            exactly like ``NumpyHandler`` (numpy_handler.py:193-200) and uploads
            them, for bit-parity runs.
        align_hubs: start every hub of a network's flat buffer on a 16-byte boundary
            (``brainstorm_b200.layout``): the reference packs hubs back to back, which
            leaves most of them at odd element offsets, where kernels cannot use 128-bit
            accesses and GEMM operands must be copied before TMA can fetch them.
    """
    __undescribed__ = {'context', 'dtype', 'EMPTY', 'rnd', 'device', 'seed', 'rng_mode',
                       '_scratch', '_flags', '_flag_host', '_rng_calls', '_label_check',
                       '_pinned', '_comm', 'axis0_reduce', 'align_hubs', '_axis0_skip'}

    array_type = B200Array

    def __init__(self, seed=None, device=None, rng_mode='device', align_hubs=True):
        super(B200Handler, self).__init__()
        import os
        if device is None:
            device = int(os.environ.get('LOCAL_RANK', '0'))
        check(lib.b200_init(int(device)))
        if rng_mode not in ('device', 'host'):
            raise ValueError("rng_mode must be 'device' or 'host'")
        self.dtype = np.float32
        self.context = 'b200:%d' % device
        self.device = int(device)
        self.rng_mode = rng_mode
        self.rnd = new_random_state(seed)
        self.seed = int(self.rnd.randint(0, 2 ** 31 - 1)) if seed is None else int(seed)
        self.EMPTY = B200Array.empty((0,))
        self._scratch = None
        self._flags = B200Array.empty((4,))       # [0] bad label, [1] non-finite (int bits)
        self._flag_host = (ctypes.c_int * 4)()
        self._rng_calls = 0
        self._label_check = False
        self._pinned = []
        self._comm = None
        self.axis0_reduce = 'local'
        self._axis0_skip = (0, 0)     # address range whose sums over the batch axis need no exchange of their own
        self.align_hubs = bool(align_hubs)

    def __describe__(self):
        return {'@type': self.__class__.__name__}

    def __init_from_description__(self, description):
        self.__init__()

    # ------------------------------------------------------------------ memory
    def allocate(self, shape):
        if self.align_hubs and type(shape) is tuple and len(shape) == 1:
            from .layout import align_calling_buffer_manager
            align_calling_buffer_manager()
        return B200Array.empty(shape, zero=True)

    def zeros(self, shape):
        return B200Array.empty(shape, zero=True)

    def ones(self, shape):
        a = B200Array.empty(shape, zero=False)
        self.fill(a, 1.0)
        return a

    def create_from_numpy(self, arr):
        arr = np.asarray(arr)
        a = B200Array.empty(arr.shape, zero=False)
        self.set_from_numpy(a, arr)
        return a

    def pinned_empty(self, shape, dtype=np.float32):
        """A numpy array backed by page-locked host memory: ``set_from_numpy``
        from it is a direct asynchronous DMA without a staging copy."""
        shape = (int(shape),) if np.isscalar(shape) else tuple(int(s) for s in shape)
        nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
        p = ctypes.c_void_p()
        check(lib.b200_host_alloc(_byref(p), max(nbytes, 1)))
        buf = (ctypes.c_char * max(nbytes, 1)).from_address(p.value)
        arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape, dtype=np.int64))).reshape(shape)
        self._pinned.append((p, buf))
        return arr

    def set_from_numpy(self, mem, arr):
        arr = np.asarray(arr)
        if arr.shape != mem.shape:
            if arr.size != mem.size:
                raise AssertionError('Shape of destination ({}) != Shape of source ({})'.format(
                    mem.shape, arr.shape))
            arr = arr.reshape(mem.shape)
        if mem.size == 0:
            return
        src = np.ascontiguousarray(arr, dtype=_f32)
        if mem._contig:
            check(lib.b200_memcpy_h2d(mem.ptr, src.ctypes.data, src.nbytes))
        else:
            form = mem.as_2d()
            if form is None:
                raise NotImplementedError('view with strides %r has no row-pitched form' % (mem.strides,))
            rows, cols, ld = form
            check(lib.b200_memcpy2d_h2d(mem.ptr, ld * 4, src.ctypes.data, cols * 4, cols * 4, rows))
        # Pageable sources are staged by the runtime before the call returns;
        # page-locked ones (pinned_empty) must stay untouched until synchronize().

    def upload_async(self, mem, arr, after_event=0):
        """Start copying the page-locked float32 array ``arr`` (see pinned_empty)
        into the device array ``mem`` (contiguous or row-pitched) on the upload
        stream, after the event ``after_event`` (record_event) if given.  Kernels
        queued after ``upload_join()`` see the data."""
        arr = np.asarray(arr)
        if arr.dtype != _f32 or not arr.flags.c_contiguous or arr.size != mem.size:
            raise ValueError('upload_async needs a contiguous float32 source of the same size')
        if mem._contig:
            check(lib.b200_upload_async(mem.ptr, arr.ctypes.data, arr.nbytes, after_event))
            return
        form = mem.as_2d()
        if form is None:
            raise NotImplementedError('view with strides %r has no row-pitched form' % (mem.strides,))
        rows, cols, ld = form
        check(lib.b200_upload2d_async(mem.ptr, ld * 4, arr.ctypes.data, cols * 4, cols * 4, rows, after_event))

    def upload_join(self):
        check(lib.b200_upload_join())

    def record_event(self, event=None):
        """Record (and create if needed) an event on the compute stream."""
        if event is None:
            e = ctypes.c_uint64()
            check(lib.b200_event_create(_byref(e)))
            event = e.value
        check(lib.b200_event_record(event))
        return event

    def get_numpy_copy(self, mem):
        assert type(mem) == self.array_type
        out = np.empty(mem.shape, dtype=_f32)
        if mem.size:
            if mem._contig:
                check(lib.b200_memcpy_d2h(out.ctypes.data, mem.ptr, out.nbytes))
            else:
                form = mem.as_2d()
                if form is None:
                    raise NotImplementedError('view with strides %r has no row-pitched form' % (mem.strides,))
                rows, cols, ld = form
                check(lib.b200_memcpy2d_d2h(out.ctypes.data, cols * 4, mem.ptr, ld * 4, cols * 4, rows))
        if self._label_check:
            self._raise_on_bad_labels()
        return out

    def device_info(self):
        """(device ordinal, SM count, free bytes, total bytes) of this handler's GPU."""
        dev, sms = ctypes.c_int(), ctypes.c_int()
        free, total = ctypes.c_uint64(), ctypes.c_uint64()
        check(lib.b200_device_info(_byref(dev), _byref(sms), _byref(free), _byref(total)))
        return dev.value, sms.value, free.value, total.value

    def prepare_network(self, net):
        """What a network should do to its buffers after ``net.set_handler(self)``: start
        every hub on a 16-byte boundary (``brainstorm_b200.layout.align_buffers``)."""
        from .layout import align_buffers
        return align_buffers(net)

    def record(self, fn, *args, **kwargs):
        """Record the handler calls of ``fn(*args, **kwargs)`` instead of executing
        them; returns a ``RecordedStep`` whose ``launch()`` replays them with one
        call (see ``brainstorm_b200.graph``)."""
        from .graph import record
        kwargs['handler'] = self
        return record(fn, *args, **kwargs)

    def synchronize(self):
        check(lib.b200_sync())
        if self._label_check:
            self._raise_on_bad_labels()

    def _raise_on_bad_labels(self):
        self._label_check = False
        check(lib.b200_memcpy_d2h(ctypes.addressof(self._flag_host), self._flags.ptr, 4))
        if self._flag_host[0]:
            check(lib.b200_fill(self._flags.ptr, 0.0, 1, 1, 1))
            raise IndexError('index_m_by_v: a label lies outside [0, number of columns)')

    def fill(self, mem, val):
        if mem._contig:
            check(lib.b200_fill(mem.ptr, val, 1, mem.size, mem.size))
        else:
            rows, cols, (ld,) = _views(mem)
            check(lib.b200_fill(mem.ptr, val, rows, cols, ld))

    def copy_to(self, src, dest):
        rows, cols, (lds, ldd) = _views(src, dest)
        check(lib.b200_copy_to(src.ptr, dest.ptr, rows, cols, lds, ldd))

    def is_fully_finite(self, a):
        flag = self._flags.ptr + 4
        check(lib.b200_fill(flag, 0.0, 1, 1, 1))
        rows, cols, (ld,) = _views(a)
        check(lib.b200_nonfinite_flag(a.ptr, rows, cols, ld, flag))
        check(lib.b200_memcpy_d2h(ctypes.addressof(self._flag_host), flag, 4))
        return self._flag_host[0] == 0

    # -------------------------------------------------------- tensor (.) tensor
    def _tt(self, fn, a, b, out):
        if a._contig and b._contig and out._contig:
            n = out.size
            if a.size != n or b.size != n:
                raise ValueError('operands differ in size: %r %r %r' % (a.shape, b.shape, out.shape))
            check(fn(a.ptr, b.ptr, out.ptr, 1, n, n, n, n))
        else:
            rows, cols, (lda, ldb, ldo) = _views(a, b, out)
            check(fn(a.ptr, b.ptr, out.ptr, rows, cols, lda, ldb, ldo))

    def add_tt(self, a, b, out):
        self._tt(lib.b200_add_tt, a, b, out)

    def subtract_tt(self, a, b, out):
        assert a.shape == b.shape == out.shape
        self._tt(lib.b200_subtract_tt, a, b, out)

    def mult_tt(self, a, b, out):
        self._tt(lib.b200_mult_tt, a, b, out)

    def divide_tt(self, a, b, out):
        self._tt(lib.b200_divide_tt, a, b, out)

    def modulo_tt(self, a, b, out):
        self._tt(lib.b200_modulo_tt, a, b, out)

    def mult_add_tt(self, a, b, out):
        self._tt(lib.b200_mult_add_tt, a, b, out)

    # -------------------------------------------------------- scalar (.) tensor
    def _st(self, fn, s, t, out):
        rows, cols, (ldt, ldo) = _views(t, out)
        check(fn(s, t.ptr, out.ptr, rows, cols, ldt, ldo))

    def add_st(self, s, t, out):
        self._st(lib.b200_add_st, s, t, out)

    def mult_st(self, s, t, out):
        self._st(lib.b200_mult_st, s, t, out)

    def mult_add_st(self, s, t, out):
        self._st(lib.b200_mult_add_st, s, t, out)

    # ------------------------------------------------- matrix (.) broadcast vector
    def _mv(self, fn, tt_fn, m, v, out):
        if v.shape == m.shape:
            return self._tt(tt_fn, m, v, out)
        rows, cols, ldm = _matrix(m)
        orows, ocols, ldo = _matrix(out)
        if (orows, ocols) != (rows, cols):
            raise ValueError('out has shape %r, expected %r' % (out.shape, m.shape))
        if v.shape == (1, cols):
            is_col = 0
        elif v.shape == (rows, 1):
            is_col = 1
        else:
            raise ValueError('vector of shape %r does not broadcast against %r' % (v.shape, m.shape))
        if not v._contig:
            v = self._contiguous_copy(v)
        check(fn(m.ptr, v.ptr, out.ptr, rows, cols, ldm, ldo, is_col))

    def add_mv(self, m, v, out):
        self._mv(lib.b200_add_mv, lib.b200_add_tt, m, v, out)

    def subtract_mv(self, m, v, out):
        self._mv(lib.b200_subtract_mv, lib.b200_subtract_tt, m, v, out)

    def mult_mv(self, m, v, out):
        self._mv(lib.b200_mult_mv, lib.b200_mult_tt, m, v, out)

    def divide_mv(self, m, v, out):
        self._mv(lib.b200_divide_mv, lib.b200_divide_tt, m, v, out)

    def mult_add_mv(self, m, v, out):
        self._mv(lib.b200_mult_add_mv, lib.b200_mult_add_tt, m, v, out)

    def broadcast_t(self, a, axis, out):
        assert (out.shape[:axis] + (1,) + out.shape[axis + 1:]) == a.shape
        if out.size == 0:
            return
        if not a._contig:
            a = self._contiguous_copy(a)
        if not out._contig:
            # a strided view (a feature slice of a hub with several sources,
            # buffer_structure.py:232-245): broadcast into a contiguous temporary,
            # then one row-pitched copy
            tmp = B200Array.empty(out.shape, zero=False)
            self.broadcast_t(a, axis, tmp)
            self.copy_to(tmp, out)
            return
        # out viewed as (outer, n_axis, inner); a as (outer, 1, inner)
        outer = int(np.prod(out.shape[:axis], dtype=np.int64))
        n_axis = out.shape[axis]
        inner = int(np.prod(out.shape[axis + 1:], dtype=np.int64))
        if outer == 1:
            check(lib.b200_broadcast_t(a.ptr, out.ptr, n_axis, inner, inner, 0))
        elif inner == 1:
            check(lib.b200_broadcast_t(a.ptr, out.ptr, outer, n_axis, n_axis, 1))
        else:
            for o in range(outer):
                check(lib.b200_broadcast_t(a.ptr + 4 * o * inner, out.ptr + 4 * o * n_axis * inner,
                                           n_axis, inner, inner, 0))

    # ----------------------------------------------------------------- unary
    def _unary(self, fn, a, out):
        if a._contig and out._contig:
            n = out.size
            if a.size != n:
                raise ValueError('operands differ in size: %r %r' % (a.shape, out.shape))
            check(fn(a.ptr, out.ptr, 1, n, n, n))
        else:
            rows, cols, (lda, ldo) = _views(a, out)
            check(fn(a.ptr, out.ptr, rows, cols, lda, ldo))

    def abs_t(self, a, out):
        self._unary(lib.b200_abs_t, a, out)

    def sign_t(self, a, out):
        self._unary(lib.b200_sign_t, a, out)

    def sqrt_t(self, a, out):
        self._unary(lib.b200_sqrt_t, a, out)

    def log_t(self, a, out):
        self._unary(lib.b200_log_t, a, out)

    def clip_t(self, a, a_min, a_max, out):
        assert a_max >= a_min
        rows, cols, (lda, ldo) = _views(a, out)
        check(lib.b200_clip_t(a.ptr, a_min, a_max, out.ptr, rows, cols, lda, ldo))

    # ------------------------------------------------------------- activations
    def sigmoid(self, x, y):
        self._unary(lib.b200_sigmoid, x, y)

    def tanh(self, x, y):
        self._unary(lib.b200_tanh, x, y)

    def rel(self, x, y):
        self._unary(lib.b200_rel, x, y)

    def el(self, x, y):
        self._unary(lib.b200_el, x, y)

    def _deriv(self, fn, y, dy, dx):
        if y._contig and dy._contig and dx._contig:
            n = dx.size
            if y.size != n or dy.size != n:
                raise ValueError('operands differ in size')
            check(fn(y.ptr, dy.ptr, dx.ptr, 1, n, n, n, n))
        else:
            rows, cols, (l0, l1, l2) = _views(y, dy, dx)
            check(fn(y.ptr, dy.ptr, dx.ptr, rows, cols, l0, l1, l2))

    def sigmoid_deriv(self, x, y, dy, dx):
        self._deriv(lib.b200_sigmoid_deriv, y, dy, dx)

    def tanh_deriv(self, x, y, dy, dx):
        self._deriv(lib.b200_tanh_deriv, y, dy, dx)

    def rel_deriv(self, x, y, dy, dx):
        self._deriv(lib.b200_rel_deriv, y, dy, dx)

    def el_deriv(self, x, y, dy, dx):
        self._deriv(lib.b200_el_deriv, y, dy, dx)

    # --------------------------------------------------------------- predicated
    def copy_to_if(self, src, dest, cond):
        rows, cols, (l0, l1, l2) = _views(src, dest, cond)
        check(lib.b200_copy_to_if(src.ptr, dest.ptr, cond.ptr, rows, cols, l0, l1, l2))

    def fill_if(self, mem, val, cond):
        rows, cols, (l0, l1) = _views(mem, cond)
        check(lib.b200_fill_if(mem.ptr, val, cond.ptr, rows, cols, l0, l1))

    def add_into_if(self, a, out, cond):
        rows, cols, (l0, l1, l2) = _views(a, out, cond)
        check(lib.b200_add_into_if(a.ptr, out.ptr, cond.ptr, rows, cols, l0, l1, l2))

    # ----------------------------------------------------------- concat / split
    def merge_tt(self, a, b, out):
        assert a.shape[-1] + b.shape[-1] == out.shape[-1]
        na, nb = a.shape[-1], b.shape[-1]
        if a._contig and b._contig and out._contig:
            rows = out.size // (na + nb) if na + nb else 0
            check(lib.b200_merge_tt(a.ptr, b.ptr, out.ptr, rows, na, nb))
            return
        # strided views: two row-pitched copies into the two column ranges of out
        if na and a.size:
            self.copy_to(a, out[..., :na])
        if nb and b.size:
            self.copy_to(b, out[..., na:])

    def split_add_tt(self, x, out_a, out_b):
        assert out_a.shape[-1] + out_b.shape[-1] == x.shape[-1]
        na, nb = out_a.shape[-1], out_b.shape[-1]
        if x._contig and out_a._contig and out_b._contig:
            rows = x.size // (na + nb) if na + nb else 0
            check(lib.b200_split_add_tt(x.ptr, out_a.ptr, out_b.ptr, rows, na, nb))
            return
        # strided views: two row-pitched accumulations from the two column ranges of x
        if na and out_a.size:
            self.add_tt(out_a, x[..., :na], out_a)
        if nb and out_b.size:
            self.add_tt(out_b, x[..., na:], out_b)

    # ------------------------------------------------------------------- labels
    def binarize_v(self, v, out):
        rows, cols, ldo = _matrix(out)
        if v.size != rows:
            raise ValueError('binarize_v: %d labels for %d rows' % (v.size, rows))
        ldv = 1 if v._contig else v.strides[0]
        check(lib.b200_binarize_v(v.ptr, ldv, out.ptr, rows, cols, ldo))

    def index_m_by_v(self, m, v, out):
        rows, cols, ldm = _matrix(m)
        if v.size != rows or out.size != rows:
            raise ValueError('index_m_by_v: operands disagree on the number of rows')
        ldv = 1 if v._contig else v.strides[0]
        ldo = 1 if out._contig else out.strides[0]
        check(lib.b200_index_m_by_v(m.ptr, ldm, v.ptr, ldv, out.ptr, ldo, rows, cols, self._flags.ptr))
        self._label_check = True

    # --------------------------------------------------------------- reductions
    def _scratch_for(self, floats):
        if floats <= 0:
            return 0, 0
        if self._scratch is None or self._scratch.size < floats:
            self._scratch = B200Array.empty((max(int(floats), 1 << 16),), zero=False)
        return self._scratch.ptr, self._scratch.size

    def sum_t(self, a, axis, out):
        assert axis is None or (len(a.shape) < 3 and (axis == 0 or axis == 1))
        if axis is None:
            rows, cols, (ld,) = _views(a)
            ax, nout = -1, 1
        else:
            if len(a.shape) == 1:
                if axis != 0:
                    raise ValueError('axis 1 is out of bounds for a 1-D array')
                rows, cols, (ld,) = _views(a)
                ax, nout = -1, 1
            else:
                rows, cols, ld = _matrix(a)
                ax, nout = axis, (cols if axis == 0 else rows)
        if out.size != nout:
            raise ValueError('sum_t: out has %d elements, expected %d' % (out.size, nout))
        dst = out if out._contig else B200Array.empty((nout,), zero=False)
        need = lib.b200_sum_t_scratch_floats(rows, cols, ld, ax)
        sp, sn = self._scratch_for(need)
        exchange = False
        if ax == 0 and self._comm is not None and self.axis0_reduce != 'local':
            lo, hi = self._axis0_skip
            exchange = not (lo <= out.ptr < hi)     # sums written into the gradient vector are averaged with it
        peer_ok = getattr(self._comm, '_peer_ok', None) if exchange else None
        if peer_ok is not None and peer_ok(dst):
            # sum and exchange as one kernel: its last block completes the sums across the ranks over peer memory
            check(lib.b200_sum_t_axis0_allreduce(a.ptr, rows, cols, ld, dst.ptr, sp, sn,
                                                 1 if self.axis0_reduce == 'avg' else 0))
        else:
            check(lib.b200_sum_t(a.ptr, rows, cols, ld, ax, dst.ptr, sp, sn))
            if exchange:
                self._allreduce_axis0(dst)
        if dst is not out:
            self.copy_to(dst.reshape(out.shape), out)

    def softmax_m(self, m, out):
        rows, cols, ldm = _matrix(m)
        orows, ocols, ldo = _matrix(out)
        if (rows, cols) != (orows, ocols):
            raise ValueError('softmax_m: shapes differ')
        check(lib.b200_softmax_m(m.ptr, out.ptr, rows, cols, ldm, ldo))

    # --------------------------------------------------------------------- GEMM
    def _gemm(self, fn, a, b, out, transa, transb):
        ar, ac, lda = _matrix(a)
        br, bc, ldb = _matrix(b)
        M, N, ldo = _matrix(out)
        am, ak = (ac, ar) if transa else (ar, ac)
        bk, bn = (bc, br) if transb else (br, bc)
        if am != M or bn != N or ak != bk:
            raise ValueError('shapes %r%s . %r%s -> %r do not agree' % (
                a.shape, '^T' if transa else '', b.shape, '^T' if transb else '', out.shape))
        check(fn(a.ptr, b.ptr, out.ptr, M, N, ak, lda, ldb, ldo, 1 if transa else 0, 1 if transb else 0))

    def dot_mm(self, a, b, out, transa=False, transb=False):
        self._gemm(lib.b200_dot_mm, a, b, out, transa, transb)

    def dot_add_mm(self, a, b, out, transa=False, transb=False):
        self._gemm(lib.b200_dot_add_mm, a, b, out, transa, transb)

    # ------------------------------------------------------------------- random
    def fill_gaussian(self, mean, std, out):
        if self.rng_mode == 'host':
            self.set_from_numpy(out, std * self.rnd.standard_normal(out.shape) + mean)
            return
        dst = out if out._contig else B200Array.empty(out.shape, zero=False)
        self._rng_calls += 1
        check(lib.b200_fill_gaussian(mean, std, dst.ptr, dst.size, self.seed, self._rng_calls))
        if dst is not out:
            self.copy_to(dst, out)

    def generate_probability_mask(self, mask, probability):
        if self.rng_mode == 'host':
            self.set_from_numpy(mask, self.rnd.uniform(size=mask.shape) < probability)
            return
        dst = mask if mask._contig else B200Array.empty(mask.shape, zero=False)
        self._rng_calls += 1
        check(lib.b200_generate_probability_mask(dst.ptr, dst.size, probability, self.seed,
                                                 self._rng_calls))
        if dst is not mask:
            self.copy_to(dst, mask)

    # ------------------------------------------------------- convolution / pooling
    @staticmethod
    def _nhwc(a, what):
        if len(a.shape) != 4 or not a._contig:
            raise ValueError('%s must be a contiguous (N, H, W, C) array, got %r' % (what, a.shape))
        return a.shape

    def conv2d_forward_batch(self, inputs, weights, bias, outputs, padding, stride):
        N, H, W, C = self._nhwc(inputs, 'inputs')
        F, kh, kw, wc = self._nhwc(weights, 'weights')
        on, oh, ow, of = self._nhwc(outputs, 'outputs')
        if wc != C or on != N or of != F:
            raise ValueError('conv2d_forward_batch: shapes %r, %r, %r do not agree' % (
                inputs.shape, weights.shape, outputs.shape))
        if N * oh * ow == 0:
            return
        K = kh * kw * C
        col = B200Array.empty((N * oh * ow, K), zero=False)
        check(lib.b200_im2col(inputs.ptr, col.ptr, N, H, W, C, kh, kw, padding, stride[0], stride[1], oh, ow))
        out2 = outputs.reshape((N * oh * ow, F))
        self.dot_mm(col, weights.reshape((F, K)), out2, transb=True)
        self.add_mv(out2, bias.reshape((1, F)), out2)

    def conv2d_backward_batch(self, inputs, params, padding, stride, in_deltas, out_deltas, dparams, dbias):
        N, H, W, C = self._nhwc(inputs, 'inputs')
        F, kh, kw, wc = self._nhwc(params, 'params')
        on, oh, ow, of = self._nhwc(out_deltas, 'out_deltas')
        self._nhwc(in_deltas, 'in_deltas')
        if wc != C or on != N or of != F or in_deltas.shape != inputs.shape:
            raise ValueError('conv2d_backward_batch: shapes do not agree')
        K = kh * kw * C
        if N * oh * ow == 0:
            self.fill(dparams, 0.0)
            self.fill(dbias, 0.0)
            return
        col = B200Array.empty((N * oh * ow, K), zero=False)
        check(lib.b200_im2col(inputs.ptr, col.ptr, N, H, W, C, kh, kw, padding, stride[0], stride[1], oh, ow))
        od = out_deltas.reshape((N * oh * ow, F))
        # the reference overwrites the gradients (fill 0, then the sum over images)
        self.dot_mm(od, col, dparams.reshape((F, K)), transa=True)
        self.sum_t(od, 0, dbias.reshape((F,)) if dbias._contig else dbias)
        self.dot_mm(od, params.reshape((F, K)), col)
        check(lib.b200_col2im_add(col.ptr, in_deltas.ptr, N, H, W, C, kh, kw, padding, stride[0], stride[1], oh, ow))

    def _pool(self, fwd, mode, inputs, window, outputs, padding, stride, argmax, in_deltas, out_deltas):
        N, H, W, C = self._nhwc(inputs, 'inputs')
        on, oh, ow, oc = self._nhwc(outputs, 'outputs')
        if on != N or oc != C:
            raise ValueError('pooling: inputs %r and outputs %r do not agree' % (inputs.shape, outputs.shape))
        am = argmax.ptr if argmax is not None else 0
        if fwd:
            check(lib.b200_pool2d_forward(mode, inputs.ptr, outputs.ptr, am, N, H, W, C, window[0], window[1],
                                          padding, stride[0], stride[1], oh, ow))
        else:
            self._nhwc(in_deltas, 'in_deltas')
            self._nhwc(out_deltas, 'out_deltas')
            check(lib.b200_pool2d_backward(mode, out_deltas.ptr, am, in_deltas.ptr, N, H, W, C, window[0],
                                           window[1], padding, stride[0], stride[1], oh, ow))

    def maxpool2d_forward_batch(self, inputs, window, outputs, padding, stride, argmax):
        self._nhwc(argmax, 'argmax')
        self._pool(True, 0, inputs, window, outputs, padding, stride, argmax, None, None)

    def maxpool2d_backward_batch(self, inputs, window, outputs, padding, stride, argmax, in_deltas, out_deltas):
        self._pool(False, 0, inputs, window, outputs, padding, stride, argmax, in_deltas, out_deltas)

    def avgpool2d_forward_batch(self, inputs, window, outputs, padding, stride):
        self._pool(True, 1, inputs, window, outputs, padding, stride, None, None, None)

    def avgpool2d_backward_batch(self, inputs, window, outputs, padding, stride, in_deltas, out_deltas):
        self._pool(False, 1, inputs, window, outputs, padding, stride, None, in_deltas, out_deltas)

    # ------------------------------------------------------------------ helpers
    def _contiguous_copy(self, a):
        c = B200Array.empty(a.shape, zero=False)
        self.copy_to(a, c)
        return c

    def set_comm(self, comm, axis0_reduce='local'):
        """Complete ``sum_t(axis=0)`` across batch shards: ``'sum'`` / ``'avg'``
        all-reduce the result over ``comm`` (brainstorm_b200.parallel.Comm),
        ``'local'`` exchanges nothing."""
        if axis0_reduce not in ('local', 'sum', 'avg'):
            raise ValueError("axis0_reduce must be 'local', 'sum' or 'avg'")
        self._comm = comm
        self.axis0_reduce = axis0_reduce
        self._axis0_skip = (0, 0)

    def _allreduce_axis0(self, dst):
        self._comm.allreduce(dst, self.axis0_reduce)


_default = [None]


def _any_handler():
    if _default[0] is None:
        _default[0] = B200Handler()
    return _default[0]


def _array_binary(op, a, b):
    h = _any_handler()
    out = B200Array.empty(a.shape, zero=False)
    if isinstance(b, B200Array):
        h.mult_tt(a, b, out)
    else:
        h.mult_st(float(b), a, out)
    return out


def _array_pow(a, exponent):
    h = _any_handler()
    out = B200Array.empty(a.shape, zero=False)
    if exponent == 0.5:
        h.sqrt_t(a, out)
    elif exponent == 2:
        h.mult_tt(a, a, out)
    elif exponent == 1:
        h.copy_to(a, out)
    else:
        raise NotImplementedError('B200Array ** %r' % (exponent,))
    return out
