"""Device array views for the B200 handler.

The reference's memory layer creates ONE flat allocation per network
(brainstorm/structure/buffers.py:79) and hands out slices and reshapes of it
(buffers.py:82, buffer_structure.py:218-245); layers index time steps with
negative ints and slices (lstm_layer.py:106-117).  ``B200Array`` is therefore a
(base allocation, element offset, shape, strides) view with numpy-like
``shape / size / reshape / __getitem__``; it never owns memory itself.
"""
from __future__ import annotations

import numpy as np

from ._lib import lib, check

import ctypes

_ITEM = 4  # bytes per fp32 element


class Allocation(object):
    """One stream-ordered device allocation; freed when the last view dies."""
    __slots__ = ('ptr', 'nbytes', '__weakref__')

    def __init__(self, nbytes, zero=True):
        p = ctypes.c_uint64(0)
        check(lib.b200_malloc(ctypes.byref(p), int(nbytes), 1 if zero else 0))
        self.ptr = p.value
        self.nbytes = int(nbytes)

    def __del__(self):
        ptr, self.ptr = getattr(self, 'ptr', 0), 0
        if ptr:
            try:
                lib.b200_free(ptr)
            except Exception:  # interpreter shutdown
                pass


def _c_strides(shape):
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= max(int(s), 1) if s != 0 else 1
    return tuple(reversed(st))


def _norm_shape(shape):
    if isinstance(shape, (int, np.integer)):
        return (int(shape),)
    return tuple(int(s) for s in shape)


class B200Array(object):
    __slots__ = ('base', 'ptr', 'shape', 'strides', 'size', '_contig')
    dtype = np.dtype(np.float32)

    def __init__(self, base, ptr, shape, strides=None):
        self.base = base
        self.ptr = ptr
        self.shape = shape
        size = 1
        for s in shape:
            size *= s
        self.size = size
        if strides is None:
            self.strides = _c_strides(shape)
            self._contig = True
        else:
            self.strides = strides
            self._contig = size <= 1 or _is_c_contiguous(shape, strides)

    # -- construction ---------------------------------------------------------
    @classmethod
    def empty(cls, shape, zero=True):
        shape = _norm_shape(shape)
        n = 1
        for s in shape:
            if s < 0:
                raise ValueError('negative dimension in shape %r' % (shape,))
            n *= s
        base = Allocation(n * _ITEM, zero)
        return cls(base, base.ptr, shape)

    # -- numpy-like surface used by the reference's memory layer -----------------
    @property
    def ndim(self):
        return len(self.shape)

    @property
    def nbytes(self):
        return self.size * _ITEM

    @property
    def is_contiguous(self):
        return self._contig

    def __len__(self):
        if not self.shape:
            raise TypeError('len() of a 0-d array')
        return self.shape[0]

    def __repr__(self):
        return '<B200Array shape=%r strides=%r ptr=0x%x>' % (self.shape, self.strides, self.ptr)

    def reshape(self, *shape):
        if len(shape) == 1:
            shape = shape[0]
        shape = list(_norm_shape(shape))
        if shape.count(-1) > 1:
            raise ValueError('can only specify one unknown dimension')
        if -1 in shape:
            known = 1
            for s in shape:
                if s != -1:
                    known *= s
            if known == 0 or self.size % known:
                raise ValueError('cannot reshape array of size %d into shape %r' % (self.size, tuple(shape)))
            shape[shape.index(-1)] = self.size // known
        shape = tuple(shape)
        n = 1
        for s in shape:
            n *= s
        if n != self.size:
            raise ValueError('cannot reshape array of size %d into shape %r' % (self.size, shape))
        if self._contig:
            return B200Array(self.base, self.ptr, shape)
        strides = _reshape_strides(self.shape, self.strides, shape)
        if strides is None:
            raise ValueError('this strided view cannot be reshaped to %r without a copy' % (shape,))
        return B200Array(self.base, self.ptr, shape, strides)

    def __getitem__(self, key):
        # fast path: one integer into a contiguous array (time-step indexing in the
        # recurrent layers: y[t - 1], Za[t], ...)
        if self._contig and type(key) is int and self.shape:
            n = self.shape[0]
            if key < 0:
                key += n
            if not 0 <= key < n:
                raise IndexError('index out of bounds for axis 0 with size %d' % n)
            sub = B200Array.__new__(B200Array)
            sub.base = self.base
            sub.shape = self.shape[1:]
            sub.strides = self.strides[1:]
            sub.size = self.size // n if n else 0
            sub.ptr = self.ptr + key * sub.size * _ITEM
            sub._contig = True
            return sub
        if not isinstance(key, tuple):
            key = (key,)
        if any(k is Ellipsis for k in key):
            i = next(j for j, k in enumerate(key) if k is Ellipsis)
            fill = len(self.shape) - (len(key) - 1)
            key = key[:i] + (slice(None),) * fill + key[i + 1:]
        if len(key) > len(self.shape):
            raise IndexError('too many indices for array')
        off = 0
        shape, strides = [], []
        for d, k in enumerate(key):
            n, st = self.shape[d], self.strides[d]
            if isinstance(k, (int, np.integer)):
                k = int(k)
                if k < 0:
                    k += n
                if not 0 <= k < n:
                    raise IndexError('index out of bounds for axis %d with size %d' % (d, n))
                off += k * st
            elif isinstance(k, slice):
                start, stop, step = k.indices(n)
                if step <= 0:
                    raise IndexError('only positive slice steps are supported')
                length = max(0, (stop - start + step - 1) // step)
                off += start * st if length else 0
                shape.append(length)
                strides.append(st * step)
            else:
                raise IndexError('unsupported index %r' % (k,))
        shape.extend(self.shape[len(key):])
        strides.extend(self.strides[len(key):])
        return B200Array(self.base, self.ptr + off * _ITEM, tuple(shape), tuple(strides))

    # -- the only arithmetic the reference does on arrays directly
    #    (value_modifiers.py:78-80: `mat * mat` and `sq_norm ** 0.5`) ------------
    def __mul__(self, other):
        from .handler import _array_binary
        return _array_binary('mult', self, other)

    __rmul__ = __mul__

    def __pow__(self, exponent):
        from .handler import _array_pow
        return _array_pow(self, exponent)

    # -- interop -------------------------------------------------------------------
    @property
    def __cuda_array_interface__(self):
        return {'shape': self.shape, 'typestr': '<f4', 'data': (self.ptr, False), 'version': 3,
                'strides': None if self._contig else tuple(s * _ITEM for s in self.strides)}

    def as_2d(self):
        """(rows, cols, ld): the view as `rows` rows of `cols` contiguous
        elements with a uniform row pitch, or None if it has no such form."""
        if self._contig:
            return 1, self.size, self.size
        shape, strides = self.shape, self.strides
        dims = [(n, s) for n, s in zip(shape, strides) if n != 1]
        if not dims:
            return 1, 1, 1
        # merge trailing dims that are contiguous into the row
        cols, k = 1, len(dims)
        while k > 0 and dims[k - 1][1] == cols:
            cols *= dims[k - 1][0]
            k -= 1
        if k == 0:
            return 1, cols, cols
        ld = dims[k - 1][1]
        rows = dims[k - 1][0]
        for j in range(k - 2, -1, -1):
            if dims[j][1] != ld * rows:
                return None
            rows *= dims[j][0]
        return rows, cols, ld


def _is_c_contiguous(shape, strides):
    acc = 1
    for n, s in zip(reversed(shape), reversed(strides)):
        if n == 1:
            continue
        if s != acc:
            return False
        acc *= n
    return True


def _reshape_strides(old_shape, old_strides, new_shape):
    """Strides of a copy-free reshape of a strided view, or None."""
    old = [(n, s) for n, s in zip(old_shape, old_strides) if n != 1]
    if any(n == 0 for n in new_shape):
        return _c_strides(new_shape)
    new_strides = [0] * len(new_shape)
    oi = ni = 0
    while oi < len(old) and ni < len(new_shape):
        # grow a group of old dims and a group of new dims of equal size
        on, nn = old[oi][0], new_shape[ni]
        oj, nj = oi + 1, ni + 1
        while on != nn:
            if on < nn:
                on *= old[oj][0]
                oj += 1
            else:
                nn *= new_shape[nj]
                nj += 1
        # the old group must be internally contiguous
        for k in range(oi, oj - 1):
            if old[k][1] != old[k + 1][1] * old[k + 1][0]:
                return None
        st = old[oj - 1][1]
        for k in range(nj - 1, ni - 1, -1):
            new_strides[k] = st
            st *= new_shape[k]
        oi, ni = oj, nj
    for k in range(ni, len(new_shape)):  # trailing 1-dims
        new_strides[k] = 1
    return tuple(new_strides)
