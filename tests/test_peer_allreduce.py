"""The library's all-reduce over peer memory with a single rank (one GPU): the kernel's
own mechanics -- slot parity, epoch publication, bounded wait, rank-order sum.  The
multi-rank behaviour is covered by tests/test_multi_gpu.py on two GPUs."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_single_rank_all_reduce_is_the_identity_through_both_slots():
    from brainstorm_b200 import B200Handler
    from brainstorm_b200._lib import lib, check
    H = B200Handler(seed=1)
    handle = ctypes.create_string_buffer(64)
    window = ctypes.c_uint64()
    check(lib.b200_peer_window_alloc(ctypes.byref(window), handle))
    windows = (ctypes.c_uint64 * 1)(window.value)
    check(lib.b200_peer_setup(0, 1, windows))
    try:
        rs = np.random.RandomState(0)
        for n in (1, 31, 4096, 65536):
            for call in range(3):                      # epochs 1, 2, 3: slots 1, 0, 1
                x = rs.randn(n).astype(np.float32)
                src, dst = H.create_from_numpy(x), H.zeros((n,))
                check(lib.b200_peer_allreduce(src.ptr, dst.ptr, n, call % 2))
                assert np.array_equal(H.get_numpy_copy(dst), x)
                check(lib.b200_peer_allreduce(src.ptr, src.ptr, n, 0))      # in place
                assert np.array_equal(H.get_numpy_copy(src), x)
        assert lib.b200_peer_allreduce(src.ptr, src.ptr, 65537, 0) != 0     # too long: refused, nothing queued
        assert b'at most' in lib.b200_last_error()
    finally:
        H.synchronize()
        check(lib.b200_peer_teardown())
