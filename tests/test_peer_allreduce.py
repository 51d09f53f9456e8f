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


def test_a_rank_that_never_arrives_makes_the_wait_run_out_and_is_reported():
    """Failure detection without a fault: "rank 1" is a second window of this process
    that nobody ever publishes to, and the wait's poll limit is set to a few
    milliseconds.  The kernel must return by itself, leave dst alone, raise the device
    error flag (reported by the next synchronising call) and switch the peer path off;
    ordinary calls keep working and a new registration brings the path back."""
    from brainstorm_b200 import B200Handler, B200Error
    from brainstorm_b200._lib import lib, check
    H = B200Handler(seed=1)
    handles = [ctypes.create_string_buffer(64) for _ in range(2)]
    wins = [ctypes.c_uint64() for _ in range(2)]
    for w, h in zip(wins, handles):
        check(lib.b200_peer_window_alloc(ctypes.byref(w), h))
    windows = (ctypes.c_uint64 * 2)(wins[0].value, wins[1].value)
    check(lib.b200_peer_setup(0, 2, windows))
    check(lib.b200_set_tuning(8, 12))                 # 2^12 polls: about 12 ms
    try:
        assert lib.b200_peer_enabled() == 1
        x = np.arange(1000, dtype=np.float32)
        src, dst = H.create_from_numpy(x), H.ones((1000,))
        H.synchronize()
        check(lib.b200_peer_allreduce(src.ptr, dst.ptr, 1000, 0))     # queued; rank 1 never comes
        with pytest.raises(B200Error, match='gave up waiting'):
            H.synchronize()
        assert lib.b200_peer_enabled() == 0
        assert np.all(H.get_numpy_copy(dst) == 1.0)                   # flag cleared, dst untouched
        assert lib.b200_peer_allreduce(src.ptr, dst.ptr, 1000, 0) != 0
        assert b'switched off' in lib.b200_last_error()
        H.add_tt(src, src, dst)                                       # the library is still usable
        assert np.array_equal(H.get_numpy_copy(dst), 2 * x)
        # registering again (alone this time) clears the counters and brings the path back
        check(lib.b200_peer_setup(0, 1, (ctypes.c_uint64 * 1)(wins[0].value)))
        assert lib.b200_peer_enabled() == 1
        check(lib.b200_peer_allreduce(src.ptr, dst.ptr, 1000, 0))
        assert np.array_equal(H.get_numpy_copy(dst), x)
    finally:
        check(lib.b200_set_tuning(8, 0))              # back to the default limit
        lib.b200_sync()
        check(lib.b200_peer_teardown())               # frees window 0 (this rank's)
        check(lib.b200_peer_window_release(wins[1].value, 1))


def _sum0_fused(H, lib, check, x, average, in_kernel=1):
    check(lib.b200_set_tuning(12, in_kernel))       # 1: the exchange inside the column-sum kernel; 0: the kernel behind it
    a = H.create_from_numpy(x)
    out = H.create_from_numpy(np.full((x.shape[1],), np.nan, np.float32))
    sp, sn = H._scratch_for(lib.b200_sum_t_scratch_floats(x.shape[0], x.shape[1], x.shape[1], 0))
    check(lib.b200_sum_t_axis0_allreduce(a.ptr, x.shape[0], x.shape[1], x.shape[1], out.ptr, sp, sn, average))
    return out


@pytest.mark.parametrize('rows,cols', [(8, 4), (64, 33), (5000, 128), (4096, 4096), (300, 1027), (70000, 12)])
def test_column_sum_with_the_exchange_inside_the_kernel_single_rank(rows, cols):
    """With one rank the completed sums are the local ones: the kernel's second ticket level,
    the hand-over to the exchange and the counters' return to zero, call after call."""
    from brainstorm_b200 import B200Handler
    from brainstorm_b200._lib import lib, check
    H = B200Handler(seed=1)
    handle = ctypes.create_string_buffer(64)
    window = ctypes.c_uint64()
    check(lib.b200_peer_window_alloc(ctypes.byref(window), handle))
    check(lib.b200_peer_setup(0, 1, (ctypes.c_uint64 * 1)(window.value)))
    try:
        x = np.random.RandomState(rows + cols).randn(rows, cols).astype(np.float32)
        a, want = H.create_from_numpy(x), H.zeros((1, cols))
        H.sum_t(a, 0, want)
        want = H.get_numpy_copy(want).ravel()
        for call in range(6):                      # both forms, interleaved: they share slots and call numbers
            got = H.get_numpy_copy(_sum0_fused(H, lib, check, x, call % 2, in_kernel=1 if call % 3 else 0))
            assert np.array_equal(got, want), 'call %d' % call
        calls, waited = ctypes.c_uint64(), ctypes.c_uint64()
        check(lib.b200_peer_wait_stats(ctypes.byref(calls), ctypes.byref(waited)))
        assert calls.value == 6
    finally:
        check(lib.b200_set_tuning(12, 0))
        H.synchronize()
        check(lib.b200_peer_teardown())


def test_column_sum_whose_exchange_gives_up_keeps_the_local_sums():
    """The fused form of the failure path above: "rank 1" never arrives, the wait inside the
    column-sum kernel runs out after a few milliseconds, the kernel returns, `out` holds the
    local sums, the error is reported at the next synchronising call and the path is off."""
    from brainstorm_b200 import B200Handler, B200Error
    from brainstorm_b200._lib import lib, check
    H = B200Handler(seed=1)
    handles = [ctypes.create_string_buffer(64) for _ in range(2)]
    wins = [ctypes.c_uint64() for _ in range(2)]
    for w, h in zip(wins, handles):
        check(lib.b200_peer_window_alloc(ctypes.byref(w), h))
    check(lib.b200_peer_setup(0, 2, (ctypes.c_uint64 * 2)(wins[0].value, wins[1].value)))
    check(lib.b200_set_tuning(8, 12))                 # 2^12 polls: about 12 ms
    try:
        x = np.random.RandomState(5).randn(3000, 256).astype(np.float32)
        a, want = H.create_from_numpy(x), H.zeros((1, 256))
        H.sum_t(a, 0, want)
        want = H.get_numpy_copy(want).ravel()
        out = _sum0_fused(H, lib, check, x, 0)        # queued; rank 1 never comes
        with pytest.raises(B200Error, match='gave up waiting'):
            H.synchronize()
        assert lib.b200_peer_enabled() == 0
        assert np.array_equal(H.get_numpy_copy(out), want)
        sp, sn = H._scratch_for(lib.b200_sum_t_scratch_floats(3000, 256, 256, 0))
        assert lib.b200_sum_t_axis0_allreduce(a.ptr, 3000, 256, 256, out.ptr, sp, sn, 0) != 0
        assert b'no usable peer registration' in lib.b200_last_error()
        got = H.zeros((1, 256))
        H.sum_t(a, 0, got)                            # ordinary column sums still work: the tickets are back at zero
        assert np.array_equal(H.get_numpy_copy(got).ravel(), want)
    finally:
        check(lib.b200_set_tuning(8, 0))
        check(lib.b200_set_tuning(12, 0))
        lib.b200_sync()
        check(lib.b200_peer_teardown())
        check(lib.b200_peer_window_release(wins[1].value, 1))
