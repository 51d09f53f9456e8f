"""The GEMM kernel that runs a 256 x 256 tile on a pair of SMs (tcgen05 cta_group::2,
opt-in through tuning key 7) against float64: all four transpose forms, odd numbers of
row tiles (the last pair has an idle half), ragged edges, split-K, accumulation."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def H():
    from brainstorm_b200 import B200Handler
    return B200Handler(seed=3)


@pytest.fixture()
def pair_kernel():
    from brainstorm_b200._lib import lib, check
    check(lib.b200_set_tuning(2, 2))      # tensor cores only
    check(lib.b200_set_tuning(3, 256))    # 256-wide tiles
    check(lib.b200_set_tuning(7, 1))      # on pairs of SMs
    yield
    check(lib.b200_set_tuning(7, 0))
    check(lib.b200_set_tuning(3, 0))
    check(lib.b200_set_tuning(2, 0))


@pytest.mark.parametrize('M,N,K', [(256, 256, 64), (300, 700, 1000), (1000, 1000, 2500), (130, 520, 4096),
                                   (128, 1000, 4000), (2000, 250, 6400)])
@pytest.mark.parametrize('ta,tb', [(False, True), (False, False), (True, True), (True, False)])
def test_pair_kernel_matches_float64(H, pair_kernel, M, N, K, ta, tb):
    from brainstorm_b200._lib import lib
    rs = np.random.RandomState(M + N + K)
    a = rs.randn(*((K, M) if ta else (M, K))).astype(np.float32)
    b = rs.randn(*((N, K) if tb else (K, N))).astype(np.float32)
    c0 = rs.randn(M, N).astype(np.float32)
    A = (a.T if ta else a).astype(np.float64)
    B = (b.T if tb else b).astype(np.float64)
    da, db = H.create_from_numpy(a), H.create_from_numpy(b)
    for accumulate in (False, True):
        dc = H.create_from_numpy(c0)
        before = lib.b200_launch_count()
        (H.dot_add_mm if accumulate else H.dot_mm)(da, db, dc, transa=ta, transb=tb)
        H.synchronize()
        assert lib.b200_launch_count() > before
        ref = A @ B + (c0 if accumulate else 0)
        terms = np.abs(A) @ np.abs(B) + (np.abs(c0) if accumulate else 0)
        err = np.abs(H.get_numpy_copy(dc) - ref)
        assert np.all(err <= 1e-5 * np.abs(ref) + 1e-5 * terms), (err / terms).max()


def test_pair_kernel_same_sign_operands_keep_relative_accuracy(H, pair_kernel):
    rs = np.random.RandomState(5)
    a = rs.uniform(0, 1, (256, 16384)).astype(np.float32)
    b = rs.uniform(0, 1, (512, 16384)).astype(np.float32)
    dc = H.zeros((256, 512))
    H.dot_mm(H.create_from_numpy(a), H.create_from_numpy(b), dc, transb=True)
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    assert (np.abs(H.get_numpy_copy(dc) - ref) / ref).max() < 5e-6
