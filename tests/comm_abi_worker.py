"""Worker of tests/test_multi_gpu.py::test_all_reduce_through_the_c_abi_without_a_framework:
one process per GPU, no torch, no torch.distributed.  The NCCL id travels through a file,
as any host could pass it; everything else is libb200handler.so through ctypes."""
import ctypes
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, id_file = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    from brainstorm_b200 import B200Handler
    from brainstorm_b200._lib import lib, check
    H = B200Handler(seed=rank, device=rank)
    ident = ctypes.create_string_buffer(128)
    if rank == 0:
        check(lib.b200_comm_unique_id(ident))
        with open(id_file + '.tmp', 'wb') as f:
            f.write(ident.raw)
        os.rename(id_file + '.tmp', id_file)
    else:
        for _ in range(600):
            if os.path.exists(id_file):
                break
            time.sleep(0.1)
        with open(id_file, 'rb') as f:
            ident = ctypes.create_string_buffer(f.read(), 128)
    check(lib.b200_comm_init(rank, world, ident))
    assert lib.b200_comm_world() == world
    rs = [np.random.RandomState(10 + r) for r in range(world)]
    ok = True
    for n in (1, 1000, 1 << 20):
        parts = [r.randn(n).astype(np.float32) for r in rs]          # every rank can compute all ranks' inputs
        want = np.sum(np.stack(parts).astype(np.float64), axis=0)
        scale = np.sum(np.abs(np.stack(parts)).astype(np.float64), axis=0)
        for average, asynchronous in ((0, False), (1, False), (0, True)):
            x = H.create_from_numpy(parts[rank])
            if asynchronous:
                check(lib.b200_comm_allreduce_async(x.ptr, n, average))
                H.mult_st(2.0, H.ones((8,)), H.ones((8,)))            # work that runs beside the collective
                check(lib.b200_comm_join())
            else:
                check(lib.b200_comm_allreduce(x.ptr, n, average))
            got = H.get_numpy_copy(x).astype(np.float64)
            ref = want / world if average else want
            ok = ok and bool(np.all(np.abs(got - ref) <= 1e-5 * np.abs(ref) + 1e-5 * scale / (world if average else 1)))
    # the same call recorded into a graph and replayed on new data
    x = H.create_from_numpy(np.full(64, rank + 1.0, np.float32))
    step = H.record(lambda: check(lib.b200_comm_allreduce(x.ptr, 64, 0)))
    for k in range(2):
        H.fill(x, rank + 1.0 + k)
        step.launch()
        ok = ok and bool(np.all(H.get_numpy_copy(x) == sum(r + 1.0 + k for r in range(world))))
    step.release()
    H.synchronize()
    check(lib.b200_comm_destroy())
    assert 'torch' not in sys.modules
    print('COMM_ABI_OK' if ok else 'COMM_ABI_MISMATCH')


if __name__ == '__main__':
    main()
