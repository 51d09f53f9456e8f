"""Worker of tests/test_multi_gpu.py: one rank per GPU (torch.distributed.run), on as many
GPUs as the box shows (2, 4 or 8).
Each rank trains on its batch shard with B200Handler + data_parallel; rank 0 checks
the result against the single-process run of the reference stack on NumpyHandler
with the whole batch."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, 'baseline', '_ref')):
    sys.path.insert(0, p)


def main():
    import torch
    import torch.distributed as dist
    local = int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, world = dist.get_rank(), dist.get_world_size()
    from brainstorm.handlers import NumpyHandler
    from brainstorm_b200 import B200Handler, workloads
    from brainstorm_b200.fused_lstm import fuse_lstm_layers
    from brainstorm_b200 import parallel
    from brainstorm_b200.parallel import Comm, data_parallel, shard_batch
    from brainstorm_b200.workloads import train_steps
    from brainstorm_b200._lib import lib, check
    H = B200Handler(seed=3, device=local)
    ok = True
    # ---- the library's all-reduce over peer memory against NCCL, op by op
    plain, peer = Comm(), Comm()
    peer_on = peer.enable_peer()
    if rank == 0:
        print('PEER_ON' if peer_on else 'PEER_OFF')
    if peer_on:
        rs = np.random.RandomState(100 + rank)
        for n in (1, 5, 1000, 4096, 65536):
            for op in ('sum', 'avg'):
                for rep in range(3):             # repeated calls walk through both slots
                    x = rs.randn(n).astype(np.float32)
                    a, b = H.create_from_numpy(x), H.create_from_numpy(x)
                    plain.allreduce(a, op)
                    peer.allreduce(b, op)
                    got, want = H.get_numpy_copy(b), H.get_numpy_copy(a)
                    gathered = [None] * world
                    dist.all_gather_object(gathered, got)
                    same = all(np.array_equal(g, gathered[0]) for g in gathered)
                    close = np.allclose(got, want, rtol=1e-6, atol=1e-6)
                    if not (same and close):
                        ok = False
                        if rank == 0:
                            print('peer all-reduce n=%d %s: replicas equal %s, max diff to NCCL %.3g' % (
                                n, op, same, np.abs(got - want).max()))
        # the column sum with the exchange inside its kernel against the sum followed by NCCL
        for rows, cols in ((4096, 4096), (300, 1027), (64, 8), (20000, 512)):
            x = np.random.RandomState(7 * rank + rows).randn(rows, cols).astype(np.float32)
            a = H.create_from_numpy(x)
            for op, in_kernel in (('sum', 1), ('avg', 1), ('sum', 0), ('avg', 0)):
                check(lib.b200_set_tuning(12, in_kernel))
                want, got = H.zeros((1, cols)), H.zeros((1, cols))
                H.sum_t(a, 0, want)
                plain.allreduce(want, op)
                two_calls = H.zeros((1, cols))
                H.sum_t(a, 0, two_calls)
                peer.allreduce(two_calls, op)
                H.set_comm(peer, op)
                H.sum_t(a, 0, got)
                H.set_comm(None, 'local')
                g, w = H.get_numpy_copy(got), H.get_numpy_copy(want)
                if not np.array_equal(g, H.get_numpy_copy(two_calls)):
                    ok = False
                    print('fused column sum (%d, %d) %s: bits differ from sum_t + peer all-reduce on rank %d' % (rows, cols, op, rank))
                gathered = [None] * world
                dist.all_gather_object(gathered, g)
                same = all(np.array_equal(v, gathered[0]) for v in gathered)
                close = np.allclose(g, w, rtol=1e-6, atol=1e-5 * np.abs(x).sum(0).max())
                if not (same and close):
                    ok = False
                    if rank == 0:
                        print('fused column sum (%d, %d) %s: replicas equal %s, max diff to NCCL %.3g' % (
                            rows, cols, op, same, np.abs(g - w).max()))
        check(lib.b200_set_tuning(12, 0))
        peer.close()
    for which, build, mode in (
            ('highway_bn', lambda: workloads.highway_bn(batch=32 * world, width=64, classes=7, blocks=2), 'avg'),
            ('highway_bn_fused', lambda: workloads.highway_bn(batch=32 * world, width=64, classes=7, blocks=2), 'avg'),
            ('lstm', lambda: workloads.lstm(time=6, batch=16 * world, vocab=20, hidden=32), 'local')):
        net, data, stepper = build()
        net.set_handler(H)
        if which == 'lstm':
            fuse_lstm_layers(net)
        if which == 'highway_bn_fused':
            from brainstorm_b200.fused_layers import fuse_layers
            assert len(fuse_layers(net)) == 2 * 4 + 1
        # one network with an all-reduce per layer (what large networks get), one with a single one
        parallel.OVERLAP_MIN_BYTES = 0 if which.startswith('highway_bn') else (1 << 40)
        data_parallel(net, Comm(), axis0_reduce=mode, peer=True)
        losses = train_steps(net, shard_batch(data, rank, world), stepper(), 3)
        params = net.get('parameters')
        gathered = [None] * world
        dist.all_gather_object(gathered, (params, losses))
        if rank == 0:
            ref, rdata, rstepper = build()
            ref.set_handler(NumpyHandler(np.float32))
            rl = train_steps(ref, rdata, rstepper(), 3)
            want = ref.get('parameters')
            for r, (p, l) in enumerate(gathered):
                assert np.array_equal(p, gathered[0][0]), '%s: replicas diverged on rank %d' % (which, r)
            scale = np.abs(want).max()
            err = np.abs(params - want).max()
            mean_loss = np.mean([g[1] for g in gathered], axis=0)
            print('%s: param err %.3g (scale %.3g), loss %s vs %s' % (which, err, scale, mean_loss, rl))
            ok = ok and err <= 1e-4 * scale and np.allclose(mean_loss, rl, rtol=1e-4)
    if rank == 0:
        print('MULTI_GPU_OK' if ok else 'MULTI_GPU_MISMATCH')
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
