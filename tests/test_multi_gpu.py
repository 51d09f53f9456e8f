"""Batch-sharded training on all visible B200s (2, 4 or 8; NCCL and the library's own
all-reduce over peer memory) equals the single-process run of the reference stack on
the whole batch.  Needs two visible GPUs; skipped otherwise (the CPU half of the same
check runs in tests/test_parallel_gloo.py)."""
import os
import subprocess
import sys

import pytest

from conftest import needs_reference, ROOT

pytestmark = [pytest.mark.gpu, needs_reference]


def test_sharded_training_matches_global_batch():
    import torch
    gpus = torch.cuda.device_count()
    if gpus < 2:
        pytest.skip('needs two GPUs')
    world = 8 if gpus >= 8 else (4 if gpus >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    out = subprocess.run([sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', str(world),
                          '--master-addr', '127.0.0.1', '--master-port', '29533',
                          os.path.join(ROOT, 'tests', 'multi_gpu_worker.py')],
                         capture_output=True, text=True, timeout=600, env=env)
    assert 'MULTI_GPU_OK' in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
    # the all-reduce over peer memory must really have been in use on this box
    assert 'PEER_ON' in out.stdout, out.stdout[-3000:]


def test_all_reduce_through_the_c_abi_without_a_framework(tmp_path):
    """b200_comm_*: a host that binds libb200handler.so and nothing else (no torch in the
    worker processes) gets the gradient all-reduce, blocking, overlapped and recorded."""
    import torch
    gpus = torch.cuda.device_count()
    if gpus < 2:
        pytest.skip('needs two GPUs')
    world = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    id_file = str(tmp_path / 'nccl_id')
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, 'tests', 'comm_abi_worker.py'), str(r), str(world), id_file],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env) for r in range(world)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0 and 'COMM_ABI_OK' in out, out[-2000:] + err[-3000:]
