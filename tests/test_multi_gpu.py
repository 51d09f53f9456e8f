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
