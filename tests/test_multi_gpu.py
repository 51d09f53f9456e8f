"""Batch-sharded training on two B200s (NCCL) equals the single-process run of
the reference stack on the whole batch.  Needs two visible GPUs; skipped otherwise
(the CPU half of the same check runs in tests/test_parallel_gloo.py)."""
import os
import subprocess
import sys

import pytest

from conftest import needs_reference, ROOT

pytestmark = [pytest.mark.gpu, needs_reference]


def test_two_rank_training_matches_global_batch():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    out = subprocess.run([sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2',
                          '--master-addr', '127.0.0.1', '--master-port', '29533',
                          os.path.join(ROOT, 'tests', 'multi_gpu_worker.py')],
                         capture_output=True, text=True, timeout=600, env=env)
    assert 'MULTI_GPU_OK' in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
    # the all-reduce over peer memory must really have been in use on this box
    assert 'PEER_ON' in out.stdout, out.stdout[-3000:]
