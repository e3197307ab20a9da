"""The sharded Evoformer stack as separate processes exchanging over NCCL, one per GPU.  Needs at least two GPUs on the
box (skipped on a single-GPU box, where tests/test_gpu_sharded.py covers the same partitioned path with the ranks as host
threads)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_two_processes_over_nccl_match_the_unsharded_stack(lib):
    env = dict(os.environ, NCCL_NVLS_ENABLE='0', PYTHONPATH=ROOT + os.pathsep + os.environ.get('PYTHONPATH', ''))
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2', '--master-addr', '127.0.0.1',
           '--master-port', '29541', '-m', 'bindcraft2_b200.shard_check', '--n-res', '256', '--msa-rows', '2', '--depth', '2']
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    line = [l for l in r.stdout.splitlines() if l.startswith('{')][-1]
    rep = json.loads(line)
    print(rep)
    assert rep['ok'] and rep['pair_rel_l2'] <= 1e-3 and rep['d_pair_rel_l2'] <= 2e-2
