"""Expert-parallel layer on 2+ GPUs of one box: dispatch and combine over
NVLink peer stores, checked against the CPU oracle of the whole world.  Each
rank is a child process (torchrun); skipped when fewer than two GPUs are
visible."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'multirank_worker.py')


def _run(world):
    env = dict(os.environ, NCCL_NVLS_ENABLE='0', GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS='5')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={world}',
           '--master-addr', '127.0.0.1', '--master-port', str(29650 + world), WORKER]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    # ranks share stdout: two JSON objects may end up on one line
    lines, decoder, text, pos = [], json.JSONDecoder(), out.stdout, 0
    while (pos := text.find('{"rank"', pos)) >= 0:
        obj, end = decoder.raw_decode(text, pos)
        lines.append(obj)
        pos = end
    assert len(lines) == world, out.stdout[-2000:] + out.stderr[-4000:]
    for line in lines:
        assert line['failures'] == [], line
    assert out.returncode == 0, out.stderr[-2000:]


@pytest.mark.parametrize('world', [2, 4, 8])
def test_expert_parallel_layer(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    _run(world)
