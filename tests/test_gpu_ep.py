"""Expert parallelism on two GPUs: each rank's expert-parallel engine (its expert shard + NCCL all-gather /
reduce-scatter) must give the bits its single-GPU engine gives on the same sequences. One process per GPU."""
import os
import signal
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("nccl_only", [False, True])
def test_two_rank_expert_parallel_equals_single_gpu(nccl_only):
    """Default: many-row passes dispatch and combine by packed all-to-all, and the one-token step exchanges rows and results
    through peer memory (stores over NVLink into CUDA-IPC-mapped regions, flags with bounded waits). nccl_only: every pass
    uses the NCCL all-gather / reduce-scatter form (which batched decode steps always use). Both must give the single-GPU
    engine's bits."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if nccl_only:
        env["ITB_EP_A2A_OFF"] = "1"; env["ITB_EP_P2P"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29511", "-m", "tests.ep_check"]
    # own process group, so that a rank stuck in a collective is ended with the launcher instead of outliving the test
    p = subprocess.Popen(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True)
    try:
        out, err = p.communicate(timeout=300)
    except subprocess.TimeoutExpired:
        os.killpg(p.pid, signal.SIGKILL)
        out, err = p.communicate()
        pytest.fail("expert-parallel check timed out\n" + out[-2000:] + err[-2000:])
    assert p.returncode == 0, out[-2000:] + err[-2000:]
    assert out.count("ep_check ok") == 2
