"""Multi-GPU gates: fused GEMM+all-reduce and TP argmax against NCCL twins, TP engine losslessness."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(nproc: int, *args, timeout=600, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "tp_worker.py"), *args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    return r.returncode, r.stdout + r.stderr


def test_fused_collectives_two_ranks():
    rc, out = _launch(2)
    assert rc == 0 and "TP_WORKER_OK" in out, out[-3000:]


def test_one_shot_allreduce_two_ranks():
    """The one-shot form (every rank receives every partial; the default is the two-shot form), engine included."""
    rc, out = _launch(2, "engine", JETSPEC_TP_ALLREDUCE="ll")
    assert rc == 0 and "TP_WORKER_OK" in out, out[-3000:]


def test_tp_engine_two_ranks():
    rc, out = _launch(2, "engine")
    assert rc == 0 and "TP_WORKER_OK" in out, out[-3000:]


def test_expert_parallel_engine_two_ranks():
    """Token-sharded expert parallelism inside the engine: each rank's own request, sharded experts."""
    rc, out = _launch(2, "ep_engine")
    assert rc == 0 and "TP_WORKER_OK" in out, out[-3000:]


def test_disaggregated_draft_head_two_ranks():
    rc, out = _launch(2, "disagg")
    assert rc == 0 and "TP_WORKER_OK" in out, out[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp_engine_four_ranks():
    rc, out = _launch(4, "engine")
    assert rc == 0 and "TP_WORKER_OK" in out, out[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_tp_engine_eight_ranks():
    rc, out = _launch(8, "engine", timeout=900)
    assert rc == 0 and "TP_WORKER_OK" in out, out[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_expert_parallel_engine_four_ranks():
    rc, out = _launch(4, "ep_engine")
    assert rc == 0 and "TP_WORKER_OK" in out, out[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_expert_parallel_engine_eight_ranks():
    """Eight requests with prompts of 2 .. 6 prefill chunks and different round counts, 16 experts per rank."""
    rc, out = _launch(8, "ep_engine", timeout=900)
    assert rc == 0 and "TP_WORKER_OK" in out, out[-3000:]
