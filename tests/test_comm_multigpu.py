"""Fused compute+collective kernels on 2 GPUs (child processes; skipped with fewer than 2 devices)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_comm_kernels_two_ranks():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29621", os.path.join(HERE, "dist_worker_comm_gpu.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0 and "COMM_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_rollout_engine_two_ranks():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29622", os.path.join(HERE, "dist_worker_tp_rollout_gpu.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0 and "TP_ROLLOUT_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_full_shard_engine_two_ranks():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29623", os.path.join(HERE, "dist_worker_fullshard_gpu.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0 and "FULLSHARD_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_moe_two_ranks():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29627", os.path.join(HERE, "dist_worker_ep_moe_gpu.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0 and "EP_MOE_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_weight_reshard_from_full_shard_to_tp_layout():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29629", os.path.join(HERE, "dist_worker_reshard_gpu.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0 and "RESHARD_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_streamed_full_shard_engine_two_ranks():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29631", os.path.join(HERE, "dist_worker_streamshard_gpu.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0 and "STREAMSHARD_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
