"""Fused compute+collective kernels on 2 GPUs (child processes; skipped with fewer than 2 devices)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _dist_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_comm_kernels_two_ranks():
    rc, out, err = run_ranks(os.path.join(HERE, "dist_worker_comm_gpu.py"), 29621, multimem=True)
    assert rc == 0 and "COMM_OK" in out, out[-3000:] + err[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fused", ["1", "0"])
def test_tp_rollout_engine_two_ranks(fused):
    """fused=1: decode GEMMs with the all-reduce in their epilogue (peer reductions + arrival counters);
    fused=0: library GEMMs + the all-reduce kernel."""
    rc, out, err = run_ranks(os.path.join(HERE, "dist_worker_tp_rollout_gpu.py"), 29622 + 20 * int(fused),
                             extra_env={"TRL_B200_TP_FUSED": fused})
    assert rc == 0 and "TP_ROLLOUT_OK" in out, out[-3000:] + err[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_rollout_engine_with_expert_layers():
    """Mixture-of-experts model under tensor parallelism: every expert sliced along its intermediate dimension."""
    rc, out, err = run_ranks(os.path.join(HERE, "dist_worker_tp_rollout_gpu.py"), 29682,
                             extra_env={"TRL_B200_TP_FUSED": "0", "TP_TEST_MOE": "1"})
    assert rc == 0 and "TP_ROLLOUT_OK" in out, out[-3000:] + err[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_full_shard_engine_two_ranks():
    rc, out, err = run_ranks(os.path.join(HERE, "dist_worker_fullshard_gpu.py"), 29623)
    assert rc == 0 and "FULLSHARD_OK" in out, out[-3000:] + err[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_moe_two_ranks():
    rc, out, err = run_ranks(os.path.join(HERE, "dist_worker_ep_moe_gpu.py"), 29627)
    assert rc == 0 and "EP_MOE_OK" in out, out[-3000:] + err[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("tiled", ["0", "1"])
def test_weight_reshard_from_full_shard_to_tp_layout(tiled):
    """tiled=1: the rollout engine keeps its slices tile-major (fused TP decode), the reshard re-tiles per layer."""
    rc, out, err = run_ranks(os.path.join(HERE, "dist_worker_reshard_gpu.py"), 29629 + 40 * int(tiled),
                             extra_env={"TRL_B200_TP_FUSED": tiled})
    assert rc == 0 and "RESHARD_OK" in out, out[-3000:] + err[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fused", [1, 0])
def test_streamed_full_shard_engine_two_ranks(fused):
    """fused=1: slices pulled over peer loads on a side stream and per-layer gradient reduction by the own kernel;
    fused=0: the backend's all-gather / reduce-scatter."""
    rc, out, err = run_ranks(os.path.join(HERE, "dist_worker_streamshard_gpu.py"), 29631 + 20 * fused,
                             extra_env={"TRL_B200_STREAM_FUSED": str(fused)})
    assert rc == 0 and "STREAMSHARD_OK" in out, out[-3000:] + err[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_model_trains_like_replicated_experts():
    rc, out, err = run_ranks(os.path.join(HERE, "dist_worker_ep_model_gpu.py"), 29671)
    assert rc == 0 and "EP_MODEL_OK" in out, out[-3000:] + err[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sequence_and_context_parallel_match_one_rank_on_gpus():
    rc, out, err = run_ranks(os.path.join(HERE, "dist_worker_spcp_gpu.py"), 29681)
    assert rc == 0 and "SPCP_OK" in out, out[-3000:] + err[-3000:]
