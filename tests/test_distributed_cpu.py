"""Distributed equivalence on CPU (gloo): the same global batch trained with world_size 1 and 2, in
ddp and zero2 modes, must give the same loss / grad-norm trajectory."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, mode, out, steps=4, port=29611):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    if world == 1:
        cmd = [sys.executable, os.path.join(HERE, "dist_worker_sft.py"), out, mode, str(steps)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dist_worker_sft.py"), out,
               mode, str(steps)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    with open(out) as f:
        return json.load(f)


_SFT_REF = {}


@pytest.mark.parametrize("mode,port", [("ddp", 29611), ("zero2", 29612), ("sp2", 29613), ("cp2", 29614), ("full_shard_stream", 29615)])
def test_sft_world1_vs_world2(tmp_path, tmp_path_factory, mode, port):
    if "sft_w1" not in _SFT_REF:  # the single-process trajectory is the same for every mode: run it once
        _SFT_REF["sft_w1"] = _run(1, "ddp", str(tmp_path_factory.mktemp("w1") / "w1.json"))
    ref = _SFT_REF["sft_w1"]
    two = _run(2, mode, str(tmp_path / f"w2_{mode}.json"), port=port)
    assert len(ref) == len(two) == 4
    for a, b in zip(ref, two):
        assert abs(a["loss"] - b["loss"]) < 2e-4, (ref, two)
        assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-3 * max(1.0, a["grad_norm"]), (ref, two)
    assert ref[-1]["loss"] < ref[0]["loss"] + 0.05


def test_custom_optimizer_sharded_over_two_ranks_matches_one_rank(tmp_path):
    """SGD with momentum through `optim`: zero2 over two ranks (every rank updates its half of the master copy, the
    momentum buffers are sharded with it) follows the single-process trajectory."""
    ref = _run(1, "ddp+sgd", str(tmp_path / "w1.json"))
    two = _run(2, "zero2+sgd", str(tmp_path / "w2.json"), port=29616)
    assert len(ref) == len(two) == 4
    for a, b in zip(ref, two):
        assert abs(a["loss"] - b["loss"]) < 2e-4, (ref, two)
        assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-3 * max(1.0, a["grad_norm"]), (ref, two)
    assert ref[-1]["loss"] < ref[0]["loss"] + 0.05 and ref[-1]["loss"] != ref[0]["loss"]


def _run_stream(world, mode, variant, out, port, load=True):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    worker = os.path.join(HERE, "dist_worker_stream.py")
    if world == 1:
        cmd = [sys.executable, worker, out, mode, variant]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), worker, out, mode, variant]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    if not load:
        return None
    from safetensors.torch import load_file

    return load_file(os.path.join(out, "final", "model.safetensors"))


_REF_CACHE = {}


def _ddp_reference(tmp_path_factory):
    """Weights of the uninterrupted world-1 ddp run (3 steps), computed once per session."""
    if "ref" not in _REF_CACHE:
        _REF_CACHE["ref"] = _run_stream(1, "ddp", "straight", str(tmp_path_factory.mktemp("ddp_ref")), 0)
    return _REF_CACHE["ref"]


def test_streamed_full_shard_saves_and_resumes_like_ddp(tmp_path, tmp_path_factory):
    """Weights after 3 steps (weight decay on): world-1 ddp == world-2 streamed shards == world-2 streamed shards with a
    checkpoint after step 2 and a resume in a new trainer."""
    import torch

    ref = _ddp_reference(tmp_path_factory)
    a = _run_stream(2, "full_shard_stream", "straight", str(tmp_path / "s"), 29616)
    b = _run_stream(2, "full_shard_stream", "resume", str(tmp_path / "r"), 29617)
    assert set(ref) == set(a) == set(b)
    for k in ref:
        # (three AdamW steps amplify summation-order differences between one and two ranks; the resume check below,
        # same world size on both sides, stays tight)
        assert torch.allclose(ref[k], a[k], atol=1e-4), (k, (ref[k] - a[k]).abs().max())
        assert torch.allclose(a[k], b[k], atol=1e-6), (k, (a[k] - b[k]).abs().max())


@pytest.mark.parametrize("kind,port", [("dense", 29618), ("moe", 29620)])
def test_grpo_with_streamed_shards_matches_zero2(tmp_path, kind, port):
    """Online RL on sharded weights: the generation replica refreshed from the slices must give the same samples, rewards
    and updates as generation from the policy in place."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    res = {}
    for j, mode in enumerate(("zero2", "full_shard_stream")):
        out = str(tmp_path / f"{mode}.json")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
               "127.0.0.1", "--master-port", str(port + j), os.path.join(HERE, "dist_worker_grpo_stream.py"), out, mode, kind]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
        with open(out) as f:
            res[mode] = json.load(f)
    a, b = res["zero2"], res["full_shard_stream"]
    assert len(a) == len(b) == 3
    for x, y in zip(a, b):
        assert x["reward"] == y["reward"], (a, b)  # same samples
        assert abs(x["loss"] - y["loss"]) < 2e-4 and abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, x["grad_norm"]), (a, b)


@pytest.mark.parametrize("mode1,world1,mode2,world2,port", [("zero2", 2, "ddp", 1, 29622), ("ddp", 1, "zero2", 2, 29624),
                                                             ("full_shard_stream", 2, "full_shard_stream", 1, 29626)])
def test_elastic_resume_with_another_world_size(tmp_path, tmp_path_factory, mode1, world1, mode2, world2, port):
    """Two steps with one world size / shard mode, checkpoint, third step with another: the optimizer slices are put
    back together and cut again, and the weights end where an uninterrupted run ends."""
    import torch

    ref = _ddp_reference(tmp_path_factory)
    out = str(tmp_path / "el")
    _run_stream(world1, mode1, "phase1", out, port, load=False)
    got = _run_stream(world2, mode2, "phase2", out, port + 1)
    for k in ref:  # AdamW at lr 1e-3 turns summation-order noise into up to a few 1e-5; a wrong slice shows as 1e-3
        assert torch.allclose(ref[k], got[k], atol=1e-4), (k, (ref[k] - got[k]).abs().max())


def test_grpo_completions_are_dealt_to_ranks_by_length(tmp_path):
    """After scoring, the job's completions are exchanged (token ids only) so that the ranks train on equal work."""
    out = str(tmp_path / "bal.json")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(HERE, "dist_worker_grpo_balance.py"), out, "1"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    with open(out) as f:
        res = json.load(f)
    r0, r1 = res["calls"]
    assert len(r0) == len(r1) >= 1
    for a, b in zip(r0, r1):
        # the job keeps exactly the same (completion, advantage) pairs; each rank keeps its sample count
        assert sorted(map(tuple, a["before"] + b["before"])) == sorted(map(tuple, a["after"] + b["after"]))
        assert len(a["after"]) == len(a["before"]) == len(b["after"])
        # token counts end up at least as even as they started
        assert abs(a["tok_after"] - b["tok_after"]) <= abs(a["tok_before"] - b["tok_before"])
        assert a["tok_after"] + b["tok_after"] == a["tok_before"] + b["tok_before"]
    assert len(res["log"]) == 2 and all(h["loss"] == h["loss"] for h in res["log"])


def test_balanced_partition_is_deterministic_and_even():
    from trl_b200.trainer.utils import balanced_partition

    costs = [1000, 10, 20, 990, 500, 480, 30, 15]
    parts = balanced_partition(costs, 2, 4)
    assert sorted(i for p in parts for i in p) == list(range(8)) and all(len(p) == 4 for p in parts)
    loads = [sum(costs[i] for i in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= 40 and parts == balanced_partition(costs, 2, 4)
    with pytest.raises(ValueError):
        balanced_partition(costs, 3, 3)


_EP_REF = {}


@pytest.mark.parametrize("mode,port", [("ddp", 29651), ("zero2", 29652)])
def test_expert_parallel_sft_matches_replicated_experts(tmp_path, tmp_path_factory, mode, port):
    """Experts split over two ranks (tokens exchanged with all-to-all, expert gradients unreduced and scaled by
    1 / world, optimizer state whole on the owner) must train like one process holding every expert, and the saved
    checkpoint must hold all of them."""

    def run(world, mode, out, port):
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
        worker = os.path.join(HERE, "dist_worker_ep_sft.py")
        cmd = ([sys.executable, worker, out, mode, "4"] if world == 1 else
               [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
                "127.0.0.1", "--master-port", str(port), worker, out, mode, "4"])
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
        with open(out) as f:
            return json.load(f)

    if "w1" not in _EP_REF:
        _EP_REF["w1"] = run(1, "ddp", str(tmp_path_factory.mktemp("epw1") / "w1.json"), 0)
    ref, two = _EP_REF["w1"], run(2, mode, str(tmp_path / f"ep_{mode}.json"), port)
    assert len(ref["hist"]) == len(two["hist"]) == 4
    for a, b in zip(ref["hist"], two["hist"]):
        assert abs(a["loss"] - b["loss"]) < 3e-4, (ref["hist"], two["hist"])
        assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-3 * max(1.0, a["grad_norm"]), (ref["hist"], two["hist"])
    # sums over whole matrices after four AdamW steps: elements whose gradients sit at rounding level move differently
    # (Adam normalises them), so the sums agree to a fraction of the total movement (4096+ elements x 4e-4), not bit-wise
    for k, v in ref["digest"].items():
        assert abs(v - two["digest"][k]) < 2e-3, k


def test_server_rollout_with_two_training_ranks():
    """`vllm_mode="server"` with two training processes: prompts gathered, one request by the main process, every rank
    gets its own completions back; one weight push for the job."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29631", os.path.join(HERE, "dist_worker_server_rollout.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "SERVER_ROLLOUT_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
