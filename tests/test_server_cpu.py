"""Generation server: data-parallel worker processes over pipes, packed weight updates, the log-prob batching window,
and the spawned rollout worker of asynchronous GRPO talking to it.  Failures are made on the host (a server that is
not there, a reward function that raises)."""
import socket
import threading
import time

import numpy as np
import pytest
import torch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Server:
    def __init__(self, pool):
        import uvicorn

        from trl_b200.scripts.rollout_serve import build_app

        self.port = _free_port()
        self.app = build_app(pool)
        self.server = uvicorn.Server(uvicorn.Config(self.app, host="127.0.0.1", port=self.port, log_level="error"))
        self.thread = threading.Thread(target=self.server.run, daemon=True)
        self.pool = pool

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *exc):
        self.server.should_exit = True
        self.thread.join(timeout=10)
        self.pool.close()


def test_data_parallel_workers_packed_updates_and_logprob_batching():
    from trl_b200.generation import RolloutClient
    from trl_b200.scripts.rollout_serve import ServeArguments, WorkerPool
    from trl_b200.testing import make_tiny_model

    pool = WorkerPool(ServeArguments(model="preset:tiny-qwen2", data_parallel_size=2, max_model_len=64))
    assert len(pool.procs) == 2 and pool.world_size == 2
    with _Server(pool) as srv:
        c = RolloutClient(host="127.0.0.1", server_port=srv.port, connection_timeout=30)
        prompts = [[5, 6, 7], [8, 9, 10], [11, 12], [13, 14, 15, 16], [17]]
        out = c.generate(prompts, n=2, max_tokens=4, generation_kwargs={"seed": 3})
        assert len(out["completion_ids"]) == 10 and out["prompt_ids"] == prompts  # request order, both replicas
        info = c.init_communicator()
        assert "packed" in info["transports"] and info["world_size"] == 2
        # new weights reach BOTH replicas in one packed body: their log-probs then equal a local model with those weights
        local = make_tiny_model("tiny-qwen2")
        with torch.no_grad():
            for p in local.parameters():
                p.add_(0.05 * torch.randn_like(p))
        assert c.update_model_params(local, transport="packed") == len(local.state_dict_hf())
        seqs = [p + o for p, o in zip([q for q in prompts for _ in range(2)], out["completion_ids"])]
        pls = [len(q) for q in prompts for _ in range(2)]
        lps = c.get_sequence_logprobs(seqs, pls)
        from trl_b200.scripts.rollout_serve import EngineHolder

        ref = EngineHolder.sequence_logprobs(type("H", (), {"model": local, "max_model_len": 64})(), seqs, pls)
        for a, b in zip(lps, ref):
            assert a.shape == b.shape and np.allclose(a, b, atol=1e-4)
        # concurrent requests inside the window are scored together
        before = srv.app.state.logprob_batcher.batches
        res = [None] * 6
        ths = [threading.Thread(target=lambda i=i: res.__setitem__(i, RolloutClient(host="127.0.0.1", server_port=srv.port)
                                                                    .get_sequence_logprobs(seqs[i:i + 1], pls[i:i + 1]))) for i in range(6)]
        [t.start() for t in ths]
        [t.join(timeout=60) for t in ths]
        assert all(r is not None and np.allclose(r[0], ref[i], atol=1e-4) for i, r in enumerate(res))
        assert srv.app.state.logprob_batcher.batches - before < 6
        c.reset_prefix_cache()


def _len_reward(prompts, completions, completion_ids, **kw):
    return [float(len(c)) for c in completion_ids]


def _broken_reward(prompts, completions, completion_ids, **kw):
    raise RuntimeError("reward exploded")


def test_process_rollout_worker_feeds_samples_and_reports_failures(tiny_tokenizer):
    from trl_b200.experimental.async_grpo.async_grpo_trainer import _ServerSideReward
    from trl_b200.experimental.async_grpo.async_rollout_worker import ProcessRolloutWorker
    from trl_b200.scripts.rollout_serve import ServeArguments, WorkerPool

    pool = WorkerPool(ServeArguments(model="preset:tiny-qwen2", max_model_len=64))
    with _Server(pool) as srv:
        url = f"http://127.0.0.1:{srv.port}"
        rows = [{"prompt": [5, 6, 7, 8], "prompt_text": "a"}, {"prompt": [9, 10], "prompt_text": "b"}]
        w = ProcessRolloutWorker(rows, url, _ServerSideReward([_len_reward], tiny_tokenizer), num_generations=2, max_tokens=5,
                                 prompts_per_call=2, max_inflight=2, server_timeout=30)
        w.update_model_version(7)
        w.start()
        try:
            got = [w.get(timeout=60) for _ in range(8)]
            w.check_health(60)
            assert all(s.model_version == 7 and 1 <= len(s.completion_ids) <= 5 and len(s.logprobs) == len(s.completion_ids) for s in got)
            by_group = {}
            for s in got:
                by_group.setdefault(s.group_id, []).append(s)
            full = [g for g in by_group.values() if len(g) == 2]
            assert full and all(abs(g[0].advantage + g[1].advantage) < 1e-4 for g in full)  # group-centred
        finally:
            w.stop()
        assert not w._proc.is_alive()
        # a reward function that raises in the child surfaces in check_health on the parent
        bad = ProcessRolloutWorker(rows, url, _ServerSideReward([_broken_reward], tiny_tokenizer), num_generations=2,
                                   max_tokens=3, prompts_per_call=1, server_timeout=30)
        bad.start()
        try:
            deadline = time.time() + 60
            with pytest.raises(RuntimeError, match="reward exploded|rollout worker"):
                while time.time() < deadline:
                    bad.check_health(120)
                    time.sleep(0.2)
                raise AssertionError("no failure reported")
        finally:
            bad.stop()
    # no server at all: the child gives up after its deadline and says so
    nowhere = ProcessRolloutWorker(rows, f"http://127.0.0.1:{_free_port()}", _ServerSideReward([_len_reward], tiny_tokenizer),
                                   num_generations=2, server_timeout=2)
    nowhere.start()
    try:
        deadline = time.time() + 60
        with pytest.raises(RuntimeError, match="not healthy|rollout worker"):
            while time.time() < deadline:
                nowhere.check_health(120)
                time.sleep(0.2)
            raise AssertionError("no failure reported")
    finally:
        nowhere.stop()


def test_grpo_trains_against_the_rollout_server(tmp_path, tiny_tokenizer):
    """`vllm_mode="server"`: completions come from the server over HTTP, the policy's weights are pushed to it before
    every generation batch (after the push the server's log-probs follow the trained policy)."""
    from trl_b200 import GRPOConfig, GRPOTrainer
    from trl_b200.generation.server_rollout import ServerRollout
    from trl_b200.scripts.rollout_serve import ServeArguments, WorkerPool
    from trl_b200.testing import make_dataset, make_tiny_model

    pool = WorkerPool(ServeArguments(model="preset:tiny-qwen2", data_parallel_size=1, max_model_len=96))
    with _Server(pool) as srv:
        model = make_tiny_model("tiny-qwen2", seed=0)
        args = GRPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, num_generations=4, max_completion_length=6,
                          max_steps=2, logging_steps=1, learning_rate=5e-3, use_cpu=True, save_strategy="no", report_to="none",
                          beta=0.0, use_vllm=True, vllm_mode="server", vllm_server_host="127.0.0.1",
                          vllm_server_port=srv.port, vllm_server_timeout=30)
        seen = []

        def reward(completion_ids, **kw):
            seen.append(len(completion_ids))
            return [float(sum(c) % 5) for c in completion_ids]
        tr = GRPOTrainer(model, reward, args, train_dataset=make_dataset("standard_prompt_only", 8), processing_class=tiny_tokenizer)
        tr.train()
        assert isinstance(tr._rollout, ServerRollout) and tr._rollout.stats["requests"] >= 2 and sum(seen) >= 8
        logs = [h for h in tr.state.log_history if "reward" in h]
        assert len(logs) == 2 and all(np.isfinite(h["loss"]) for h in logs)
        # the server holds the weights of the last push: after one more push its log-probs equal the trained policy's
        tr._rollout.sync_weights()
        seq = [5, 6, 7, 8, 9, 10, 11]
        got = tr._rollout.client.get_sequence_logprobs([seq], [3])[0]
        with torch.no_grad():
            lp = torch.log_softmax(model(input_ids=torch.tensor([seq])).logits[0].float(), -1)
        want = lp[torch.arange(2, 6), torch.tensor(seq[3:])]
        assert np.allclose(got, want.numpy(), atol=1e-4), (got, want)
