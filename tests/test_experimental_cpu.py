"""Experimental trainers: two optimizer steps each on the tiny fixtures (CPU, fp32), parameters move, metrics logged."""
import pytest
import torch

from trl_b200.testing import make_dataset, make_tiny_model

COMMON = dict(per_device_train_batch_size=4, max_steps=2, logging_steps=1, learning_rate=1e-3, use_cpu=True,
              save_strategy="no", report_to="none")


def _snap(model):
    return {n: p.detach().clone() for n, p in model.named_parameters()}


def _unchanged(model, before):
    return [n for n, p in model.named_parameters() if p.requires_grad and n in before and torch.equal(before[n], p)]


@pytest.mark.parametrize("loss_type,extra", [("sigmoid", {}), ("simpo", {"cpo_alpha": 0.0}), ("ipo", {}), ("hinge", {}),
                                             ("sigmoid", {"alpha": 0.5})])
def test_cpo_family(tmp_path, tiny_tokenizer, loss_type, extra):
    from trl_b200.experimental.cpo import CPOConfig, CPOTrainer

    model = make_tiny_model()
    before = _snap(model)
    tr = CPOTrainer(model, CPOConfig(output_dir=str(tmp_path), loss_type=loss_type, **COMMON, **extra),
                    train_dataset=make_dataset("standard_preference", 16), processing_class=tiny_tokenizer)
    assert tr.ref_model is None
    tr.train()
    assert _unchanged(model, before) == []
    h = [x for x in tr.state.log_history if "rewards/chosen" in x][-1]
    assert "nll_loss" in h and "rewards/margins" in h


def test_orpo(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.orpo import ORPOConfig, ORPOTrainer
    from trl_b200.experimental.orpo.orpo_trainer import log1mexp

    x = torch.tensor([-1e-3, -0.5, -5.0, -30.0], dtype=torch.float64)
    assert torch.allclose(log1mexp(x), torch.log(1 - torch.exp(x)), atol=1e-9)
    model = make_tiny_model()
    before = _snap(model)
    tr = ORPOTrainer(model, ORPOConfig(output_dir=str(tmp_path), **COMMON),
                     train_dataset=make_dataset("conversational_preference", 16), processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []
    h = [x for x in tr.state.log_history if "log_odds_ratio" in x][-1]
    assert h["log_odds_ratio"] < 0


def test_tpo_three_branches(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.tpo import TPOConfig, TPOTrainer

    ds = [dict(ex, reference=ex["chosen"] + " indeed") for ex in make_dataset("standard_preference", 16)]
    model = make_tiny_model()
    before = _snap(model)
    tr = TPOTrainer(model, TPOConfig(output_dir=str(tmp_path), loss_type="tpo-l", **COMMON), train_dataset=ds,
                    processing_class=tiny_tokenizer)
    batch = next(iter(tr.get_train_dataloader()))
    assert batch["input_ids"].shape[0] == 12  # chosen, rejected and gold rows of 4 examples
    tr.train()
    assert _unchanged(model, before) == []
    assert any("gold_nll_loss" in h for h in tr.state.log_history)


def test_bco_running_moments_and_training(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.bco import BCOConfig, BCOTrainer, RunningMoments

    rm = RunningMoments()
    xs = torch.randn(1000, dtype=torch.float64) * 3 + 2
    for chunk in xs.split(100):
        rm.update(chunk)
    assert abs(rm.mean - float(xs.mean())) < 1e-4 and abs(rm.std - float(xs.std())) < 1e-3
    model = make_tiny_model()
    before = _snap(model)
    tr = BCOTrainer(model, args=BCOConfig(output_dir=str(tmp_path), **COMMON),
                    train_dataset=make_dataset("standard_unpaired_preference", 24), processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []
    assert any("delta" in h for h in tr.state.log_history)
    with pytest.warns(FutureWarning):
        import importlib

        import trl_b200.experimental.kto as shim
        importlib.reload(shim)
    assert shim.KTOTrainer is not None


def _reward_len(completion_ids, **kw):
    return [float(sum(c) % 5) for c in completion_ids]


GR = dict(per_device_train_batch_size=4, num_generations=4, max_completion_length=8, max_steps=2, logging_steps=1,
          learning_rate=1e-3, use_cpu=True, save_strategy="no", report_to="none", beta=0.0)


def test_gmpo_and_gspo_token(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.gmpo import GMPOConfig, GMPOTrainer
    from trl_b200.experimental.gspo_token import GRPOTrainer as GSPOTokenTrainer
    from trl_b200.trainer.grpo_config import GRPOConfig

    ds = make_dataset("standard_prompt_only", 16)
    model = make_tiny_model()
    before = _snap(model)
    tr = GMPOTrainer(model, _reward_len, GMPOConfig(output_dir=str(tmp_path / "a"), num_iterations=2, **GR), train_dataset=ds,
                     processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []
    model = make_tiny_model()
    before = _snap(model)
    tr = GSPOTokenTrainer(model, _reward_len, GRPOConfig(output_dir=str(tmp_path / "b"), num_iterations=2, loss_type="grpo", **GR),
                          train_dataset=ds, processing_class=tiny_tokenizer)
    assert tr.importance_sampling_level == "sequence_token"
    tr.train()
    assert _unchanged(model, before) == []


def test_replay_buffer_replaces_flat_groups(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.grpo_with_replay_buffer import (GRPOWithReplayBufferConfig, GRPOWithReplayBufferTrainer,
                                                               ReplayBuffer)

    rb = ReplayBuffer(2)
    rb.add([1.0, 3.0, 2.0], [{"i": 0}, {"i": 1}, {"i": 2}])
    assert sorted(h[2]["i"] for h in rb.heap) == [1, 2]
    assert len(rb.sample(4)) == 4
    calls = {"n": 0}

    def reward(completion_ids, **kw):  # first generation batch has variance, later ones are flat
        calls["n"] += 1
        return [float(i % 3) for i in range(len(completion_ids))] if calls["n"] == 1 else [1.0] * len(completion_ids)

    model = make_tiny_model()
    tr = GRPOWithReplayBufferTrainer(model, reward, GRPOWithReplayBufferConfig(output_dir=str(tmp_path), replay_buffer_size=4,
                                                                              **dict(GR, max_steps=3)),
                                     train_dataset=make_dataset("standard_prompt_only", 16), processing_class=tiny_tokenizer)
    tr.train()
    assert len(tr.replay_buffer) >= 1
    assert any(h.get("replay_buffer/replaced_groups", 0) > 0 for h in tr.state.log_history)


def test_generalized_jsd_limits():
    from trl_b200.experimental.gkd import GKDTrainer

    torch.manual_seed(0)
    s, t = torch.randn(2, 5, 11), torch.randn(2, 5, 11)
    ls, lt = torch.log_softmax(s, -1), torch.log_softmax(t, -1)
    fwd = (lt.exp() * (lt - ls)).sum(-1).sum() / 10
    rev = (ls.exp() * (ls - lt)).sum(-1).sum() / 10
    assert torch.allclose(GKDTrainer.generalized_jsd_loss(s, t, beta=0.0), fwd, atol=1e-6)
    assert torch.allclose(GKDTrainer.generalized_jsd_loss(s, t, beta=1.0), rev, atol=1e-6)
    mid = GKDTrainer.generalized_jsd_loss(s, t, beta=0.5)
    assert 0 < float(mid) < max(float(fwd), float(rev))
    assert float(GKDTrainer.generalized_jsd_loss(s, s, beta=0.3)) < 1e-7


@pytest.mark.parametrize("lmbda,seq_kd", [(0.0, False), (1.0, False), (0.0, True)])
def test_gkd(tmp_path, tiny_tokenizer, lmbda, seq_kd):
    from trl_b200.experimental.gkd import GKDConfig, GKDTrainer

    model, teacher = make_tiny_model(seed=0), make_tiny_model(seed=1)
    before = _snap(model)
    tr = GKDTrainer(model, teacher, GKDConfig(output_dir=str(tmp_path), lmbda=lmbda, seq_kd=seq_kd, max_new_tokens=6,
                                              **COMMON),
                    train_dataset=make_dataset("standard_prompt_completion", 16), processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []
    assert any("jsd" in h for h in tr.state.log_history)


ON = dict(per_device_train_batch_size=4, max_new_tokens=6, max_steps=2, logging_steps=1, learning_rate=1e-3, use_cpu=True,
          save_strategy="no", report_to="none")


def _reward_ids(completion_ids, **kw):
    return [float(sum(c) % 7) for c in completion_ids]


@pytest.mark.parametrize("kind", ["online_dpo", "xpo", "nash_md"])
def test_online_preference_trainers(tmp_path, tiny_tokenizer, kind):
    if kind == "online_dpo":
        from trl_b200.experimental.online_dpo import OnlineDPOConfig as C, OnlineDPOTrainer as T
        extra = dict(missing_eos_penalty=1.0, loss_type="ipo")
    elif kind == "xpo":
        from trl_b200.experimental.xpo import XPOConfig as C, XPOTrainer as T
        extra = dict(alpha=[1e-3, 1e-4])
    else:
        from trl_b200.experimental.nash_md import NashMDConfig as C, NashMDTrainer as T
        extra = dict(mixture_coef=0.3)
    model = make_tiny_model()
    before = _snap(model)
    tr = T(model, reward_funcs=_reward_ids, args=C(output_dir=str(tmp_path), **ON, **extra),
           train_dataset=make_dataset("standard_prompt_only", 16), processing_class=tiny_tokenizer)
    assert tr.ref_model is not None
    tr.train()
    assert _unchanged(model, before) == []
    h = [x for x in tr.state.log_history if "objective/kl" in x]
    assert h and "beta" in h[-1]


@pytest.mark.parametrize("separate_value_model", [False, True])
def test_ppo(tmp_path, tiny_tokenizer, separate_value_model):
    from trl_b200.experimental.ppo import AutoModelForCausalLMWithValueHead, PPOConfig, PPOTrainer
    from trl_b200.experimental.ppo.ppo_trainer import masked_whiten

    x, mk = torch.randn(4, 9), (torch.rand(4, 9) > 0.3).float()
    w = masked_whiten(x, mk)
    assert abs(float((w * mk).sum() / mk.sum())) < 1e-5
    model = make_tiny_model()
    value_model = make_tiny_model(seed=3, num_labels=1) if separate_value_model else None
    before = _snap(model)
    cfg = PPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, num_mini_batches=2, num_ppo_epochs=2,
                    response_length=6, max_steps=4, learning_rate=1e-3, use_cpu=True, save_strategy="no", report_to="none",
                    missing_eos_penalty=0.5, kl_estimator="k3")
    assert cfg.local_batch_size == 8 and cfg.local_mini_batch_size == 4
    tr = PPOTrainer(cfg, tiny_tokenizer, model, reward_funcs=_reward_ids, value_model=value_model,
                    train_dataset=make_dataset("standard_prompt_only", 32))
    tr.train()
    assert [n for n in _unchanged(model, before) if not n.startswith("value_model.")] == []
    assert any("loss/policy_avg" in x for x in tr.state.log_history)
    assert any("objective/rlhf_reward" in x for x in tr.state.log_history)
    # sample generations: default 10 over the run -> at least one table of near-greedy completions with scores
    tab = tr.sample_generations
    assert set(tab) == {"query", "model response", "score"} and len(tab["score"]) == len(tab["query"]) > 0
    wrapped = AutoModelForCausalLMWithValueHead(make_tiny_model())
    ids = torch.randint(5, 100, (2, 7))
    logits, _, values = wrapped(input_ids=ids, attention_mask=torch.ones_like(ids))
    assert logits.shape[:2] == (2, 7) and values.shape == (2, 7)
    assert any(k.startswith("v_head.") for k in wrapped.state_dict())


def test_prm(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.prm import PRMConfig, PRMTrainer

    row = PRMTrainer.tokenize_row({"prompt": "a b", "completions": ["c d", "e"], "labels": [True, False]}, tiny_tokenizer,
                                  "\n", None, None, False, False)
    assert len(row["input_ids"]) == len(row["labels"])
    assert [l for l in row["labels"] if l != -100] == [1, 0]
    last = PRMTrainer.tokenize_row({"prompt": "a b", "completions": ["c d", "e"], "labels": [True, False]}, tiny_tokenizer,
                                   "\n", None, None, True, False)
    assert [l for l in last["labels"] if l != -100] == [0]
    model = make_tiny_model(num_labels=2)
    before = _snap(model)
    tr = PRMTrainer(model, PRMConfig(output_dir=str(tmp_path), **COMMON),
                    train_dataset=make_dataset("standard_stepwise_supervision", 16), processing_class=tiny_tokenizer)
    tr.train()
    assert "score" not in _unchanged(model, before)
    assert any("accuracy" in h for h in tr.state.log_history)


def test_minillm_and_a2po(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.a2po import A2POConfig, A2POTrainer
    from trl_b200.experimental.minillm import MiniLLMConfig, MiniLLMTrainer

    ds = make_dataset("standard_prompt_only", 16)
    model, teacher = make_tiny_model(seed=0), make_tiny_model(seed=2)
    before = _snap(model)
    tr = MiniLLMTrainer(model, teacher, args=MiniLLMConfig(output_dir=str(tmp_path / "m"), gamma=0.9, **GR), train_dataset=ds,
                        processing_class=tiny_tokenizer)
    adv = tr._compute_advantage(torch.zeros(1, 3), torch.tensor([[1.0, 2.0, 3.0]]), torch.ones(1, 3))
    g = 0.9
    expect0 = (1 + g * 2 + g * g * 3) / (1 + g + g * g)
    assert abs(float(adv[0, 0]) - expect0) < 1e-5
    tr.train()
    assert _unchanged(model, before) == []
    assert any("single_step_rkl" in h for h in tr.state.log_history)
    model = make_tiny_model()
    before = _snap(model)
    cfg = A2POConfig(output_dir=str(tmp_path / "a"), per_device_train_batch_size=4, max_completion_length=6, max_steps=2,
                     num_value_samples=3, logging_steps=1, learning_rate=1e-3, use_cpu=True, save_strategy="no",
                     report_to="none", beta2=0.1)
    tr = A2POTrainer(model, _reward_ids, cfg, train_dataset=ds, processing_class=tiny_tokenizer)
    tr.train()
    assert len(tr._optimal_values) == 16
    assert _unchanged(model, before) == []


def test_self_distillation_losses():
    from trl_b200.experimental.sdft import loss_utils as L

    torch.manual_seed(0)
    s, t = torch.randn(6, 50), torch.randn(6, 50)
    full = L.compute_full_logit_self_distillation_loss(s, t, distillation_alpha=1.0)
    ls, lt = torch.log_softmax(s, -1), torch.log_softmax(t, -1)
    assert torch.allclose(full, (ls.exp() * (ls - lt)).sum(-1), atol=1e-5)
    topk_all = L.compute_topk_self_distillation_loss(s, t, distillation_topk=50, distillation_alpha=1.0, distillation_add_tail=False)
    assert torch.allclose(topk_all, full, atol=1e-4)
    tail = L.add_tail_bucket(torch.log_softmax(s, -1)[:, :10])
    assert torch.allclose(tail.exp().sum(-1), torch.ones(6), atol=1e-5)
    with pytest.raises(ValueError):
        L.compute_sampled_token_self_distillation_loss(s, t, torch.zeros(6, dtype=torch.long), distillation_alpha=0.5)


def test_sdft_sdpo_ssd_distillation(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.distillation import DistillationConfig, DistillationTrainer
    from trl_b200.experimental.sdft import SDFTConfig, SDFTTrainer
    from trl_b200.experimental.sdpo import SDPOConfig, SDPOTrainer
    from trl_b200.experimental.ssd import SSDConfig, SSDTrainer

    base = dict(per_device_train_batch_size=4, max_completion_length=6, max_steps=2, logging_steps=1, learning_rate=1e-3,
                use_cpu=True, save_strategy="no", report_to="none")
    ds = [dict(ex, privileged_context="the answer is " + str(i)) for i, ex in enumerate(make_dataset("standard_prompt_only", 16))]
    model = make_tiny_model()
    before = _snap(model)
    tr = SDFTTrainer(model, SDFTConfig(output_dir=str(tmp_path / "f"), num_generations=2, teacher_model_kind="ema",
                                       distillation_topk=20, distillation_add_tail=True, **base),
                     train_dataset=ds, processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []
    assert any("distillation_loss" in h for h in tr.state.log_history)

    model = make_tiny_model()
    before = _snap(model)
    tr = SDPOTrainer(model, lambda completion_ids, **kw: [float(sum(c) % 2) for c in completion_ids],
                     SDPOConfig(output_dir=str(tmp_path / "p"), num_generations=4, distillation_weight=0.5,
                                distillation_mode="full_logits", beta=0.0, **base),
                     train_dataset=ds, processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []
    assert any("sdpo/teacher_coverage" in h for h in tr.state.log_history)

    model = make_tiny_model()
    before = _snap(model)
    tr = SSDTrainer(model, SSDConfig(output_dir=str(tmp_path / "s"), temperature=1.3, **base), train_dataset=ds,
                    processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []

    model, teacher = make_tiny_model(seed=0), make_tiny_model(seed=1)
    before = _snap(model)
    tr = DistillationTrainer(model, teacher, DistillationConfig(output_dir=str(tmp_path / "d"), max_completion_length=6,
                                                                num_generations=2, **COMMON),
                             train_dataset=make_dataset("standard_prompt_completion", 16), processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []


def test_iw_opd_weights_and_training(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.iw_opd import IWOPDConfig, IWOPDTrainer
    from trl_b200.experimental.iw_opd.iw_opd_trainer import iw_opd_weights

    a = torch.tensor([[1.0, -1.0, 2.0, 0.0]])
    w = iw_opd_weights(a, torch.tensor([[1.0, 1.0, 1.0, 0.0]]), gamma=0.5, eps=1e-8)
    assert torch.allclose(w[0, :3], torch.tensor([1.5, 1.5 - 0.5 * 0.25, 1.5 - 0.5 * 0.5]))
    model, teacher = make_tiny_model(seed=0), make_tiny_model(seed=1)
    before = _snap(model)
    tr = IWOPDTrainer(model, teacher, IWOPDConfig(output_dir=str(tmp_path), max_completion_length=6, **COMMON),
                      train_dataset=make_dataset("standard_prompt_completion", 16), processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []
    assert any("iw_opd/mean_weight" in h for h in tr.state.log_history)


def test_gold_uld_and_server_distillation(tmp_path, tiny_tokenizer):
    import numpy as np

    from trl_b200.experimental.gold import GOLDConfig, GOLDTrainer
    from trl_b200.experimental.gold.gold_trainer import ULDLoss, align_spans
    from trl_b200.experimental.server_distillation import ServerDistillationConfig, ServerDistillationTrainer

    assert align_spans(["ab", "c", "de"], ["a", "bc", "d", "e"]) == [([0, 1], [0, 1]), ([2], [2, 3])]
    p = torch.softmax(torch.randn(3, 7), -1)
    assert float(ULDLoss._sorted_l1(p, p[:, torch.randperm(7)]).abs().max()) < 1e-6  # permutation invariant
    ds = make_dataset("standard_prompt_completion", 16)
    model, teacher = make_tiny_model(seed=0), make_tiny_model(seed=1)
    before = _snap(model)
    tr = GOLDTrainer(model, teacher, GOLDConfig(output_dir=str(tmp_path / "g"), use_uld_loss=True, lmbda=0.0,
                                                uld_use_hybrid_loss=True, uld_crossentropy_weight=0.1, **COMMON),
                     teacher_processing_class=tiny_tokenizer, train_dataset=ds, processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []

    class FakeTeacherClient:  # stands in for the HTTP client: uniform teacher
        def get_sequence_logprobs(self, sequences, prompt_lengths, temperature=1.0):
            return [np.full(len(s) - p, -np.log(1024.0), dtype=np.float32) for s, p in zip(sequences, prompt_lengths)]

    model = make_tiny_model()
    before = _snap(model)
    cfg = ServerDistillationConfig(output_dir=str(tmp_path / "s"), teacher_model_server_url="http://127.0.0.1:1", lmbda=0.0,
                                   **COMMON)
    tr = ServerDistillationTrainer(model, cfg, teacher_client=FakeTeacherClient(), train_dataset=ds,
                                   processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []


def test_token_budget_batcher_balances_squared_lengths():
    from trl_b200.experimental.async_grpo import RolloutSample, TokenBudgetBatcher

    def mk(n):
        return RolloutSample([0] * 2, [1] * (n - 2), [0.0] * (n - 2), 0.0, 0.0, 0, 0)
    lens = [50, 40, 30, 30, 20, 10, 10, 10]
    rows, left = TokenBudgetBatcher(world=2, token_budget=100, per_rank=4).assign([mk(n) for n in lens])
    assert left == [] and all(sum(len(s) for s in r) <= 100 for r in rows)
    sq = [sum(len(s) ** 2 for s in r) for r in rows]
    assert abs(sq[0] - sq[1]) <= 0.35 * max(sq)
    rows, left = TokenBudgetBatcher(world=2, token_budget=0, per_rank=2).assign([mk(n) for n in lens])
    assert [len(r) for r in rows] == [2, 2] and len(left) == 4


def test_async_grpo_trains_from_queue_and_drops_stale(tmp_path, tiny_tokenizer):
    from trl_b200.experimental.async_grpo import AsyncGRPOConfig, AsyncGRPOTrainer

    model = make_tiny_model()
    before = _snap(model)
    cfg = AsyncGRPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, num_generations=2, max_completion_length=6,
                          max_steps=3, learning_rate=1e-3, use_cpu=True, save_strategy="no", report_to="none",
                          vllm_server_base_url=None, max_staleness=1, heartbeat_stale_after_s=60.0)
    tr = AsyncGRPOTrainer(model, lambda completion_ids, **kw: [float(sum(c) % 3) for c in completion_ids], cfg,
                          train_dataset=make_dataset("standard_prompt_only", 16), processing_class=tiny_tokenizer)
    tr.train()
    assert _unchanged(model, before) == []
    assert tr.worker.groups_done > 0 and not tr.worker._thread.is_alive()
    assert any("async/staleness_mean" in h for h in tr.state.log_history)


def test_async_worker_failure_is_reported():
    from trl_b200.experimental.async_grpo import AsyncRolloutWorker

    def broken(prompts, n):
        raise ValueError("generation backend down")
    w = AsyncRolloutWorker([{"prompt": "x"}], broken, lambda *a: [], 2)
    w.start()
    w._thread.join(timeout=5)
    with pytest.raises(RuntimeError):
        w.check_health(60.0)


def test_merge_methods(tmp_path):
    from safetensors.torch import load_file

    from trl_b200.experimental.merge_model_callback import MergeConfig, merge_models

    a, b = make_tiny_model(seed=0), make_tiny_model(seed=1)
    a.save_pretrained(str(tmp_path / "a"))
    b.save_pretrained(str(tmp_path / "b"))
    A, B = load_file(str(tmp_path / "a" / "model.safetensors")), load_file(str(tmp_path / "b" / "model.safetensors"))
    key = next(k for k in A if "q_proj" in k or "qkv" in k or "gate_proj" in k)
    for method in ("linear", "slerp", "ties", "dare_ties"):
        cfg = MergeConfig(method)
        cfg.policy_model_path, cfg.target_model_path, cfg.dtype = str(tmp_path / "a"), str(tmp_path / "b"), "float32"
        merge_models(cfg, str(tmp_path / method))
        M = load_file(str(tmp_path / method / "model.safetensors"))
        assert set(M) == set(A) and (tmp_path / method / "config.json").exists()
        if method == "linear":
            assert torch.allclose(M[key], 0.5 * (A[key] + B[key]), atol=1e-6)
        if method == "ties":  # densities < 1 keep only the largest task-vector entries
            assert torch.isfinite(M[key]).all()
    cfg = MergeConfig("slerp")
    cfg.policy_model_path = cfg.target_model_path = str(tmp_path / "a")
    cfg.dtype = "float32"
    merge_models(cfg, str(tmp_path / "same"))
    assert torch.allclose(load_file(str(tmp_path / "same" / "model.safetensors"))[key], A[key], atol=1e-5)


def test_harbor_local_and_openreward_adapter(tmp_path):
    from trl_b200.experimental.harbor import HarborSpec
    from trl_b200.experimental.openreward import OpenRewardSpec

    t = tmp_path / "suite" / "tasks" / "t0"
    (t / "tests").mkdir(parents=True)
    (t / "environment").mkdir()
    (t / "instruction.md").write_text("Create a file named done.txt")
    (t / "task.toml").write_text('[metadata]\ndifficulty = "easy"\n')
    (t / "tests" / "test.sh").write_text("test -f done.txt\n")
    spec = HarborSpec(str(tmp_path / "suite"), environment_type="local")
    rows = spec.dataset
    assert len(rows) == 1 and rows[0]["difficulty"] == "easy"
    env = spec.environment_factory()
    text = env.reset(task_dir=rows[0]["task_dir"])
    assert "done.txt" in text
    assert "[exit code" in env.bash("ls missing_file")
    env.bash("touch done.txt")
    assert spec.reward_funcs[0](environments=[env]) == [1.0]
    env.close()

    class Session:
        def __init__(self, **row):
            self.row, self.calls = row, 0

        def call_tool(self, name, arguments):
            self.calls += 1
            return {"blocks": [{"text": f"{name}:{arguments}"}], "reward": 0.5, "finished": self.calls >= 2}
    tools = [{"name": "lookup", "description": "Look something up.",
              "input_schema": {"properties": {"query": {"type": "string", "description": "what"}}, "required": ["query"]}}]
    ors = OpenRewardSpec.from_session_factory(lambda **row: Session(**row), tools, [{"task_id": 1, "prompt": "hi"}])
    e = ors.environment_factory()
    e.reset(**{k: v for k, v in ors.dataset[0].items() if k != "prompt"})
    assert "lookup" in e.lookup(query="x") and "Args:" in type(e).lookup.__doc__
    e.lookup(query="y")
    assert e.reward == 1.0 and e.lookup(query="z").startswith("error")


def test_experimental_utils(tiny_tokenizer):
    from trl_b200.experimental import utils as U

    b = torch.tensor([[False, True, True], [False, False, False]])
    assert U.first_true_indices(b).tolist() == [1, 3]
    ids, mask = U.truncate_right(torch.tensor([[5, 6, 2, 7, 8]]), 2, 0)
    assert ids.tolist() == [[5, 6, 2, 0, 0]] and mask.tolist() == [[1, 1, 1, 0, 0]]
    assert U.pad_to_length(torch.ones(2, 3), 5, -1).shape == (2, 5)
    assert U.pad_byte_offsets([(0, 2), (2, 5)], 4, "left").tolist() == [[-1, -1], [-1, -1], [0, 2], [2, 5]]
    col = U.DPODataCollatorWithPadding(pad_token_id=0)
    out = col([{"prompt_input_ids": [1, 2], "chosen_labels": [3], "tag": "a"}, {"prompt_input_ids": [1], "chosen_labels": [3, 4], "tag": "b"}])
    assert out["prompt_input_ids"].tolist() == [[1, 2], [0, 1]] and out["chosen_labels"].tolist() == [[3, -100], [3, 4]]
    model = make_tiny_model(num_labels=1)
    q = torch.randint(5, 100, (2, 6))
    q[1, 4:] = 0
    per_tok, score, lens = U.get_reward(model, q, 0, 2)
    assert per_tok.shape == (2, 6) and lens.tolist() == [5, 3] and torch.allclose(score[1], per_tok[1, 3])
    ref = U.create_reference_model(make_tiny_model(), num_shared_layers=1)
    assert not any(p.requires_grad for p in ref.parameters())


def test_bema_refreshes_the_dpo_reference_model(tmp_path, tiny_tokenizer):
    """trl/experimental/bema_for_ref_model: the reference model receives the running BEMA weights every
    ``ref_model_update_freq`` steps after ``ref_model_update_after``; without ``update_ref_model`` it stays frozen."""
    from trl_b200 import DPOConfig
    from trl_b200.experimental.bema_for_ref_model import BEMACallback, DPOTrainer

    def run(sub, **kw):
        cb = BEMACallback(update_freq=2, **kw)
        model = make_tiny_model("tiny-qwen2", seed=0)
        cfg = DPOConfig(output_dir=str(tmp_path / sub), per_device_train_batch_size=4, max_steps=6, learning_rate=1e-3,
                        save_strategy="no", report_to="none", use_cpu=True, bf16=False, logging_steps=100)
        tr = DPOTrainer(model, None, cfg, train_dataset=make_dataset("standard_preference", 24),
                        processing_class=tiny_tokenizer, callbacks=[cb])
        ref0 = {n: p.detach().clone() for n, p in tr.ref_model.named_parameters()}
        tr.train()
        return cb, tr, ref0

    cb, tr, ref0 = run("on", update_ref_model=True, ref_model_update_freq=3, ref_model_update_after=0)
    ref = dict(tr.ref_model.named_parameters())
    name = cb.names[len(cb.names) // 2]
    assert not torch.equal(ref[name], ref0[name])
    # steps 3 and 6 copied the running weights; the last BEMA update (step 6) came first in the same callback
    assert torch.allclose(ref[name].detach().float(), cb.running[cb.names.index(name)], atol=1e-6)
    cb, tr, ref0 = run("off")
    assert all(torch.equal(p, ref0[n]) for n, p in tr.ref_model.named_parameters())
