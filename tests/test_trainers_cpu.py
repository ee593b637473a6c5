"""Trainer integration on CPU with tiny random-init models and synthetic datasets.  Criterion (as in the
reference's smoke tests): ``train_loss`` is logged and every trainable parameter changed."""
import json
import os

import pytest
import torch

from trl_b200.testing import make_dataset, make_tiny_model
from trl_b200 import (DPOConfig, DPOTrainer, GRPOConfig, GRPOTrainer, KTOConfig, KTOTrainer, RewardConfig,
                      RewardTrainer, RLOOConfig, RLOOTrainer, SFTConfig, SFTTrainer)

COMMON = dict(per_device_train_batch_size=4, max_steps=2, logging_steps=1, learning_rate=1e-3, use_cpu=True,
              save_strategy="no", report_to="none")


def _changed(model, before):
    return [n for n, p in model.named_parameters() if p.requires_grad and torch.equal(before[n], p)]


def _snap(model):
    return {n: p.detach().clone() for n, p in model.named_parameters()}


@pytest.mark.parametrize("kind,extra", [
    ("standard_language_modeling", {}),
    ("conversational_language_modeling", {"assistant_only_loss": True}),
    ("standard_prompt_completion", {"padding_free": True}),
    ("conversational_prompt_completion", {"packing": True, "max_length": 64}),
    ("standard_language_modeling", {"loss_type": "dft"}),
    ("standard_language_modeling", {"packing": True, "packing_strategy": "wrapped", "max_length": 32}),
])
def test_sft_trains(tmp_path, tiny_tokenizer, kind, extra):
    model = make_tiny_model()
    before = _snap(model)
    tr = SFTTrainer(model, SFTConfig(output_dir=str(tmp_path), **COMMON, **extra), train_dataset=make_dataset(kind, 24),
                    processing_class=tiny_tokenizer)
    tr.train()
    assert tr.state.log_history[-1]["train_loss"] is not None
    assert _changed(model, before) == []
    logged = [h for h in tr.state.log_history if "entropy" in h]
    assert logged and "num_tokens" in logged[-1]


def test_sft_moe_aux_loss(tmp_path, tiny_tokenizer):
    model = make_tiny_model("tiny-qwen3-moe")
    before = _snap(model)
    tr = SFTTrainer(model, SFTConfig(output_dir=str(tmp_path), **COMMON), train_dataset=make_dataset("standard_language_modeling", 16),
                    processing_class=tiny_tokenizer)
    tr.train()
    assert _changed(model, before) == []
    assert any("aux_loss" in h for h in tr.state.log_history)


def test_sft_eval_and_checkpoint_resume(tmp_path, tiny_tokenizer):
    ds = make_dataset("standard_language_modeling", 32)
    cfg = dict(COMMON, max_steps=4, save_strategy="steps", save_steps=2, eval_strategy="steps", eval_steps=2,
               lr_scheduler_type="constant", train_sampling_strategy="sequential")
    m1 = make_tiny_model()
    t1 = SFTTrainer(m1, SFTConfig(output_dir=str(tmp_path / "a"), **cfg), train_dataset=ds, eval_dataset=ds.select(range(8)),
                    processing_class=tiny_tokenizer)
    t1.train()
    ck = tmp_path / "a" / "checkpoint-2"
    for f in ("model.safetensors", "config.json", "trainer_state.json", "optimizer.pt", "scheduler.pt", "rng_state.pth"):
        assert (ck / f).exists(), f
    assert any("eval_loss" in h for h in t1.state.log_history)
    state = json.load(open(ck / "trainer_state.json"))
    assert state["global_step"] == 2
    m2 = make_tiny_model(seed=123)  # different init: everything must come from the checkpoint
    t2 = SFTTrainer(m2, SFTConfig(output_dir=str(tmp_path / "a"), **cfg), train_dataset=ds, eval_dataset=ds.select(range(8)),
                    processing_class=tiny_tokenizer)
    t2.train(resume_from_checkpoint=str(ck))
    assert t2.state.global_step == 4
    for (n, p), (_, q) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.allclose(p, q, atol=1e-6), n


@pytest.mark.parametrize("kind,extra", [
    ("standard_preference", {}),
    ("conversational_implicit_prompt_preference", {"loss_type": ["sigmoid", "bco_pair", "sft"], "loss_weights": [0.8, 0.2, 1.0]}),
    ("standard_preference", {"loss_type": "ipo", "precompute_ref_log_probs": True}),
    ("standard_preference", {"loss_type": "aot", "use_weighting": True, "ld_alpha": 0.5}),
    ("standard_preference", {"f_divergence_type": "js_divergence", "label_smoothing": 0.1}),
])
def test_dpo_trains(tmp_path, tiny_tokenizer, kind, extra):
    model = make_tiny_model()
    before = _snap(model)
    tr = DPOTrainer(model, args=DPOConfig(output_dir=str(tmp_path), **COMMON, **extra), train_dataset=make_dataset(kind, 16),
                    processing_class=tiny_tokenizer)
    tr.train()
    assert _changed(model, before) == []
    h = [x for x in tr.state.log_history if "rewards/chosen" in x][-1]
    for k in ("rewards/rejected", "rewards/accuracies", "rewards/margins", "logps/chosen", "logps/rejected", "entropy"):
        assert k in h


def test_dpo_first_step_loss_is_log2(tmp_path, tiny_tokenizer):
    model = make_tiny_model()
    tr = DPOTrainer(model, args=DPOConfig(output_dir=str(tmp_path), **dict(COMMON, max_steps=1)),
                    train_dataset=make_dataset("standard_preference", 8), processing_class=tiny_tokenizer)
    tr.train()
    first = [x for x in tr.state.log_history if "loss" in x][0]["loss"]
    assert abs(first - 0.6931) < 1e-3  # policy == reference at step 1


def test_dpo_with_lora_uses_adapter_off_reference(tmp_path, tiny_tokenizer):
    from trl_b200.models.lora import LoraConfig

    model = make_tiny_model()
    tr = DPOTrainer(model, args=DPOConfig(output_dir=str(tmp_path), **COMMON), train_dataset=make_dataset("standard_preference", 16),
                    processing_class=tiny_tokenizer, peft_config=LoraConfig(r=4, target_modules=["q_proj", "v_proj"]))
    assert tr.ref_model is None and tr._ref_adapter_off
    tr.train()
    tr.save_model(str(tmp_path / "out"))
    assert (tmp_path / "out" / "adapter_model.safetensors").exists()


def test_kto_kl_rotation_and_training(tmp_path, tiny_tokenizer):
    model = make_tiny_model()
    before = _snap(model)
    tr = KTOTrainer(model, args=KTOConfig(output_dir=str(tmp_path), **COMMON), train_dataset=make_dataset("standard_unpaired_preference", 16),
                    processing_class=tiny_tokenizer)
    rows = [tr.train_dataset[i] for i in range(8)]
    for s in (0, 4):  # completions rotated by one inside every per-device batch
        comps = [r["completion_ids"] for r in rows[s:s + 4]]
        assert [r["KL_completion_ids"] for r in rows[s:s + 4]] == [comps[-1]] + comps[:-1]
    tr.train()
    assert _changed(model, before) == []
    assert any("kl" in h for h in tr.state.log_history)
    with pytest.raises(ValueError):
        KTOTrainer(make_tiny_model(), args=KTOConfig(output_dir=str(tmp_path), **dict(COMMON, per_device_train_batch_size=1)),
                   train_dataset=make_dataset("standard_unpaired_preference", 8), processing_class=tiny_tokenizer)


def test_reward_trainer(tmp_path, tiny_tokenizer):
    model = make_tiny_model(num_labels=1)
    before = _snap(model)
    tr = RewardTrainer(model, args=RewardConfig(output_dir=str(tmp_path), center_rewards_coefficient=0.01, **COMMON),
                       train_dataset=make_dataset("conversational_preference", 16), processing_class=tiny_tokenizer)
    tr.train()
    assert _changed(model, before) == []
    h = [x for x in tr.state.log_history if "accuracy" in x][-1]
    assert {"min_reward", "mean_reward", "max_reward", "margin", "num_tokens"} <= set(h)


def _len_reward(completions, completion_ids=None, **kw):
    if completion_ids is not None:  # works for text and conversational completions alike
        return [float(sum(ids)) % 7 / 7 + len(ids) / 10 for ids in completion_ids]
    return [float(len(c)) / 10 for c in completions]


def _none_reward(completions, **kw):
    return [None for _ in completions]


@pytest.mark.parametrize("extra", [
    {"loss_type": "dapo"}, {"loss_type": "grpo", "beta": 0.04}, {"loss_type": "bnpo", "num_iterations": 2},
    {"loss_type": "dr_grpo", "scale_rewards": "batch"}, {"loss_type": "cispo"}, {"loss_type": "sapo"},
    {"loss_type": "luspo", "importance_sampling_level": "sequence"}, {"loss_type": "vespo"},
    {"top_entropy_quantile": 0.5}, {"entropy_coef": 0.01, "use_adaptive_entropy": True},
    {"multi_objective_aggregation": "normalize_then_sum"}, {"mask_truncated_completions": True, "delta": 2.0},
])
def test_grpo_variants_train(tmp_path, tiny_tokenizer, extra):
    model = make_tiny_model()
    before = _snap(model)
    args = GRPOConfig(output_dir=str(tmp_path), **dict(COMMON, learning_rate=1e-2), num_generations=4,
                      max_completion_length=8, gradient_accumulation_steps=2, **extra)
    rf = [_len_reward, _len_reward] if "multi_objective_aggregation" in extra else _len_reward
    tr = GRPOTrainer(model, rf, args, train_dataset=make_dataset("standard_prompt_only", 16), processing_class=tiny_tokenizer)
    tr.train()
    if not extra.get("mask_truncated_completions"):
        assert _changed(model, before) == []
    h = [x for x in tr.state.log_history if "reward" in x][-1]
    assert "completions/mean_length" in h and "rewards/_len_reward/mean" in h


def test_grpo_unscorable_completions_get_zero_advantage(tmp_path, tiny_tokenizer):
    model = make_tiny_model()
    before = _snap(model)
    args = GRPOConfig(output_dir=str(tmp_path), **COMMON, num_generations=4, max_completion_length=4, loss_type="grpo")
    tr = GRPOTrainer(model, _none_reward, args, train_dataset=make_dataset("standard_prompt_only", 8), processing_class=tiny_tokenizer)
    tr.train()
    assert len(_changed(model, before)) == len(before)  # no signal -> no update


def test_grpo_generation_batch_schedule_prompts_seen_by_training_step(tmp_path, tiny_tokenizer):
    """per_device_bs=6, steps_per_generation=4, num_generations=4, num_iterations=2, GA=3: one generation batch of
    24 rows = 6 prompts x 4 serves 8 consecutive training steps; 48 training_step calls for 3 epochs over 12 prompts."""
    ds = make_dataset("standard_prompt_only", 12)
    args = GRPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=6, steps_per_generation=4, num_generations=4,
                      num_iterations=2, gradient_accumulation_steps=3, num_train_epochs=3, max_completion_length=4,
                      use_cpu=True, save_strategy="no", report_to="none", shuffle_dataset=False)
    assert args.generation_batch_size == 24
    tr = GRPOTrainer(make_tiny_model(), _len_reward, args, train_dataset=ds, processing_class=tiny_tokenizer)
    seen, gens = [], []
    orig_gen = tr._generate_and_score_completions

    def spy_gen(inputs):
        gens.append([x["prompt"] for x in inputs])
        return orig_gen(inputs)
    tr._generate_and_score_completions = spy_gen
    orig_step = type(tr).training_step

    def spy_step(self, model, inputs, n=None):
        seen.append([x["prompt"] for x in inputs])
        return orig_step(self, model, inputs, n)
    tr.training_step = spy_step.__get__(tr)
    tr.train()
    assert len(seen) == 48
    assert all(seen[i] == seen[0] for i in range(8)) and seen[8] != seen[0]
    assert len(gens) == 6 and len(gens[0]) == 24
    prompts = [r["prompt"] for r in ds]
    assert gens[0] == [p for p in prompts[:6] for _ in range(4)]


def test_rloo_trains(tmp_path, tiny_tokenizer):
    model = make_tiny_model()
    before = _snap(model)
    tr = RLOOTrainer(model, _len_reward, RLOOConfig(output_dir=str(tmp_path), **COMMON, num_generations=4, max_completion_length=8),
                     train_dataset=make_dataset("conversational_prompt_only", 16), processing_class=tiny_tokenizer)
    tr.train()
    assert _changed(model, before) == []


def test_grpo_reward_model_and_rollout_func(tmp_path, tiny_tokenizer):
    rm = make_tiny_model(num_labels=1, seed=5)
    calls = []

    def rollout(prompts, trainer):
        calls.append(len(prompts))
        ids = trainer._tokenize_prompts(prompts)
        return {"prompt_ids": ids, "completion_ids": [[7, 8, 9, trainer.eos_token_id] for _ in ids],
                "logprobs": [[-1.0] * 4 for _ in ids]}
    args = GRPOConfig(output_dir=str(tmp_path), **COMMON, num_generations=4, max_completion_length=8)
    tr = GRPOTrainer(make_tiny_model(), [rm, _len_reward], args, train_dataset=make_dataset("standard_prompt_only", 8),
                     processing_class=tiny_tokenizer, rollout_func=rollout)
    tr.train()
    assert calls and any("rewards/_len_reward/mean" in h for h in tr.state.log_history)


def test_config_validation():
    with pytest.raises(ValueError):
        GRPOConfig(output_dir="x", per_device_train_batch_size=3, num_generations=4, use_cpu=True)
    with pytest.raises(ValueError):
        GRPOConfig(output_dir="x", num_generations=1, per_device_train_batch_size=4, use_cpu=True)
    with pytest.raises(ValueError):
        GRPOConfig(output_dir="x", parallelism_config={"cp_size": 2}, use_cpu=True)
    with pytest.raises(ValueError):
        DPOConfig(output_dir="x", loss_type="nope")
    c = SFTConfig(output_dir="x", packing_strategy="bfd-requeue")
    assert c.packing_strategy == "bfd_split" and c.loss_type == "chunked_nll" and c.logging_steps == 10
    assert GRPOConfig(output_dir="x", use_cpu=True).loss_type == "dapo"


def test_grpo_generation_batch_schedule(tmp_path, tiny_tokenizer):
    """per_device_bs=6, steps_per_generation=4, num_generations=4, num_iterations=2, GA=3: a generation batch is 24 rows
    (6 prompts x 4) and serves 8 consecutive training_step calls; 48 calls for 3 epochs over 12 prompts."""
    from trl_b200.trainer.grpo_config import GRPOConfig
    from trl_b200.trainer.grpo_trainer import GRPOTrainer

    calls = {"gen": 0, "rows": []}
    model = make_tiny_model()
    cfg = GRPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=6, steps_per_generation=4, num_generations=4,
                     num_iterations=2, gradient_accumulation_steps=3, max_completion_length=4, num_train_epochs=3, logging_steps=1,
                     learning_rate=1e-4, use_cpu=True, save_strategy="no", report_to="none", beta=0.0)
    assert cfg.generation_batch_size == 24
    tr = GRPOTrainer(model, lambda completion_ids, **kw: [float(sum(c) % 3) for c in completion_ids], cfg,
                     train_dataset=make_dataset("standard_prompt_only", 12), processing_class=tiny_tokenizer)
    orig = tr._generate_and_score_completions

    def spy(inputs):
        calls["gen"] += 1
        calls["rows"].append(len(inputs))
        assert len({str(x["prompt"]) for x in inputs}) == 6
        return orig(inputs)
    tr._generate_and_score_completions = spy
    tr.train()
    # 12 prompts -> 2 generation batches per epoch, each served by 8 training_step calls: 16 per epoch, 48 in total
    assert tr._step == 48 and calls["gen"] == 6 and set(calls["rows"]) == {24}


def test_grpo_unscorable_and_truncated_completions(tmp_path, tiny_tokenizer):
    from trl_b200.trainer.grpo_config import GRPOConfig
    from trl_b200.trainer.grpo_trainer import GRPOTrainer

    def reward(completion_ids, **kw):  # every second completion cannot be scored
        return [None if i % 2 else float(sum(c) % 5) for i, c in enumerate(completion_ids)]
    model = make_tiny_model()
    cfg = GRPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, num_generations=4, max_completion_length=5,
                     max_steps=1, logging_steps=1, learning_rate=1e-4, use_cpu=True, save_strategy="no", report_to="none",
                     beta=0.0, mask_truncated_completions=True)
    tr = GRPOTrainer(model, reward, cfg, train_dataset=make_dataset("standard_prompt_only", 8), processing_class=tiny_tokenizer)
    batch = next(iter(tr.get_train_dataloader()))
    out = tr._generate_and_score_completions(batch)
    adv = out["advantages"]
    assert torch.isfinite(adv).all() and float(adv[1::2].abs().max()) == 0.0  # unscorable rows carry no signal
    eos, pad_id = tiny_tokenizer.eos_token_id, tiny_tokenizer.pad_token_id
    for ids, row in zip(out["completion_ids_list"], out["completion_mask"]):
        if ids[-1] not in (eos, pad_id):  # truncated: the whole row is masked out
            assert float(row.sum()) == 0.0


def test_fused_lm_head_losses_reject_an_adapted_lm_head(tmp_path, tiny_tokenizer):
    from trl_b200.models.lora import LoraConfig

    with pytest.raises(ValueError, match="lm_head"):
        SFTTrainer(make_tiny_model(), SFTConfig(output_dir=str(tmp_path), **COMMON),
                   train_dataset=make_dataset("standard_language_modeling", 8), processing_class=tiny_tokenizer,
                   peft_config=LoraConfig(r=4, target_modules=["q_proj", "lm_head"]))


@pytest.mark.parametrize("name", ["tiny-gemma", "tiny-phi3", "tiny-mistral"])
def test_sft_trains_other_families(tmp_path, tiny_tokenizer, name):
    model = make_tiny_model(name)
    before = _snap(model)
    tr = SFTTrainer(model, SFTConfig(output_dir=str(tmp_path), **COMMON), train_dataset=make_dataset("standard_language_modeling", 16),
                    processing_class=tiny_tokenizer)
    tr.train()
    assert _changed(model, before) == []


def _sft_trajectory(tmp_path, tag, **over):
    g = torch.Generator().manual_seed(5)
    rows = []
    for _ in range(8 * 4):  # 4 optimizer steps of 8 single-document sequences of different lengths
        n = int(torch.randint(16, 49, (1,), generator=g))
        rows.append({"input_ids": torch.randint(0, 1024, (n,), generator=g).tolist(),
                     "completion_mask": [0] * (n // 2) + [1] * (n - n // 2)})
    torch.manual_seed(0)
    kw = dict(output_dir=str(tmp_path / tag), per_device_train_batch_size=8, gradient_accumulation_steps=1, max_steps=4,
              logging_steps=1, learning_rate=1e-3, use_cpu=True, save_strategy="no", report_to="none",
              lr_scheduler_type="constant", train_sampling_strategy="sequential", padding_free=True,
              completion_only_loss=True, dataset_kwargs={"skip_prepare_dataset": True}, gradient_checkpointing=True,
              max_length=None)
    kw.update(over)
    tr = SFTTrainer(make_tiny_model(seed=0), SFTConfig(**kw), train_dataset=rows, processing_class=_Tok())
    tr.train()
    return [(h["loss"], h["grad_norm"]) for h in tr.state.log_history if "grad_norm" in h]


class _Tok:
    pad_token, eos_token, pad_token_id, eos_token_id, chat_template = "<pad>", "<eos>", 0, 1, None

    def save_pretrained(self, p):
        pass

    def convert_tokens_to_ids(self, t):
        return 1


def test_sft_trajectory_equivalence_classes(tmp_path):
    """One global batch, four ways to run it: the loss / grad-norm series must agree (the reference's invariant suite:
    default == per-device batch 1 x accumulation 8 == no activation checkpointing; padding-free == padded)."""
    base = _sft_trajectory(tmp_path, "base")
    assert len(base) == 4
    variants = {
        "bs1_ga8": dict(per_device_train_batch_size=1, gradient_accumulation_steps=8),
        "no_ckpt": dict(gradient_checkpointing=False),
        "padded": dict(padding_free=False),
        "partial_ckpt": dict(gradient_checkpointing_kwargs={"num_layers": 1}),
    }
    for name, over in variants.items():
        got = _sft_trajectory(tmp_path, name, **over)
        for (l0, g0), (l1, g1) in zip(base, got):
            assert abs(l0 - l1) < 1e-4 and abs(g0 - g1) < 1e-3 * max(1.0, g0), (name, base, got)


def _dpo_trajectory(tmp_path, tag, tok, **over):
    torch.manual_seed(0)
    kw = dict(output_dir=str(tmp_path / tag), per_device_train_batch_size=4, gradient_accumulation_steps=1, max_steps=3,
              logging_steps=1, learning_rate=1e-3, use_cpu=True, save_strategy="no", report_to="none", beta=0.5,
              lr_scheduler_type="constant", train_sampling_strategy="sequential", gradient_checkpointing=False)
    kw.update(over)
    tr = DPOTrainer(make_tiny_model(seed=0), args=DPOConfig(**kw), train_dataset=make_dataset("standard_preference", 12),
                    processing_class=tok)
    tr.train()
    return [(h["loss"], h["grad_norm"], h["rewards/margins"]) for h in tr.state.log_history if "grad_norm" in h]


def test_dpo_trajectory_equivalence_classes(tmp_path, tiny_tokenizer):
    """Same pairs, same order: accumulation, precomputed reference log-probs, padding-free batches and activation
    checkpointing must not change the loss / grad-norm / margin series."""
    base = _dpo_trajectory(tmp_path, "base", tiny_tokenizer)
    assert len(base) == 3 and abs(base[0][0] - 0.6931) < 1e-3
    for name, over in {"bs1_ga4": dict(per_device_train_batch_size=1, gradient_accumulation_steps=4),
                       "precomputed_ref": dict(precompute_ref_log_probs=True),
                       "padding_free": dict(padding_free=True),
                       "ckpt": dict(gradient_checkpointing=True)}.items():
        got = _dpo_trajectory(tmp_path, name, tiny_tokenizer, **over)
        for a, b in zip(base, got):
            assert all(abs(x - y) < 2e-4 * max(1.0, abs(x)) for x, y in zip(a, b)), (name, base, got)


def test_grpo_adaptive_entropy_moves_one_delta_per_optimizer_step(tmp_path, tiny_tokenizer):
    """The controller sees the whole accumulation window once, at the optimizer-step boundary: with GA=4 the
    coefficient moves by exactly one delta per step, the first window applies no bonus (nothing measured yet), and
    the measured entropy is checkpointed with the coefficient."""
    model = make_tiny_model()
    args = GRPOConfig(output_dir=str(tmp_path), **dict(COMMON, max_steps=3, save_strategy="steps", save_steps=3),
                      num_generations=4, max_completion_length=6, gradient_accumulation_steps=4, loss_type="grpo",
                      entropy_coef=0.02, use_adaptive_entropy=True, entropy_target=1e9, entropy_coef_delta=0.003,
                      entropy_coef_max=1.0)
    tr = GRPOTrainer(model, _len_reward, args, train_dataset=make_dataset("standard_prompt_only", 32),
                     processing_class=tiny_tokenizer)
    assert tr._last_world_entropy == float("inf")
    tr.train()
    # entropy <= target on every step -> +delta three times
    assert abs(tr.entropy_coef - (0.02 + 3 * 0.003)) < 1e-9
    assert 0.0 < tr._last_world_entropy < 20.0 and tr._entropy_window_stats is None
    coefs = [h["entropy_coef"] for h in tr.state.log_history if "entropy_coef" in h]
    assert [round(c, 6) for c in coefs] == [0.023, 0.026, 0.029]
    assert any("policy_loss" in h for h in tr.state.log_history)
    with open(os.path.join(str(tmp_path), "checkpoint-3", "entropy_ctrl_state.json")) as f:
        st = json.load(f)
    assert abs(st["entropy_coef"] - tr.entropy_coef) < 1e-12 and st["last_world_entropy"] == tr._last_world_entropy
    # target below any entropy: the coefficient walks down, and the gate closes the bonus
    model2 = make_tiny_model()
    args2 = GRPOConfig(output_dir=str(tmp_path / "b"), **dict(COMMON, max_steps=2), num_generations=4,
                       max_completion_length=6, gradient_accumulation_steps=2, loss_type="grpo", entropy_coef=0.02,
                       use_adaptive_entropy=True, entropy_target=-1.0, entropy_coef_delta=0.003)
    tr2 = GRPOTrainer(model2, _len_reward, args2, train_dataset=make_dataset("standard_prompt_only", 16),
                      processing_class=tiny_tokenizer)
    tr2.train()
    assert abs(tr2.entropy_coef - (0.02 - 2 * 0.003)) < 1e-9 and tr2._last_world_entropy > -1.0


def test_grpo_entropy_bonus_is_the_differentiable_mean_entropy():
    """d(mean entropy)/d(hidden) through the chunked lm_head equals autograd over explicit logits."""
    from trl_b200.ops import functional as ops

    torch.manual_seed(0)
    h = torch.randn(6, 16, requires_grad=True)
    w = torch.randn(40, 16) * 0.3
    y = torch.randint(0, 40, (6,))
    _, ent = ops.lm_head_logprobs(h, w, y, 0.7, compute_entropy=True, entropy_grad=True)
    ent.mean().backward()
    h2 = h.detach().clone().requires_grad_()
    z = (h2 @ w.t()) / 0.7
    p = torch.softmax(z, -1)
    (-(p * torch.log_softmax(z, -1)).sum(-1)).mean().backward()
    assert torch.allclose(h.grad, h2.grad, atol=1e-5)
    _, ent_stat = ops.lm_head_logprobs(h, w, y, 0.7, compute_entropy=True)
    assert not ent_stat.requires_grad


def test_grpo_vespo_weights_and_rollout_ratio_guards():
    adv = torch.tensor([[1.0], [-1.0]])
    mask = torch.ones(2, 4)
    huge = torch.full((2, 4), 50.0)  # exp(200) overflows without the clamps
    phi = GRPOTrainer.get_gamma_weights(adv, huge, mask, None, 2.0, 3.0, 3.0, 2.0)
    assert torch.isfinite(phi).all() and (phi >= 0).all()
    # hand value for a small ratio: log w = 0.1 * 4, phi = exp(k * lw + lam * (1 - exp(lw)))
    lw = torch.tensor(0.4)
    want = torch.exp(2.0 * lw + 3.0 * (1 - torch.exp(lw)))
    got = GRPOTrainer.get_gamma_weights(adv[:1], torch.full((1, 4), 0.1), mask[:1], None, 2.0, 3.0, 3.0, 2.0)
    assert torch.allclose(got.squeeze(), want, atol=1e-6)
    # the rollout correction enters unmasked, as one more log factor of the sequence weight
    isr = torch.full((1, 1), 2.0)
    got2 = GRPOTrainer.get_gamma_weights(adv[:1], torch.zeros(1, 4), mask[:1], isr, 2.0, 3.0, 3.0, 2.0)
    lw2 = torch.log(torch.tensor(2.0))
    assert torch.allclose(got2.squeeze(), torch.exp(2.0 * lw2 + 3.0 * (1 - torch.exp(lw2))), atol=1e-6)

    class _A:
        vllm_importance_sampling_mode = "token_truncate"
        vllm_importance_sampling_clip_max = None
        vllm_importance_sampling_clip_min = None

    class _T:
        args = _A()

    train, samp = torch.tensor([[0.0, 2.0]]), torch.tensor([[0.0, 0.0]])
    r = GRPOTrainer._rollout_is_ratio(_T(), train, samp, torch.ones(1, 2))
    assert torch.allclose(r, torch.exp(torch.tensor([[0.0, 2.0]])))  # no bound on either side
    _A.vllm_importance_sampling_mode, _A.vllm_importance_sampling_clip_max = "token_mask", 3.0
    r = GRPOTrainer._rollout_is_ratio(_T(), train, samp, torch.ones(1, 2))
    assert r.tolist() == [[1.0, 0.0]]


def test_deferred_metrics_resolve_to_global_ratios_and_means():
    from trl_b200.trainer.utils import defer_mean, defer_ratio, resolve_deferred_metrics

    m = {"entropy": [defer_ratio(torch.tensor(6.0), torch.tensor(4.0)), defer_ratio(torch.tensor(1.0), torch.tensor(0.0))],
         "policy_loss": [defer_mean(torch.tensor(0.25))], "plain": [1.5]}
    resolve_deferred_metrics(m)
    assert m == {"entropy": [1.5, 1.0], "policy_loss": [0.25], "plain": [1.5]}


def test_grpo_trains_from_a_streaming_dataset_with_functools_partial_reward(tmp_path, tiny_tokenizer):
    """A dataset without ``__len__`` goes through ``repeat_iterable_dataset``: every prompt of a generation batch
    appears ``num_generations`` times in a row, as with the index sampler; the reward's display name is the wrapped
    function's."""
    import functools

    class Stream:
        def __init__(self, rows):
            self.rows = rows

        def __iter__(self):
            return iter(self.rows)

    rows = [dict(r) for r in make_dataset("standard_prompt_only", 16)]
    seen = []

    def reward(completions, prompts=None, bonus=0.0, **kw):
        seen.append(list(prompts))
        return [len(c) * 0.1 + bonus for c in completions]

    args = GRPOConfig(output_dir=str(tmp_path), **dict(COMMON, max_steps=2), num_generations=4, max_completion_length=4)
    tr = GRPOTrainer(make_tiny_model(), functools.partial(reward, bonus=1.0), args, train_dataset=Stream(rows),
                     processing_class=tiny_tokenizer)
    assert tr.reward_func_names == ["reward"]
    tr.train()
    assert tr.state.global_step == 2 and seen
    first = seen[0]
    assert len(first) % 4 == 0 and all(len(set(first[i:i + 4])) == 1 for i in range(0, len(first), 4))


def test_other_optimizers_through_optim_and_optimizer_cls(tmp_path, tiny_tokenizer):
    """`optim="sgd"` and `optimizer_cls_and_kwargs` put the caller's update rule on the engine's fp32 master slices:
    one SGD step equals p - lr * clipped gradient, decay-exempt parameters get no weight decay, and the optimizer state
    survives a checkpoint."""
    from trl_b200 import SFTConfig, SFTTrainer

    rows = make_dataset("standard_language_modeling", 16)
    one_batch = make_dataset("standard_language_modeling", 4)  # whatever the order, the step sees these four rows
    base = dict(COMMON, max_steps=1, max_grad_norm=0.0, lr_scheduler_type="constant", learning_rate=0.5, weight_decay=0.0)
    model = make_tiny_model(seed=0)
    before = _snap(model)
    tr = SFTTrainer(model, SFTConfig(output_dir=str(tmp_path / "sgd"), optim="sgd", **base), train_dataset=one_batch,
                    processing_class=tiny_tokenizer)
    tr.train()
    assert isinstance(tr.engine.custom_opt, torch.optim.SGD)
    # the same gradient through autograd on a copy of the model and the same batch
    ref = make_tiny_model(seed=0)
    tr2 = SFTTrainer(ref, SFTConfig(output_dir=str(tmp_path / "ref"), **dict(base, max_steps=1, learning_rate=0.0)),
                     train_dataset=one_batch, processing_class=tiny_tokenizer)
    batch = next(iter(tr2.get_train_dataloader()))
    loss = tr2.compute_loss(ref, tr2._prepare_inputs(batch))
    loss.backward()
    g = {n: p.grad for n, p in ref.named_parameters()}  # no engine yet: plain autograd gradients
    # the loop divides the summed loss by the number of labelled tokens of the batch (first tokens included, as
    # transformers counts num_items_in_batch), compute_loss alone by the number of targets: one common factor
    d0, g0 = (before["lm_head"] - dict(model.named_parameters())["lm_head"]) / 0.5, g["lm_head"]
    c = float((d0 * g0).sum() / (g0 * g0).sum())
    assert 0.85 < c <= 1.0 + 1e-6
    for n, p in model.named_parameters():
        assert torch.allclose(p, before[n] - 0.5 * c * g[n], atol=1e-5), n

    # a class of the caller's, with weight decay: norm weights and biases are exempt
    class SignSGD(torch.optim.Optimizer):
        def __init__(self, params, lr=1e-3, weight_decay=0.0):
            super().__init__(params, dict(lr=lr, weight_decay=weight_decay))

        @torch.no_grad()
        def step(self):
            for grp in self.param_groups:
                for p in grp["params"]:
                    if p.grad is not None:
                        p.mul_(1 - grp["lr"] * grp["weight_decay"]).add_(p.grad.sign(), alpha=-grp["lr"])
                        self.state[p]["steps"] = self.state[p].get("steps", 0) + 1

    model = make_tiny_model(seed=0)
    before = _snap(model)
    cfg = SFTConfig(output_dir=str(tmp_path / "sign"), save_steps=2,
                    **dict(base, max_steps=2, learning_rate=0.01, weight_decay=0.5, save_strategy="steps"))
    tr = SFTTrainer(model, cfg, train_dataset=rows, processing_class=tiny_tokenizer, optimizer_cls_and_kwargs=(SignSGD, {}))
    tr.train()
    groups = tr.engine.custom_opt.param_groups
    assert groups[0]["weight_decay"] == 0.5 and groups[1]["weight_decay"] == 0.0 and groups[1]["params"]
    norm_name = next(n for n, _ in model.named_parameters() if "layernorm" in n)
    moved = (dict(model.named_parameters())[norm_name] - before[norm_name]).abs()
    assert float(moved.max()) <= 2 * 0.01 + 1e-6            # two sign steps, no decay on a norm weight (value 1.0)
    w_name = next(n for n, p in model.named_parameters() if p.ndim == 2 and "embed" not in n)
    assert float((dict(model.named_parameters())[w_name] - before[w_name]).abs().max()) > 0
    # resume: the custom state comes back
    model2 = make_tiny_model(seed=0)
    cfg2 = SFTConfig(output_dir=str(tmp_path / "sign"), **dict(base, max_steps=3, learning_rate=0.01, weight_decay=0.5))
    tr3 = SFTTrainer(model2, cfg2, train_dataset=rows, processing_class=tiny_tokenizer, optimizer_cls_and_kwargs=(SignSGD, {}))
    tr3.train(resume_from_checkpoint=True)
    assert tr3.state.global_step == 3
    assert max(st["steps"] for st in tr3.engine.custom_opt.state.values()) == 3
    with pytest.raises(NotImplementedError):
        SFTTrainer(make_tiny_model(), SFTConfig(output_dir=str(tmp_path / "x"), **COMMON), train_dataset=rows,
                   processing_class=tiny_tokenizer, optimizers=(torch.optim.SGD([torch.zeros(1, requires_grad=True)], lr=0.1), None))
    with pytest.raises(ValueError):
        SFTTrainer(make_tiny_model(), SFTConfig(output_dir=str(tmp_path / "y"), optim="lion_8bit", **COMMON),
                   train_dataset=rows, processing_class=tiny_tokenizer).train()


def test_sft_loss_matches_cross_entropy_and_its_corner_cases(tmp_path, tiny_tokenizer):
    """The fused lm_head loss of the SFT trainer against ``F.cross_entropy`` on explicit logits: ignore_index,
    ``num_items_in_batch`` as an int and as a tensor, a batch with no target at all (zero loss, connected graph),
    and ``shift_labels`` taking precedence over ``labels``."""
    import torch.nn.functional as F

    from trl_b200 import SFTConfig, SFTTrainer

    model = make_tiny_model(seed=0)
    tr = SFTTrainer(model, SFTConfig(output_dir=str(tmp_path), **COMMON), train_dataset=make_dataset("standard_language_modeling", 4),
                    processing_class=tiny_tokenizer)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(5, 1000, (3, 9), generator=g)
    labels = ids.clone()
    labels[0, :4] = -100      # a masked prompt
    labels[2, 5:] = -100      # a masked tail
    batch = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": labels}

    def reference(lab_shifted, denom=None):
        logits = model(input_ids=ids).logits.float()
        flat = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), lab_shifted.reshape(-1), ignore_index=-100, reduction="sum")
        n = (lab_shifted != -100).sum()
        return flat / (denom if denom is not None else n)
    shifted = torch.full_like(labels, -100)
    shifted[:, :-1] = labels[:, 1:]
    loss = tr.compute_loss(model, dict(batch))
    assert torch.allclose(loss, reference(shifted), atol=1e-5)
    # gradients agree too
    model.zero_grad()
    loss.backward()
    got = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    reference(shifted).backward()
    for n, p in model.named_parameters():
        assert torch.allclose(got[n], p.grad, atol=2e-5), n
    model.zero_grad()
    # the denominator handed over by the loop: an int or a tensor
    for denom in (7, torch.tensor(7)):
        assert torch.allclose(tr.compute_loss(model, dict(batch), num_items_in_batch=denom), reference(shifted, 7), atol=1e-5)
    # shift_labels (already shifted, e.g. by a sequence-parallel loader) win over labels
    other = torch.full_like(labels, -100)
    other[:, 2:5] = ids[:, 3:6]
    loss_s = tr.compute_loss(model, {**batch, "shift_labels": other})
    assert torch.allclose(loss_s, reference(other), atol=1e-5) and not torch.allclose(loss_s, loss)
    # nothing to predict: zero loss whose backward still reaches every parameter the forward used
    empty = tr.compute_loss(model, {**batch, "labels": torch.full_like(labels, -100)})
    assert float(empty) == 0.0 and empty.requires_grad
    empty.backward()
    assert all(p.grad is not None and float(p.grad.abs().sum()) == 0.0 for n, p in model.named_parameters())


def test_load_best_model_at_end_neftune_and_ignored_arguments(tmp_path, tiny_tokenizer):
    from safetensors.torch import load_file

    from trl_b200 import SFTConfig, SFTTrainer

    rows = make_dataset("standard_language_modeling", 16)
    model = make_tiny_model(seed=0)
    # a learning rate that makes the evaluation loss rise after the first checkpoint: the best one is the first
    args = SFTConfig(output_dir=str(tmp_path / "o"), eval_strategy="steps", eval_steps=1, save_steps=1, load_best_model_at_end=True,
                     metric_for_best_model="loss", **dict(COMMON, max_steps=3, learning_rate=0.3, save_strategy="steps",
                                                          lr_scheduler_type="constant"))
    with pytest.warns(UserWarning, match="torch_compile"):
        args.torch_compile = True
        tr = SFTTrainer(model, args, train_dataset=rows, eval_dataset=rows[:4] if isinstance(rows, list) else rows.select(range(4)),
                        processing_class=tiny_tokenizer)
        tr.train()
    evals = [(h["step"], h["eval_loss"]) for h in tr.state.log_history if "eval_loss" in h]
    best_step = min(evals, key=lambda t: t[1])[0]
    assert tr.state.best_model_checkpoint.endswith(f"checkpoint-{best_step}")
    saved = load_file(os.path.join(tr.state.best_model_checkpoint, "model.safetensors"))
    from trl_b200.models.hf_io import to_hf_state_dict

    now = to_hf_state_dict(model)
    assert all(torch.equal(now[k].float(), saved[k].float()) for k in saved)
    if best_step != 3:  # the final weights were replaced
        last = load_file(os.path.join(str(tmp_path / "o"), "checkpoint-3", "model.safetensors"))
        assert any(not torch.equal(last[k], saved[k]) for k in saved)
    # NEFTune: noise on the embeddings in training mode only, scaled by alpha / sqrt(L * H), removed after train()
    m2 = make_tiny_model(seed=0)
    ids = torch.randint(5, 1000, (2, 12))
    m2.train()
    clean = m2(input_ids=ids).logits
    m2.neftune_noise_alpha = 5.0
    noisy = m2(input_ids=ids).logits
    assert not torch.allclose(clean, noisy)
    m2.eval()
    assert torch.allclose(m2(input_ids=ids).logits, clean, atol=1e-6)
    tr2 = SFTTrainer(m2, SFTConfig(output_dir=str(tmp_path / "n"), neftune_noise_alpha=5.0, **COMMON), train_dataset=rows,
                     processing_class=tiny_tokenizer)
    m2.neftune_noise_alpha = None
    seen = {}
    orig = m2.forward_hidden

    def spy(*a, **kw):
        seen["alpha"] = m2.neftune_noise_alpha
        return orig(*a, **kw)
    m2.forward_hidden = spy
    tr2.train()
    assert seen["alpha"] == 5.0 and m2.neftune_noise_alpha is None


def test_group_by_length_batches_hold_similar_lengths(tmp_path, tiny_tokenizer):
    from trl_b200 import SFTConfig, SFTTrainer
    from trl_b200.loop.trainer import LengthGroupedSampler

    lengths = [3, 50, 4, 48, 5, 47, 6, 46, 7, 45, 8, 44]
    order = list(LengthGroupedSampler(lengths, batch_size=4, seed=0))
    assert sorted(order) == list(range(12)) and lengths[order[0]] == 50          # the longest sample comes first
    spans = [max(lengths[j] for j in order[i:i + 4]) - min(lengths[j] for j in order[i:i + 4]) for i in range(0, 12, 4)]
    assert sum(s < 10 for s in spans) >= 2, spans                                # batches are homogeneous in length
    assert list(LengthGroupedSampler(lengths, 4, seed=0)) == order               # reproducible
    s2 = LengthGroupedSampler(lengths, 4, seed=0)
    s2.set_epoch(1)
    assert sorted(s2) == list(range(12))
    rows = [{"text": " ".join(["word"] * n)} for n in (2, 30, 3, 28, 2, 31, 4, 29)]
    tr = SFTTrainer(make_tiny_model(), SFTConfig(output_dir=str(tmp_path), group_by_length=True, **COMMON), train_dataset=rows,
                    processing_class=tiny_tokenizer)
    batches = list(tr.get_train_dataloader())
    widths = [b["input_ids"].shape[1] for b in batches]
    assert max(widths) > 2 * min(widths)        # short samples sit together, long ones together
    tr.train()


def test_sft_evaluation_with_compute_metrics(tmp_path, tiny_tokenizer):
    """`compute_metrics` receives predictions and labels of the whole evaluation set (batches of different width are
    padded with -100); `preprocess_logits_for_metrics` turns logits into token ids before they are collected."""
    from trl_b200 import SFTConfig, SFTTrainer

    rows = [{"text": " ".join(["word"] * n)} for n in (3, 9, 4, 12, 5, 7)]
    seen = {}

    def metrics(ep):
        seen["pred"], seen["lab"] = ep.predictions.shape, ep.label_ids.shape
        valid = ep.label_ids[:, 1:] != -100
        acc = ((ep.predictions[:, :-1] == ep.label_ids[:, 1:]) & valid).sum() / max(1, valid.sum())
        return {"token_accuracy": float(acc)}
    tr = SFTTrainer(make_tiny_model(), SFTConfig(output_dir=str(tmp_path), per_device_eval_batch_size=2, **COMMON),
                    train_dataset=rows, eval_dataset=rows, processing_class=tiny_tokenizer, compute_metrics=metrics,
                    preprocess_logits_for_metrics=lambda logits, labels: logits.argmax(-1))
    out = tr.evaluate()
    assert "eval_token_accuracy" in out and 0.0 <= out["eval_token_accuracy"] <= 1.0 and "eval_loss" in out
    assert seen["pred"] == seen["lab"] and seen["pred"][0] == 6 and seen["pred"][1] >= 12


def test_bema_callback_schedule_weights_and_saved_model(tmp_path, tiny_tokenizer):
    """tests/test_callbacks.py:120-240: theta_0 restarts at ``update_after``, updates run every ``update_freq`` steps
    after it with the global step in beta/alpha, and ``output_dir/bema`` holds the running weights."""
    from unittest.mock import call, patch

    from trl_b200 import BEMACallback, load_model

    def run(cb, sub, patched=True):
        model = make_tiny_model("tiny-qwen2", seed=0)
        cfg = SFTConfig(output_dir=str(tmp_path / sub), per_device_train_batch_size=8, max_steps=9, learning_rate=1e-3,
                        save_strategy="no", report_to="none", use_cpu=True, bf16=False, logging_steps=100)
        tr = SFTTrainer(model, cfg, train_dataset=make_dataset("standard_language_modeling", 24), processing_class=tiny_tokenizer,
                        callbacks=[cb])
        if patched:
            with patch.object(cb, "_update_bema_weights") as m:
                tr.train()
            return m.call_args_list
        tr.train()
        return model

    assert run(BEMACallback(update_freq=2), "a") == [call(2), call(4), call(6), call(8)]
    assert run(BEMACallback(update_freq=3), "b") == [call(3), call(6), call(9)]
    assert run(BEMACallback(update_freq=2, update_after=3), "c") == [call(5), call(7), call(9)]

    cb = BEMACallback(update_freq=2, lag=10, multiplier=1.0)
    assert cb._ema_beta(6) == pytest.approx(16 ** -0.5) and cb._bema_alpha(6) == pytest.approx(16 ** -0.2)
    assert BEMACallback(min_ema_multiplier=0.9)._ema_beta(100) == 0.9
    theta0 = _snap(make_tiny_model("tiny-qwen2", seed=0))
    model = run(cb, "d", patched=False)
    saved = load_model(str(tmp_path / "d" / "bema"), dtype="float32")
    trained, bema = dict(model.named_parameters()), dict(saved.named_parameters())
    name = "layers.0.mlp.gate_proj.weight" if "layers.0.mlp.gate_proj.weight" in trained else next(iter(trained))
    assert not torch.equal(bema[name], trained[name].detach()) and not torch.equal(bema[name], theta0[name])
    # last update was at step 8, so the saved weights follow e_8 + alpha_8 (theta_8 - theta_0), not theta_9
    assert torch.allclose(cb.running[cb.names.index(name)], bema[name].detach().float(), atol=1e-6)
    for kw in (dict(bias_power=0.0), dict(ema_power=0.0)):
        run(BEMACallback(update_freq=2, **kw), "e" + str(len(kw)) + next(iter(kw)), patched=False)
    # a run too short for any update still writes the (initial) weights
    cb = BEMACallback(update_freq=400)
    run(cb, "f", patched=False)
    first = load_model(str(tmp_path / "f" / "bema"), dtype="float32")
    assert torch.allclose(dict(first.named_parameters())[name].detach(), theta0[name], atol=1e-6)


def test_sft_rejects_a_dataset_with_transform_unless_preparation_is_skipped(tmp_path, tiny_tokenizer):
    """tests/test_sft_trainer.py:1004-1020."""
    from datasets import Dataset

    def add_suffix(batch):
        batch["text"] = [t + " more" for t in batch["text"]]
        return batch

    ds = Dataset.from_dict({"text": ["hello world"] * 4}).with_transform(add_suffix)
    cfg = SFTConfig(output_dir=str(tmp_path), report_to="none", use_cpu=True, bf16=False)
    with pytest.raises(ValueError, match=r"Dataset\.with_transform\(\).*skip_prepare_dataset.*trainer-ready"):
        SFTTrainer(make_tiny_model(), cfg, train_dataset=ds, processing_class=tiny_tokenizer)


def test_dpo_drops_fully_truncated_rows_and_prepares_datasets_given_to_evaluate(tmp_path, tiny_tokenizer):
    """tests/test_dpo_trainer.py:1126-1149 and :278-330."""
    from datasets import Dataset

    ds = Dataset.from_dict({"prompt": ["Hi", "This is a very long prompt that fills up the whole max_length budget on its own"],
                            "chosen": [" there", " yes"], "rejected": [" bye", " no"]})
    short = len(tiny_tokenizer("Hi")["input_ids"])
    cfg = DPOConfig(output_dir=str(tmp_path / "a"), max_length=short + 3, truncation_mode="keep_start", report_to="none",
                    use_cpu=True, bf16=False)
    tr = DPOTrainer(make_tiny_model(), None, cfg, train_dataset=ds, processing_class=tiny_tokenizer)
    assert len(tr.train_dataset) == 1 and tr.train_dataset[0]["prompt_ids"] == tiny_tokenizer("Hi")["input_ids"]

    train, held_out = make_dataset("standard_preference", 16), make_dataset("standard_preference", 8)
    cfg = DPOConfig(output_dir=str(tmp_path / "b"), max_steps=1, precompute_ref_log_probs=True, report_to="none",
                    use_cpu=True, bf16=False, per_device_train_batch_size=4, save_strategy="no")
    tr = DPOTrainer(make_tiny_model(), None, cfg, train_dataset=train, processing_class=tiny_tokenizer)
    assert tr.evaluate(eval_dataset=held_out)["eval_loss"] is not None  # raw rows: tokenised and given reference log-probs
    both = tr.evaluate(eval_dataset={"x": held_out, "y": held_out})
    assert both["eval_x_loss"] == pytest.approx(both["eval_y_loss"])
    tr.train()
    with pytest.raises(ValueError, match="Cannot compute reference log-probs for a dataset passed to"):
        tr.evaluate(eval_dataset=held_out)
    # with an explicit reference model the same call stays legal after training
    cfg = DPOConfig(output_dir=str(tmp_path / "c"), max_steps=1, precompute_ref_log_probs=True, report_to="none",
                    use_cpu=True, bf16=False, per_device_train_batch_size=4, save_strategy="no")
    tr = DPOTrainer(make_tiny_model(), make_tiny_model(), cfg, train_dataset=train, eval_dataset={"x": held_out},
                    processing_class=tiny_tokenizer)
    tr.train()
    assert tr.evaluate(eval_dataset=held_out)["eval_loss"] is not None
    assert "eval_x_loss" in tr.evaluate()


@pytest.mark.parametrize("kind", ["sft", "reward", "kto"])
def test_evaluate_accepts_raw_datasets_and_dicts_of_them(tmp_path, tiny_tokenizer, kind):
    """`evaluate(eval_dataset=...)` takes unprepared rows, a dict / DatasetDict of them, or the name of a dataset given at
    construction (tests/test_reward_trainer.py:161-187, tests/test_kto_trainer.py:366-404, the same case for SFT)."""
    from datasets import DatasetDict

    common = dict(output_dir=str(tmp_path), report_to="none", use_cpu=True, bf16=False, per_device_train_batch_size=4,
                  per_device_eval_batch_size=4, save_strategy="no", max_steps=1)
    if kind == "sft":
        cls, cfg, data = SFTTrainer, SFTConfig(**common), "standard_prompt_completion"
        model = make_tiny_model()
    elif kind == "reward":
        cls, cfg, data = RewardTrainer, RewardConfig(**common), "standard_implicit_prompt_preference"
        model = make_tiny_model(num_labels=1)
    else:
        cls, cfg, data = KTOTrainer, KTOConfig(**common), "standard_unpaired_preference"
        model = make_tiny_model()
    train, held_out = make_dataset(data, 16), make_dataset(data, 8)
    kw = dict(train_dataset=train, eval_dataset={"a": held_out}, processing_class=tiny_tokenizer)
    tr = cls(model, cfg, **kw) if kind != "kto" else cls(model, None, cfg, **kw)
    assert tr.evaluate(eval_dataset=held_out)["eval_loss"] is not None
    for given in ({"d1": held_out, "d2": held_out}, DatasetDict({"d1": held_out, "d2": held_out})):
        m = tr.evaluate(eval_dataset=given)
        assert m["eval_d1_loss"] == pytest.approx(m["eval_d2_loss"])
    assert "eval_a_loss" in tr.evaluate() and "eval_a_loss" in tr.evaluate(eval_dataset="a")


@pytest.mark.parametrize("loss_type", ["kto", "apo_zero_unpaired"])
def test_kto_precomputed_reference_log_probs_match_the_live_reference(tmp_path, tiny_tokenizer, loss_type):
    """With `precompute_ref_log_probs` the datasets carry ref_logps (and ref_KL_logps for the KL estimate), no reference
    copy is kept, and the first losses equal those of a run with a live reference (tests/test_kto_trainer.py:299-334,
    :406-426)."""
    def run(sub, **kw):
        cfg = KTOConfig(output_dir=str(tmp_path / sub), report_to="none", use_cpu=True, bf16=False, loss_type=loss_type,
                        per_device_train_batch_size=4, per_device_eval_batch_size=4, save_strategy="no", max_steps=2,
                        logging_steps=1, learning_rate=1e-4, train_sampling_strategy="sequential", **kw)
        tr = KTOTrainer(make_tiny_model(seed=0), None, cfg, train_dataset=make_dataset("standard_unpaired_preference", 16),
                        eval_dataset=make_dataset("standard_unpaired_preference", 8), processing_class=tiny_tokenizer)
        tr.train()
        return tr

    live, pre = run("live"), run("pre", precompute_ref_log_probs=True)
    assert pre.ref_model is None and "ref_logps" in pre.train_dataset.column_names
    assert ("ref_KL_logps" in pre.train_dataset.column_names) == (loss_type == "kto")
    assert "ref_logps" in pre.eval_dataset.column_names
    a = [h["loss"] for h in live.state.log_history if "loss" in h]
    b = [h["loss"] for h in pre.state.log_history if "loss" in h]
    assert a == pytest.approx(b, abs=1e-5)
    with pytest.raises(ValueError, match="Cannot compute reference log-probs"):
        pre.evaluate(eval_dataset=make_dataset("standard_unpaired_preference", 8))
    assert pre.evaluate()["eval_loss"] is not None
