"""Trainers end to end on one GPU: bf16 tiny models whose shapes take the kernel paths (head dim 128: tcgen05
attention in training and decode, fused lm_head losses, the in-process rollout engine under CUDA graphs).  Criterion as
on the CPU: the loss is logged, it is finite, and every trainable parameter moved."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

COMMON = dict(per_device_train_batch_size=4, max_steps=2, logging_steps=1, learning_rate=5e-3, save_strategy="no",
              report_to="none", bf16=True)
# the learning rate is large on purpose: norm weights start at 1.0, where one bf16 step is 2^-8, and the check below
# looks at the bf16 parameters (the fp32 master copies move with any rate)
SHAPE = dict(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128, intermediate_size=512,
             num_hidden_layers=2)


def _model():
    from trl_b200.testing import make_tiny_model

    return make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device="cuda", seed=0, **SHAPE)


def _snap(model):
    return {n: p.detach().clone() for n, p in model.named_parameters()}


def _unchanged(model, before):
    return [n for n, p in model.named_parameters() if p.requires_grad and torch.equal(before[n], p)]


def _len_reward(completions, **kw):
    return [float(len(c)) * 0.1 + (hash(c) % 7) * 0.01 for c in completions]


def _finite_losses(tr):
    losses = [h["loss"] for h in tr.state.log_history if "loss" in h]
    assert losses and all(math.isfinite(x) for x in losses), tr.state.log_history
    assert "train_loss" in tr.state.log_history[-1]


def test_sft_and_dpo_train_on_the_gpu(tmp_path, tiny_tokenizer):
    from trl_b200 import DPOConfig, DPOTrainer, SFTConfig, SFTTrainer
    from trl_b200.ops import cuda as K
    from trl_b200.testing import make_dataset

    model = _model()
    before = _snap(model)
    tr = SFTTrainer(model, SFTConfig(output_dir=str(tmp_path / "sft"), padding_free=True, **COMMON),
                    train_dataset=make_dataset("standard_prompt_completion", 16), processing_class=tiny_tokenizer)
    tr.train()
    _finite_losses(tr)
    assert _unchanged(model, before) == []
    model = _model()
    before = _snap(model)
    tr = DPOTrainer(model, None, DPOConfig(output_dir=str(tmp_path / "dpo"), **COMMON),
                    train_dataset=make_dataset("standard_preference", 16), processing_class=tiny_tokenizer)
    tr.train()
    _finite_losses(tr)
    assert _unchanged(model, before) == []
    torch.cuda.synchronize()
    K.check_status(torch.device("cuda"))


def test_grpo_trains_on_the_gpu_with_the_rollout_engine(tmp_path, tiny_tokenizer):
    from trl_b200 import GRPOConfig, GRPOTrainer
    from trl_b200.ops import cuda as K
    from trl_b200.rollout.engine import RolloutEngine
    from trl_b200.testing import make_dataset

    model = _model()
    before = _snap(model)
    args = GRPOConfig(output_dir=str(tmp_path), **COMMON, num_generations=4, max_completion_length=8, beta=0.04,
                      gradient_accumulation_steps=2, use_vllm=True, vllm_mode="colocate")
    tr = GRPOTrainer(model, _len_reward, args, train_dataset=make_dataset("standard_prompt_only", 16),
                     processing_class=tiny_tokenizer)
    tr.train()
    assert isinstance(tr._rollout, RolloutEngine)  # not the eager fallback
    _finite_losses(tr)
    assert _unchanged(model, before) == []
    h = [x for x in tr.state.log_history if "reward" in x][-1]
    assert "completions/mean_length" in h and "kl" in h
    torch.cuda.synchronize()
    K.check_status(torch.device("cuda"))


def test_grpo_with_adapters_generates_from_a_merged_replica(tmp_path, tiny_tokenizer):
    """With LoRA the decode kernels cannot read the policy's matrices directly: generation must run on a replica with
    the adapters folded in, refreshed before each generation batch, and the base weights must stay bit-identical."""
    from trl_b200 import GRPOConfig, GRPOTrainer
    from trl_b200.models.lora import LoraConfig
    from trl_b200.ops import cuda as K
    from trl_b200.testing import make_dataset

    model = _model()
    args = GRPOConfig(output_dir=str(tmp_path), **COMMON, num_generations=4, max_completion_length=8,
                      use_vllm=True, vllm_mode="colocate")
    tr = GRPOTrainer(model, _len_reward, args, train_dataset=make_dataset("standard_prompt_only", 16),
                     processing_class=tiny_tokenizer,
                     peft_config=LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj", "v_proj", "down_proj"]))
    base = {n: p.detach().clone() for n, p in tr.model.named_parameters() if not p.requires_grad}
    tr.train()
    _finite_losses(tr)
    assert getattr(tr, "_gen_model", None) is not None and tr._rollout.model is tr._gen_model
    assert all(torch.equal(base[n], p) for n, p in tr.model.named_parameters() if n in base)  # never merged into
    # the replica holds W + scaling * B A for an adapted slice, W for the rest
    l_src, l_dst = tr.model.layers[0], tr._gen_model.layers[0]
    from trl_b200.models.lora import export_merged_weights

    export_merged_weights(tr.model, tr._gen_model)
    pname, sl = l_src.proj_slices()["q_proj"]
    want = getattr(l_src, pname)[sl].float() + l_src.lora["q_proj"].delta_weight()
    assert torch.allclose(getattr(l_dst, pname)[sl].float(), want, atol=2e-2)
    assert torch.equal(l_dst.gate_up_proj, l_src.gate_up_proj)
    assert any(float(s.lora_B.abs().max()) > 0 for s in l_src.lora.values())  # the adapters were trained
    torch.cuda.synchronize()
    K.check_status(torch.device("cuda"))


def test_qwen2_vl_sft_and_grpo_on_the_gpu(tmp_path):
    """Dynamic-resolution tower + multimodal RoPE in bf16 on the GPU: SFT with images of two sizes, then GRPO whose
    rollouts run on the paged engine with the per-slot rotary lead."""
    import numpy as np

    from trl_b200 import GRPOConfig, GRPOTrainer, SFTConfig, SFTTrainer
    from trl_b200.models.configuration import preset
    from trl_b200.models.vision_processing import DynamicResolutionProcessor
    from trl_b200.models.vision_qwen import Qwen2VLArch, Qwen2VLModel, QwenVisionArch
    from trl_b200.rollout.engine import RolloutEngine
    from trl_b200.testing import make_tiny_tokenizer

    tok = make_tiny_tokenizer()  # its own copy: the processor adds the image token
    proc = DynamicResolutionProcessor(tok, min_pixels=28 * 28, max_pixels=56 * 56)
    text = preset("tiny-qwen2", vocab_size=max(1024, len(tok)), **SHAPE)
    text.extra["mrope_section"] = [16, 24, 24]
    arch = Qwen2VLArch(text, QwenVisionArch(depth=2, embed_dim=64, hidden_size=SHAPE["hidden_size"], num_heads=2, mlp_ratio=2),
                       image_token_id=proc.image_token_id)
    torch.manual_seed(0)
    model = Qwen2VLModel(arch, dtype=torch.bfloat16, device="cuda")
    rs = np.random.RandomState(0)
    imgs = [(rs.rand(28 * (1 + i % 2), 56, 3) * 255).astype("uint8") for i in range(8)]
    rows = [{"images": [im], "messages": [{"role": "user", "content": "what is this"},
                                          {"role": "assistant", "content": "a picture " + "ab"[i % 2]}]}
            for i, im in enumerate(imgs)]
    before = _snap(model)
    tr = SFTTrainer(model, SFTConfig(output_dir=str(tmp_path / "sft"), max_length=None, **COMMON), train_dataset=rows,
                    processing_class=proc)
    tr.train()
    _finite_losses(tr)
    still = _unchanged(model, before)
    assert not [n for n in still if "visual" in n and n.endswith("_w")], still
    prompts = [{"image": im, "prompt": [{"role": "user", "content": "describe"}]} for im in imgs]
    args = GRPOConfig(output_dir=str(tmp_path / "grpo"), num_generations=4, max_completion_length=8, beta=0.04,
                      temperature=1.0, **COMMON)
    tr2 = GRPOTrainer(model, lambda completion_ids, **kw: [float(sum(c) % 7) for c in completion_ids], args,
                      train_dataset=prompts, processing_class=proc)
    tr2.train()
    assert isinstance(tr2._rollout, RolloutEngine) and tr2._rollout.rope_delta is not None
    logs = [h for h in tr2.state.log_history if "reward" in h]
    assert logs and all(math.isfinite(h["loss"]) for h in logs)


def test_sft_with_another_optimizer_on_the_gpu(tmp_path, tiny_tokenizer):
    """`optim="sgd"` on a bf16 model: the update runs on the fp32 master slices and the bf16 copy follows it."""
    from trl_b200 import SFTConfig, SFTTrainer
    from trl_b200.testing import make_dataset

    model = _model()
    before = _snap(model)
    args = SFTConfig(output_dir=str(tmp_path), optim="sgd", optim_args="momentum=0.9", **dict(COMMON, learning_rate=0.5))
    tr = SFTTrainer(model, args, train_dataset=make_dataset("standard_language_modeling", 16), processing_class=tiny_tokenizer)
    tr.train()
    _finite_losses(tr)
    assert isinstance(tr.engine.custom_opt, torch.optim.SGD)
    # norm weights sit at 1.0, where one bf16 step is 2^-7: their fp32 master copies move, the bf16 values may not
    assert all("norm" in n for n in _unchanged(model, before)), _unchanged(model, before)
    b = tr.engine.buckets[0]
    assert b.master.dtype == torch.float32 and b.flat_param.dtype == torch.bfloat16
    assert torch.equal(b.flat_param[b.lo:b.hi], b.master.to(torch.bfloat16))
