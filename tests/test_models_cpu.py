"""Native decoder vs transformers reference implementations (CPU, fp32), checkpoint round trips, LoRA."""
import os

import pytest
import torch

from trl_b200.models.configuration import ModelArch, preset
from trl_b200.models.decoder import CausalLM, SeqCtx
from trl_b200.models.hf_io import load_model, to_hf_state_dict


def _hf_model(cfg: ModelArch):
    import transformers as tf

    d = cfg.to_hf_dict()
    cls = {"qwen2": (tf.Qwen2Config, tf.Qwen2ForCausalLM), "llama": (tf.LlamaConfig, tf.LlamaForCausalLM),
           "qwen3_moe": (tf.Qwen3MoeConfig, tf.Qwen3MoeForCausalLM)}[cfg.model_type]
    d.pop("architectures", None)
    d.pop("torch_dtype", None)
    hf = cls[1](cls[0](**d, attn_implementation="eager")).eval()
    return hf


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-llama", "tiny-qwen3-moe", "tiny-mistral", "tiny-phi3", "tiny-qwen3", "tiny-gemma"])
def test_logits_match_transformers(name, tmp_path):
    torch.manual_seed(0)
    cfg = preset(name)
    ours = CausalLM(cfg).eval()
    ours.save_pretrained(str(tmp_path))
    import transformers as tf

    hf = tf.AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32, attn_implementation="eager").eval()
    ids = torch.randint(0, cfg.vocab_size, (2, 17))
    am = torch.ones_like(ids)
    am[1, 11:] = 0
    with torch.no_grad():
        a = ours(input_ids=ids, attention_mask=am).logits
        b = hf(input_ids=ids, attention_mask=am).logits
    m = am.bool()
    assert torch.allclose(a[m], b[m], atol=2e-4, rtol=1e-3), (a[m] - b[m]).abs().max()


def test_packed_equals_padded():
    torch.manual_seed(0)
    m = CausalLM(preset("tiny-qwen2")).eval()
    a, b = torch.randint(0, 1024, (9,)), torch.randint(0, 1024, (5,))
    with torch.no_grad():
        packed = m(input_ids=torch.cat([a, b])[None], position_ids=torch.cat([torch.arange(9), torch.arange(5)])[None]).logits[0]
        la = m(input_ids=a[None]).logits[0]
        lb = m(input_ids=b[None]).logits[0]
    assert torch.allclose(packed[:9], la, atol=1e-5) and torch.allclose(packed[9:], lb, atol=1e-5)


def test_save_load_round_trip_and_hf_names(tmp_path):
    m = CausalLM(preset("tiny-qwen2"))
    m.save_pretrained(str(tmp_path))
    assert os.path.exists(tmp_path / "model.safetensors") and os.path.exists(tmp_path / "config.json")
    sd = to_hf_state_dict(m)
    assert "model.layers.0.self_attn.q_proj.weight" in sd and "model.layers.1.mlp.gate_proj.weight" in sd
    assert "model.layers.0.self_attn.q_proj.bias" in sd and "lm_head.weight" in sd
    m2 = load_model(str(tmp_path))
    for (n, p), (_, q) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(p, q), n


def test_reward_head_scores_last_token():
    m = CausalLM(preset("tiny-qwen2", num_labels=1)).eval()
    ids = torch.randint(0, 1024, (2, 8))
    am = torch.ones_like(ids)
    am[0, 5:] = 0
    with torch.no_grad():
        out = m(input_ids=ids, attention_mask=am).logits
        solo = m(input_ids=ids[:1, :5]).logits
    assert out.shape == (2, 1) and torch.allclose(out[0], solo[0], atol=1e-5)


def test_lora_adapters_train_and_round_trip(tmp_path):
    from trl_b200.models.lora import LoraConfig, get_peft_model, load_adapter, save_adapter

    torch.manual_seed(0)
    m = get_peft_model(CausalLM(preset("tiny-qwen2")), LoraConfig(r=4, lora_alpha=8, lora_dropout=0.0,
                                                                  target_modules=["q_proj", "v_proj", "down_proj"]))
    train = [n for n, p in m.named_parameters() if p.requires_grad]
    assert train and all("lora_" in n for n in train)
    ids = torch.randint(0, 1024, (1, 12))
    base = m(input_ids=ids).logits
    for l in m.layers:
        for s in l.lora.values():
            torch.nn.init.normal_(s.lora_B, std=0.05)
    tuned = m(input_ids=ids).logits
    assert not torch.allclose(base, tuned)
    m.set_adapter_enabled(False)
    assert torch.allclose(m(input_ids=ids).logits, base, atol=1e-6)
    m.set_adapter_enabled(True)
    save_adapter(m, str(tmp_path))
    from safetensors.torch import load_file

    keys = list(load_file(str(tmp_path / "adapter_model.safetensors")))
    assert "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight" in keys
    m2 = get_peft_model(CausalLM(preset("tiny-qwen2")), LoraConfig(r=4, lora_alpha=8, lora_dropout=0.0,
                                                                   target_modules=["q_proj", "v_proj", "down_proj"]))
    m2.load_state_dict({k: v for k, v in m.state_dict().items() if "lora" not in k}, strict=False)
    load_adapter(m2, str(tmp_path))
    assert torch.allclose(m2(input_ids=ids).logits, tuned, atol=1e-5)
    # merge == adapter forward
    m.merge_adapter()
    m.set_adapter_enabled(False)
    assert torch.allclose(m(input_ids=ids).logits, tuned, atol=1e-4)


def test_partial_gradient_checkpointing_matches_full_activations():
    torch.manual_seed(0)
    m = CausalLM(preset("tiny-qwen2")).train()
    ids = torch.randint(0, 1024, (2, 12))

    def grads():
        m.zero_grad()
        m(input_ids=ids).logits.float().logsumexp(-1).sum().backward()
        return [p.grad.clone() for p in m.parameters()]

    ref = grads()
    m.gradient_checkpointing_enable({"num_layers": 1})  # recompute layer 0 only
    assert m.checkpoint_num_layers == 1
    part = grads()
    m.gradient_checkpointing_enable()  # back to all layers
    assert m.checkpoint_num_layers is None
    full = grads()
    for a, b, c in zip(ref, part, full):
        assert torch.allclose(a, b, atol=1e-6) and torch.allclose(a, c, atol=1e-6)


def test_context_parallel_attention_segments_match_full_attention():
    """A chunk's queries against the gathered keys (mask aligned to the end of each key segment) equal the same rows
    of full packed attention."""
    from trl_b200.oracle import ops as O
    from trl_b200.parallel import context_parallel as cp
    from trl_b200.parallel.ulysses import SpInfo

    torch.manual_seed(0)
    cu = torch.tensor([0, 5, 19, 24, 32], dtype=torch.int32)  # four documents in a 32-token stream
    T, Hq, Hk, D = 32, 4, 2, 8
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hk, D), torch.randn(T, Hk, D)
    full = O.attention_varlen(q, k, v, cu)
    for size in (2, 4):
        tl = T // size
        for r in range(size):
            ctx = SeqCtx(torch.zeros(tl, dtype=torch.int32), cu, 14)
            ctx.sp = SpInfo(None, size, r, "allgather_kv")
            p = cp.plan(ctx)
            out = O.attention_varlen_qk(q[r * tl:(r + 1) * tl], k[p["k_start"]:p["k_end"]], v[p["k_start"]:p["k_end"]],
                                        p["cu_q"], p["cu_k"])
            assert torch.allclose(out, full[r * tl:(r + 1) * tl], atol=1e-5), (size, r)


def test_sliding_window_attention_matches_transformers(tmp_path):
    import transformers as tf

    torch.manual_seed(0)
    cfg = preset("tiny-mistral", sliding_window=6)
    ours = CausalLM(cfg).eval()
    ours.save_pretrained(str(tmp_path))
    assert ModelArch.from_pretrained(str(tmp_path)).sliding_window == 6
    hf = tf.AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32, attn_implementation="eager").eval()
    ids = torch.randint(0, cfg.vocab_size, (2, 19))
    with torch.no_grad():
        a = ours(input_ids=ids).logits
        b = hf(input_ids=ids).logits
        full = CausalLM(preset("tiny-mistral"))
        full.load_state_dict(ours.state_dict())
        c = full.eval()(input_ids=ids).logits
    assert torch.allclose(a, b, atol=2e-4, rtol=1e-3), (a - b).abs().max()
    assert not torch.allclose(a[:, 8:], c[:, 8:], atol=1e-3)  # the window really changes the later positions
    # the Qwen families carry a sliding_window value that is off unless use_sliding_window is set
    d = preset("tiny-qwen2").to_hf_dict()
    d["sliding_window"] = 4096
    assert ModelArch.from_hf_dict(d).sliding_window is None


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-qwen3-moe", "tiny-phi3"])
def test_loads_checkpoints_written_by_transformers(name, tmp_path):
    """The other direction of the round trip: transformers saves, the native loader reads (per-expert or fused MoE
    tensors, fused Phi-3 projections)."""
    torch.manual_seed(0)
    hf = _hf_model(preset(name)) if name != "tiny-phi3" else None
    if hf is None:
        import transformers as tf

        d = preset(name).to_hf_dict()
        d.pop("architectures", None)
        hf = tf.Phi3ForCausalLM(tf.Phi3Config(**d, attn_implementation="eager")).eval()
    hf.save_pretrained(str(tmp_path))
    ours = load_model(str(tmp_path)).eval()
    ids = torch.randint(0, ours.config.vocab_size, (2, 11))
    with torch.no_grad():
        a, b = ours(input_ids=ids).logits, hf(input_ids=ids).logits
    assert torch.allclose(a, b, atol=2e-4, rtol=1e-3), (a - b).abs().max()


def test_eager_generator_greedy_matches_transformers_generate(tmp_path):
    import transformers as tf

    from trl_b200.rollout.engine import EagerGenerator
    from trl_b200.rollout.sampling import SamplingParams

    torch.manual_seed(0)
    m = CausalLM(preset("tiny-qwen2")).eval()
    m.save_pretrained(str(tmp_path))
    hf = tf.AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    prompt = torch.randint(5, 1000, (1, 9))
    ref = hf.generate(prompt, max_new_tokens=8, do_sample=False, eos_token_id=None, pad_token_id=0)[0, 9:].tolist()
    out = EagerGenerator(m).generate([prompt[0].tolist()], SamplingParams(n=1, max_tokens=8, greedy=True, eos_token_id=None))
    assert out[0].token_ids == ref
    # the reported log-probs are those of the chosen tokens under the model
    with torch.no_grad():
        full = torch.tensor([prompt[0].tolist() + ref])
        lp = torch.log_softmax(hf(full).logits[0, 8:-1].float(), -1).gather(1, torch.tensor(ref)[:, None])[:, 0]
    assert torch.allclose(torch.tensor(out[0].logprobs), lp, atol=1e-4)


def test_export_merged_weights_gives_a_plain_model_equal_to_the_adapted_one():
    """The generation replica of an adapted policy: adapters folded in, the policy itself untouched."""
    import copy

    from trl_b200.models.decoder import CausalLM
    from trl_b200.models.lora import LoraConfig, export_merged_weights, get_peft_model
    from trl_b200.testing import make_tiny_model

    model = make_tiny_model("tiny-qwen2", seed=0)
    get_peft_model(model, LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj", "v_proj", "gate_proj", "down_proj"]))
    model.eval()  # no adapter dropout
    g = torch.Generator().manual_seed(1)
    for l in model.layers:
        for slot in l.lora.values():
            slot.lora_B.data.normal_(0, 0.05, generator=g)  # a fresh adapter has B = 0: make it matter
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    replica = CausalLM(model.config, dtype=model.dtype, init=False)
    export_merged_weights(model, replica)
    assert all(torch.equal(before[n], p) for n, p in model.named_parameters())  # the policy is not merged into
    assert not any(len(l.lora) for l in replica.layers)
    ids = torch.randint(0, 1024, (2, 17), generator=g)
    with torch.no_grad():
        want = model(input_ids=ids).logits
        got = replica(input_ids=ids).logits
        model.set_adapter_enabled(False)
        base = model(input_ids=ids).logits
        model.set_adapter_enabled(True)
    assert torch.allclose(got, want, atol=2e-5) and (want - base).abs().max() > 1e-3


def test_use_adapter_disables_and_restores():
    """`use_adapter(model, None)` runs the base model and puts the adapter back; naming the active adapter is a no-op
    (the checks of tests/test_utils.py:66-95 on the native LoRA model)."""
    import pytest

    from trl_b200.models.lora import LoraConfig, get_peft_model
    from trl_b200.testing import make_tiny_model
    from trl_b200.trainer.utils import use_adapter

    torch.manual_seed(0)
    base = make_tiny_model(seed=0).eval()
    model = get_peft_model(make_tiny_model(seed=0), LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj", "v_proj"]),
                           adapter_name="my_adapter").eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "lora" in n and n.endswith("B"):
                p.normal_(0, 0.05)  # a fresh adapter is the identity: make it matter
    ids = torch.tensor([[1, 2, 3], [4, 5, 6]])
    with torch.no_grad():
        adapted = model(input_ids=ids).logits
        plain = base(input_ids=ids).logits
        assert not torch.allclose(adapted, plain)
        with use_adapter(model, None):
            assert torch.equal(model(input_ids=ids).logits, plain)
        assert torch.equal(model(input_ids=ids).logits, adapted)
        with use_adapter(model, "my_adapter"):
            assert torch.equal(model(input_ids=ids).logits, adapted)
        assert torch.equal(model(input_ids=ids).logits, adapted)
    with pytest.raises(NotImplementedError):
        with use_adapter(model, "another"):
            pass
    with use_adapter(base, None):  # a model without adapters passes through
        pass


def test_get_peft_config_from_model_config():
    """tests/test_utils.py:253-283: nothing without `use_peft`; otherwise every `lora_*` field arrives in the LoraConfig."""
    from trl_b200 import ModelConfig
    from trl_b200.models.lora import LoraConfig
    from trl_b200.trainer.utils import get_peft_config

    assert get_peft_config(ModelConfig(use_peft=False)) is None
    kw = {"lora_r": 8, "lora_alpha": 16, "lora_dropout": 0.1, "lora_task_type": "SEQ_CLS", "use_rslora": True,
          "lora_target_modules": ["up_proj", "down_proj"], "lora_modules_to_save": ["up_proj"]}
    cfg = get_peft_config(ModelConfig(use_peft=True, **kw))
    assert isinstance(cfg, LoraConfig)
    assert (cfg.r, cfg.lora_alpha, cfg.lora_dropout, cfg.task_type, cfg.use_rslora) == (8, 16, 0.1, "SEQ_CLS", True)
    assert set(cfg.target_modules) == {"up_proj", "down_proj"} and list(cfg.modules_to_save) == ["up_proj"]
