"""Vision-language model (CLIP tower + projector + native decoder) vs transformers' LLaVA, checkpoints, SFT."""
import torch

from trl_b200.models.vision import VisionLanguageModel, tiny_vlm_arch


def _ids_with_images(cfg, n_images_per_row, length, gen):
    ids = torch.randint(10, cfg.vocab_size, (len(n_images_per_row), length), generator=gen)
    for r, n in enumerate(n_images_per_row):
        for j in range(n):
            s = 2 + j * (cfg.image_seq_length + 1)
            ids[r, s:s + cfg.image_seq_length] = cfg.image_token_index
    return ids


def test_vlm_logits_match_transformers_llava(tmp_path):
    import transformers as tf

    torch.manual_seed(0)
    cfg = tiny_vlm_arch("tiny-llama")
    ours = VisionLanguageModel(cfg).eval()
    for p in ours.vision_tower.parameters():  # biases and norms away from their init values
        if p.ndim == 1:
            p.data.add_(torch.randn_like(p) * 0.05)
    ours.save_pretrained(str(tmp_path))
    hf = tf.LlavaForConditionalGeneration.from_pretrained(str(tmp_path), dtype=torch.float32,
                                                          attn_implementation="eager").eval()
    g = torch.Generator().manual_seed(1)
    ids = _ids_with_images(cfg, [1, 2], 20, g)
    am = torch.ones_like(ids)
    am[0, 15:] = 0
    pix = torch.randn(3, 3, 28, 28, generator=g)
    with torch.no_grad():
        a = ours(input_ids=ids, attention_mask=am, pixel_values=pix).logits
        b = hf(input_ids=ids, attention_mask=am, pixel_values=pix).logits
    m = am.bool()
    assert torch.allclose(a[m], b[m], atol=3e-4, rtol=1e-3), (a[m] - b[m]).abs().max()


def test_vlm_checkpoint_round_trip_and_gradients(tmp_path):
    torch.manual_seed(0)
    cfg = tiny_vlm_arch("tiny-qwen2")
    m = VisionLanguageModel(cfg)
    m.save_pretrained(str(tmp_path))
    m2 = VisionLanguageModel.from_pretrained(str(tmp_path))
    for (n1, p1), (n2, p2) in zip(m.named_parameters(), m2.named_parameters()):
        assert n1 == n2 and torch.equal(p1, p2), n1
    g = torch.Generator().manual_seed(2)
    ids = _ids_with_images(cfg, [1], 12, g)
    pix = torch.randn(1, 3, 28, 28, generator=g)
    out = m2(input_ids=ids, pixel_values=pix, labels=ids)
    out.loss.backward()
    assert m2.vision_tower.patch_embedding.grad.abs().sum() > 0 and m2.proj1_w.grad.abs().sum() > 0
    assert m2.vision_tower.layers[-1].qkv_w.grad is None  # feature layer -2: the last tower layer is never run


def _vlm_and_processor():
    from trl_b200.models.vision_processing import VisionProcessor
    from trl_b200.testing import make_tiny_tokenizer

    tok = make_tiny_tokenizer()
    proc = VisionProcessor(tok, image_size=28, image_seq_length=4)
    torch.manual_seed(0)
    model = VisionLanguageModel(tiny_vlm_arch("tiny-qwen2", image_token_index=proc.image_token_id))
    assert VisionProcessor.for_model(tok, model).image_token_id == proc.image_token_id
    return model, proc


def test_vision_collator_language_modeling_and_prompt_completion():
    import numpy as np

    from trl_b200.trainer.sft_trainer import DataCollatorForVisionLanguageModeling

    _, proc = _vlm_and_processor()
    img = (np.random.RandomState(0).rand(40, 30, 3) * 255).astype("uint8")
    ex = [{"images": [img], "messages": [{"role": "user", "content": "what is this"},
                                         {"role": "assistant", "content": "a simple idea"}]},
          {"images": [img, img], "messages": [{"role": "user", "content": "explain"},
                                              {"role": "assistant", "content": "two"}]}]
    out = DataCollatorForVisionLanguageModeling(proc)(ex)
    assert out["pixel_values"].shape == (3, 3, 28, 28)
    n_img_tok = (out["input_ids"] == proc.image_token_id).sum(1).tolist()
    assert n_img_tok == [4, 8]
    assert (out["labels"][out["attention_mask"] == 0] == -100).all()
    # prompt-completion with completion-only loss: prompt (and its images) masked, completion kept
    pc = [{"image": img, "prompt": [{"role": "user", "content": "what is this"}],
           "completion": [{"role": "assistant", "content": "a simple idea"}]}]
    out = DataCollatorForVisionLanguageModeling(proc, completion_only_loss=True)(pc)
    lab, ids = out["labels"][0], out["input_ids"][0]
    assert (lab[ids == proc.image_token_id] == -100).all() and (lab != -100).sum() >= 3
    assert out["pixel_values"].shape[0] == 1


def test_sft_trains_vision_language_model(tmp_path):
    import numpy as np

    from trl_b200 import SFTConfig, SFTTrainer

    model, proc = _vlm_and_processor()
    rs = np.random.RandomState(1)
    rows = []
    for i in range(8):
        bright = i % 2
        img = (rs.rand(28, 28, 3) * 60 + (160 if bright else 10)).astype("uint8")
        rows.append({"images": [img], "messages": [{"role": "user", "content": "is it day or night"},
                                                   {"role": "assistant", "content": "day" if bright else "night"}]})
    args = SFTConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, max_steps=6, logging_steps=1,
                     learning_rate=3e-3, use_cpu=True, save_strategy="no", report_to="none", max_length=None,
                     lr_scheduler_type="constant")
    tr = SFTTrainer(model, args, train_dataset=rows, processing_class=proc)
    w0 = model.vision_tower.patch_embedding.detach().clone()
    tr.train()
    losses = [h["loss"] for h in tr.state.log_history if "loss" in h]
    assert losses[-1] < losses[0]
    assert not torch.equal(w0, model.vision_tower.patch_embedding)  # the tower trains through the projector
    tr.save_model(str(tmp_path / "final"))
    re = VisionLanguageModel.from_pretrained(str(tmp_path / "final"))
    assert torch.equal(re.proj1_w, model.proj1_w)


def test_dpo_trains_vision_language_model(tmp_path):
    import numpy as np

    from trl_b200 import DPOConfig, DPOTrainer
    from trl_b200.trainer.dpo_trainer import DataCollatorForVisionPreference

    model, proc = _vlm_and_processor()
    rs = np.random.RandomState(2)
    rows = []
    for i in range(8):
        bright = i % 2
        img = (rs.rand(28, 28, 3) * 60 + (160 if bright else 10)).astype("uint8")
        good, bad = ("day", "night") if bright else ("night", "day")
        rows.append({"images": [img], "prompt": [{"role": "user", "content": "is it day or night"}],
                     "chosen": [{"role": "assistant", "content": good}],
                     "rejected": [{"role": "assistant", "content": bad}]})
    batch = DataCollatorForVisionPreference(proc)(rows[:2])
    assert batch["input_ids"].shape[0] == 4 and batch["pixel_values"].shape[0] == 4
    assert (batch["completion_mask"].sum(1) > 0).all()
    args = DPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, max_steps=5, logging_steps=1,
                     learning_rate=2e-3, use_cpu=True, save_strategy="no", report_to="none", beta=0.5,
                     lr_scheduler_type="constant")
    tr = DPOTrainer(model, args=args, train_dataset=rows, processing_class=proc)
    tr.train()
    hist = [h for h in tr.state.log_history if "rewards/margins" in h]
    assert hist[-1]["rewards/margins"] > hist[0]["rewards/margins"]
    assert hist[-1]["loss"] < hist[0]["loss"]


def test_grpo_trains_vision_language_model(tmp_path):
    import numpy as np

    from trl_b200 import GRPOConfig, GRPOTrainer

    model, proc = _vlm_and_processor()
    rs = np.random.RandomState(3)
    rows = []
    for i in range(8):
        img = (rs.rand(28, 28, 3) * 255).astype("uint8")
        rows.append({"image": img, "prompt": [{"role": "user", "content": "explain the idea"}]})
    seen = {}

    def reward_len(completion_ids, **kw):
        seen["n"] = seen.get("n", 0) + len(completion_ids)
        return [float(sum(c) % 7) for c in completion_ids]

    args = GRPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, num_generations=4, max_completion_length=6,
                      max_steps=2, logging_steps=1, learning_rate=1e-3, use_cpu=True, save_strategy="no",
                      report_to="none", beta=0.04, temperature=1.0)
    tr = GRPOTrainer(model, reward_len, args, train_dataset=rows, processing_class=proc)
    w0 = model.proj1_w.detach().clone()
    tr.train()
    assert seen["n"] >= 8
    logs = [h for h in tr.state.log_history if "reward" in h]
    assert logs and all(np.isfinite(h["loss"]) for h in logs) and "kl" in logs[-1]
    assert not torch.equal(w0, model.proj1_w)  # gradients reach the projector through the image tokens


def test_rloo_runs_with_image_prompts(tmp_path):
    import numpy as np

    from trl_b200 import RLOOConfig, RLOOTrainer

    model, proc = _vlm_and_processor()
    rs = np.random.RandomState(4)
    rows = [{"images": [(rs.rand(28, 28, 3) * 255).astype("uint8")], "prompt": "explain the idea <image>"} for _ in range(4)]
    args = RLOOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, num_generations=2, max_completion_length=5,
                      max_steps=2, logging_steps=1, learning_rate=1e-3, use_cpu=True, save_strategy="no",
                      report_to="none", beta=0.05)
    tr = RLOOTrainer(model, lambda completion_ids, **kw: [float(sum(c) % 5) for c in completion_ids], args,
                     train_dataset=rows, processing_class=proc)
    tr.train()
    logs = [h for h in tr.state.log_history if "reward" in h]
    assert len(logs) == 2 and all(np.isfinite(h["loss"]) for h in logs)


def test_processor_opens_image_files_and_byte_records(tmp_path):
    import io

    import numpy as np
    from PIL import Image

    _, proc = _vlm_and_processor()
    arr = (np.random.RandomState(5).rand(31, 45, 3) * 255).astype("uint8")
    f = tmp_path / "a.png"
    Image.fromarray(arr).save(f)
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    a = proc.preprocess_images([[str(f)], [{"bytes": buf.getvalue(), "path": None}], [arr]])
    assert a.shape == (3, 3, 28, 28)
    assert torch.allclose(a[0], a[1]) and torch.allclose(a[0], a[2], atol=1e-5)


def test_vision_collator_with_a_transformers_processor():
    """The collators are written against the processor call contract, not against VisionProcessor: a genuine
    transformers LlavaProcessor (CLIP image processor + tokenizer + block-aware chat template) gives the same layout."""
    import os

    import numpy as np
    import transformers as tf

    from trl_b200.testing import make_tiny_tokenizer
    from trl_b200.trainer.sft_trainer import DataCollatorForVisionLanguageModeling

    tok = make_tiny_tokenizer()
    tok.add_special_tokens({"additional_special_tokens": ["<image>"]})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "trl_b200", "chat_templates", "llava_training.jinja")) as f:
        tpl = f.read()
    ip = tf.CLIPImageProcessor(size={"shortest_edge": 28}, crop_size={"height": 28, "width": 28})
    proc = tf.LlavaProcessor(image_processor=ip, tokenizer=tok, patch_size=14, vision_feature_select_strategy="default",
                             image_token="<image>", num_additional_image_tokens=1, chat_template=tpl)
    img = (np.random.RandomState(0).rand(40, 30, 3) * 255).astype("uint8")
    ex = [{"images": [img], "messages": [{"role": "user", "content": "what is this"},
                                         {"role": "assistant", "content": "a simple idea"}]},
          {"images": [img, img], "messages": [{"role": "user", "content": "explain"}, {"role": "assistant", "content": "two"}]}]
    out = DataCollatorForVisionLanguageModeling(proc)(ex)
    image_id = tok.convert_tokens_to_ids("<image>")
    assert out["pixel_values"].shape == (3, 3, 28, 28)
    assert (out["input_ids"] == image_id).sum(1).tolist() == [4, 8]
    # the batch trains the native model when the ids agree
    model = VisionLanguageModel(tiny_vlm_arch("tiny-qwen2", image_token_index=image_id))
    loss = model(input_ids=out["input_ids"], attention_mask=out["attention_mask"], pixel_values=out["pixel_values"],
                 labels=out["labels"]).loss
    assert torch.isfinite(loss)


def test_vlm_loads_a_checkpoint_written_by_transformers(tmp_path):
    import transformers as tf

    torch.manual_seed(0)
    vc = tf.CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, image_size=28,
                             patch_size=14, projection_dim=16)
    tc = tf.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=1024, rms_norm_eps=1e-6)
    hf = tf.LlavaForConditionalGeneration(tf.LlavaConfig(vision_config=vc, text_config=tc, image_token_index=5,
                                                         vision_feature_layer=-2)).eval()
    hf.save_pretrained(str(tmp_path))
    from trl_b200.models.hf_io import load_model

    ours = load_model(str(tmp_path)).eval()
    assert isinstance(ours, VisionLanguageModel) and ours.config.image_token_index == 5
    g = torch.Generator().manual_seed(1)
    ids = _ids_with_images(ours.config, [1, 1], 14, g)
    pix = torch.randn(2, 3, 28, 28, generator=g)
    with torch.no_grad():
        a = ours(input_ids=ids, pixel_values=pix).logits
        b = hf(input_ids=ids, pixel_values=pix).logits
    assert torch.allclose(a, b, atol=3e-4, rtol=1e-3), (a - b).abs().max()
