"""Qwen2-VL-style model (dynamic-resolution tower, 2 x 2 patch merger, multimodal RoPE) against transformers'
implementation, its checkpoints, processor and trainers."""
import numpy as np
import pytest
import torch

from trl_b200.models.vision_qwen import Qwen2VLModel, patchify, rope_index, tiny_qwen2_vl_arch


def _rows_with_images(tokens_per_image, rows_of, gen):
    """Padded ids/mask: row r holds the images ``rows_of[r]`` (indices), each as start + placeholders + end."""
    rows = []
    for imgs in rows_of:
        ids = []
        for k in imgs:
            ids += torch.randint(10, 1000, (4,), generator=gen).tolist() + [3] + [5] * tokens_per_image[k] + [4]
        rows.append(ids + torch.randint(10, 1000, (5,), generator=gen).tolist())
    L = max(map(len, rows))
    ids = torch.zeros(len(rows), L, dtype=torch.long)
    mask = torch.zeros(len(rows), L, dtype=torch.long)
    for i, r in enumerate(rows):
        ids[i, :len(r)] = torch.tensor(r)
        mask[i, :len(r)] = 1
    return ids, mask


def _hf_model(arch):
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    d = arch.to_hf_dict()
    text = {k: v for k, v in d["text_config"].items() if k not in ("architectures", "mrope_section", "rope_parameters",
                                                                    "torch_dtype")}
    hc = Qwen2VLConfig(text_config=text, vision_config=d["vision_config"], image_token_id=arch.image_token_id,
                       video_token_id=arch.video_token_id, vision_start_token_id=arch.vision_start_token_id,
                       vision_end_token_id=arch.vision_end_token_id)
    return Qwen2VLForConditionalGeneration(hc).eval().float()


def test_logits_match_transformers_qwen2_vl():
    torch.manual_seed(0)
    arch = tiny_qwen2_vl_arch()
    hf = _hf_model(arch)
    m = Qwen2VLModel(arch).eval()
    m.load_hf_state_dict(hf.state_dict())
    g = torch.Generator().manual_seed(1)
    # images of two different sizes: grids 4 x 6 and 2 x 4 patches
    pv_a, grid_a = patchify(torch.randn(2, 3, 56, 84, generator=g), arch.vision)
    pv_b, grid_b = patchify(torch.randn(1, 3, 28, 56, generator=g), arch.vision)
    pv, grid = torch.cat([pv_a, pv_b]), torch.cat([grid_a, grid_b])
    per_image = (grid.prod(-1) // 4).tolist()
    ids, mask = _rows_with_images(per_image, [[0, 1], [2]], g)
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=mask, pixel_values=pv, image_grid_thw=grid,
                 mm_token_type_ids=(ids == arch.image_token_id).long()).logits
        out = m(input_ids=ids, attention_mask=mask, pixel_values=pv, image_grid_thw=grid).logits
    assert (ref - out).abs()[mask.bool()].max() < 2e-5
    # text only: the three position rows coincide and the model is an ordinary decoder
    t_ids = torch.randint(10, 1000, (2, 9), generator=g)
    with torch.no_grad():
        assert (hf(input_ids=t_ids).logits - m(input_ids=t_ids).logits).abs().max() < 2e-5


def test_rope_index_text_and_image_positions():
    arch = tiny_qwen2_vl_arch()
    # one sequence: 2 text tokens, an image of 1 x 4 x 6 patches (2 x 3 merged tokens), 2 text tokens; then a text sequence
    ids = torch.tensor([11, 3] + [5] * 6 + [4, 12] + [13, 14, 15])
    cu = torch.tensor([0, 10, 13], dtype=torch.int32)
    pos = rope_index(ids, cu, torch.tensor([[1, 4, 6]]), arch)
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6                       # one frame
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3]            # rows
    assert pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]            # columns
    assert pos[:, 8:10].tolist() == [[5, 6]] * 3                 # text resumes after the larger side (3 columns)
    assert pos[:, 10:].tolist() == [[0, 1, 2]] * 3               # the next sequence starts from zero
    with pytest.raises(ValueError):
        rope_index(torch.tensor([5, 5, 5]), torch.tensor([0, 3]), torch.tensor([[1, 4, 6]]), arch)


def test_checkpoint_round_trip_load_model_and_gradients(tmp_path):
    from trl_b200.models.hf_io import load_model

    torch.manual_seed(0)
    arch = tiny_qwen2_vl_arch()
    m = Qwen2VLModel(arch)
    m.save_pretrained(str(tmp_path))
    re = load_model(str(tmp_path))
    assert isinstance(re, Qwen2VLModel) and re.config.text.extra["mrope_section"] == [2, 3, 3]
    for (n, a), (_, b) in zip(m.named_parameters(), re.named_parameters()):
        assert torch.equal(a, b), n
    pv, grid = patchify(torch.randn(1, 3, 28, 28), arch.vision)
    ids = torch.tensor([[11, 3, 5, 4, 12, 13]])
    out = m(input_ids=ids, pixel_values=pv, image_grid_thw=grid, labels=ids)
    out.loss.backward()
    assert m.visual.patch_w.grad.abs().sum() > 0 and m.visual.merge2_w.grad.abs().sum() > 0
    with pytest.raises(ValueError):  # 4 merged features for one placeholder
        m(input_ids=ids, pixel_values=torch.cat([pv] * 4), image_grid_thw=torch.tensor([[1, 4, 4]]))


def test_loads_a_checkpoint_written_by_transformers(tmp_path):
    torch.manual_seed(0)
    arch = tiny_qwen2_vl_arch()
    hf = _hf_model(arch)
    hf.save_pretrained(str(tmp_path))
    m = Qwen2VLModel.from_pretrained(str(tmp_path)).eval()
    ids = torch.randint(10, 1000, (1, 7))
    with torch.no_grad():
        assert (hf(input_ids=ids).logits - m(input_ids=ids).logits).abs().max() < 2e-5


def _model_and_processor():
    from trl_b200.models.vision_processing import DynamicResolutionProcessor
    from trl_b200.testing import make_tiny_tokenizer

    tok = make_tiny_tokenizer()
    proc = DynamicResolutionProcessor(tok, min_pixels=28 * 28, max_pixels=56 * 56)
    arch = tiny_qwen2_vl_arch()
    arch.image_token_id = proc.image_token_id
    arch.text.vocab_size = max(arch.text.vocab_size, len(tok))
    torch.manual_seed(0)
    model = Qwen2VLModel(arch)
    assert DynamicResolutionProcessor.for_model(tok, model).patch_size == 14
    return model, proc


def test_dynamic_resolution_processor(tmp_path):
    from trl_b200.models.vision_processing import DynamicResolutionProcessor

    model, proc = _model_and_processor()
    assert proc.target_size(28, 28) == (28, 28)
    assert proc.target_size(30, 50) == (28, 56)
    H, W = proc.target_size(400, 200)          # scaled into the pixel budget, aspect kept, sides on the 28 grid
    assert H * W <= 56 * 56 and H % 28 == 0 and W % 28 == 0 and H > W
    assert proc.target_size(10, 10) == (28, 28)
    rs = np.random.RandomState(0)
    imgs = [(rs.rand(30, 50, 3) * 255).astype("uint8"), (rs.rand(28, 28, 3) * 255).astype("uint8")]
    enc = proc(images=[[imgs[0]], [imgs[1]]], text=["look <image> here", "<image>"], padding=True, return_tensors="pt")
    assert enc["image_grid_thw"].tolist() == [[1, 2, 4], [1, 2, 2]]
    assert enc["pixel_values"].shape == (12, 3 * 2 * 14 * 14)
    assert (enc["input_ids"] == proc.image_token_id).sum(1).tolist() == [2, 1]
    out = model(input_ids=enc["input_ids"], attention_mask=enc["attention_mask"], pixel_values=enc["pixel_values"],
                image_grid_thw=enc["image_grid_thw"])
    assert torch.isfinite(out.logits).all()
    proc.save_pretrained(str(tmp_path))
    re = DynamicResolutionProcessor.from_pretrained(str(tmp_path))
    assert (re.max_pixels, re.min_pixels, re.image_token_id) == (proc.max_pixels, proc.min_pixels, proc.image_token_id)
    with pytest.raises(ValueError):
        proc(images=[imgs], text=["one placeholder <image>"])


def _day_night_rows(n, seed, sizes=((28, 28), (28, 56))):
    rs = np.random.RandomState(seed)
    rows = []
    for i in range(n):
        bright = i % 2
        h, w = sizes[(i // 2) % len(sizes)]
        img = (rs.rand(h, w, 3) * 60 + (160 if bright else 10)).astype("uint8")
        rows.append((img, bright))
    return rows


def test_sft_trains_qwen2_vl(tmp_path):
    from trl_b200 import SFTConfig, SFTTrainer

    model, proc = _model_and_processor()
    rows = [{"images": [img], "messages": [{"role": "user", "content": "is it day or night"},
                                           {"role": "assistant", "content": "day" if b else "night"}]}
            for img, b in _day_night_rows(8, 1)]
    args = SFTConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, max_steps=6, logging_steps=1,
                     learning_rate=3e-3, use_cpu=True, save_strategy="no", report_to="none", max_length=None,
                     lr_scheduler_type="constant")
    tr = SFTTrainer(model, args, train_dataset=rows, processing_class=proc)
    w0 = model.visual.patch_w.detach().clone()
    tr.train()
    losses = [h["loss"] for h in tr.state.log_history if "loss" in h]
    assert losses[-1] < losses[0]
    assert not torch.equal(w0, model.visual.patch_w)
    tr.save_model(str(tmp_path / "final"))
    re = Qwen2VLModel.from_pretrained(str(tmp_path / "final"))
    assert torch.equal(re.visual.merge2_w, model.visual.merge2_w)


def test_dpo_trains_qwen2_vl(tmp_path):
    from trl_b200 import DPOConfig, DPOTrainer

    model, proc = _model_and_processor()
    rows = []
    for img, b in _day_night_rows(8, 2):
        good, bad = ("day", "night") if b else ("night", "day")
        rows.append({"images": [img], "prompt": [{"role": "user", "content": "is it day or night"}],
                     "chosen": [{"role": "assistant", "content": good}],
                     "rejected": [{"role": "assistant", "content": bad}]})
    args = DPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, max_steps=5, logging_steps=1,
                     learning_rate=2e-3, use_cpu=True, save_strategy="no", report_to="none", beta=0.5,
                     lr_scheduler_type="constant")
    tr = DPOTrainer(model, args=args, train_dataset=rows, processing_class=proc)
    tr.train()
    hist = [h for h in tr.state.log_history if "rewards/margins" in h]
    assert hist[-1]["rewards/margins"] > hist[0]["rewards/margins"]


def test_grpo_trains_qwen2_vl(tmp_path):
    from trl_b200 import GRPOConfig, GRPOTrainer

    model, proc = _model_and_processor()
    rows = [{"image": img, "prompt": [{"role": "user", "content": "explain the idea"}]} for img, _ in _day_night_rows(8, 3)]
    args = GRPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, num_generations=4, max_completion_length=6,
                      max_steps=2, logging_steps=1, learning_rate=1e-3, use_cpu=True, save_strategy="no",
                      report_to="none", beta=0.04, temperature=1.0)
    tr = GRPOTrainer(model, lambda completion_ids, **kw: [float(sum(c) % 7) for c in completion_ids], args,
                     train_dataset=rows, processing_class=proc)
    w0 = model.visual.merge2_w.detach().clone()
    tr.train()
    logs = [h for h in tr.state.log_history if "reward" in h]
    assert logs and all(np.isfinite(h["loss"]) for h in logs) and "kl" in logs[-1]
    assert not torch.equal(w0, model.visual.merge2_w)


def test_vision_entries_split_merge_and_compare():
    from trl_b200.models.vision import (merge_vision_entries, same_vision_entry, split_vision_batch,
                                        vision_entry_numel)

    # fixed-resolution towers: one tensor [n_images, C, S, S] per example
    pv = torch.arange(3 * 2 * 2 * 2, dtype=torch.float32).view(3, 2, 2, 2)
    per = split_vision_batch({"pixel_values": pv}, [2, 0, 1])
    assert [vision_entry_numel(e) for e in per] == [16, 0, 8]
    kw = merge_vision_entries(per, "cpu")
    assert set(kw) == {"pixel_values"} and torch.equal(kw["pixel_values"], pv)
    assert same_vision_entry(per[0], per[0].clone()) and not same_vision_entry(per[0], per[2])
    assert merge_vision_entries([None, per[1]], "cpu") == {"pixel_values": None}
    # flat patches + grids: example 0 owns images of 4 and 8 patches, example 1 none, example 2 one of 4
    grid = torch.tensor([[1, 2, 2], [1, 2, 4], [1, 2, 2]])
    patches = torch.arange(16 * 3, dtype=torch.float32).view(16, 3)
    per = split_vision_batch({"pixel_values": patches, "image_grid_thw": grid}, [2, 0, 1])
    assert per[1] is None and per[0][0].shape == (12, 3) and per[2][0].shape == (4, 3)
    assert per[0][1].tolist() == [[1, 2, 2], [1, 2, 4]]
    kw = merge_vision_entries([per[2], None, per[0]], "cpu")   # any order of sequences inside a packed batch
    assert torch.equal(kw["pixel_values"], torch.cat([patches[12:], patches[:12]]))
    assert kw["image_grid_thw"].tolist() == [[1, 2, 2], [1, 2, 2], [1, 2, 4]]
    assert same_vision_entry(per[0], (per[0][0].clone(), per[0][1].clone()))
    assert not same_vision_entry(per[0], per[2]) and not same_vision_entry(per[0], pv) and not same_vision_entry(None, per[0])
    assert split_vision_batch({}, [1, 1]) == [None, None]


def test_mrope_with_equal_rows_is_plain_rope_and_sections_pick_their_row():
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    x = torch.randn(7, 3, 16)
    pos = torch.arange(7)
    same = ref.apply_mrope(x, pos[None].expand(3, 7), 10000.0, [2, 3, 3])
    assert torch.equal(same, ref.apply_rope(x, pos, 10000.0))
    # only the height row differs: the frequencies of the temporal and width sections do not move
    pos3 = torch.stack([pos, pos + 5, pos])
    out = ref.apply_mrope(x, pos3, 10000.0, [2, 3, 3])
    half = 8
    keep = [0, 1, 5, 6, 7]        # temporal (2) and width (last 3) frequency slots
    moved = [2, 3, 4]             # height section
    for f in keep:
        assert torch.equal(out[..., f], same[..., f]) and torch.equal(out[..., half + f], same[..., half + f])
    assert any(not torch.equal(out[..., f], same[..., f]) for f in moved)
