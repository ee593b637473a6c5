"""Pure-function specifications (literal vectors taken from the behaviour the reference documents)."""
import math

import pytest
import torch

from trl_b200.oracle import ops as ref
from trl_b200.ops import functional as F_
from trl_b200.trainer.utils import (RepeatSampler, entropy_from_logits, flush_left, nanmax, nanmin, nanstd, pad,
                                    selective_log_softmax, shuffle_sequence_dict, split_tensor_dict,
                                    compute_flops_per_token, hash_module)


def test_pad_right_left_multiple():
    a, b = torch.tensor([1, 2, 3]), torch.tensor([4, 5])
    assert pad([a, b], 0).tolist() == [[1, 2, 3], [4, 5, 0]]
    assert pad([a, b], 0, "left").tolist() == [[1, 2, 3], [0, 4, 5]]
    assert pad([a, b], 9, "right", pad_to_multiple_of=4).tolist() == [[1, 2, 3, 9], [4, 5, 9, 9]]
    x = pad([torch.ones(2, 2), torch.ones(1, 3)], -1)
    assert x.shape == (2, 2, 3) and x[1, 1, 0] == -1


def test_flush_left():
    mask = torch.tensor([[0, 0, 1, 1, 1], [0, 1, 1, 0, 0]])
    t = torch.tensor([[0, 0, 2, 3, 4], [0, 5, 6, 0, 0]])
    m2, t2 = flush_left(mask, t)
    assert m2.tolist() == [[1, 1, 1], [1, 1, 0]] and t2.tolist() == [[2, 3, 4], [5, 6, 0]]


def test_repeat_sampler_order():
    s = RepeatSampler(list("abcdefg"), mini_repeat_count=2, batch_size=3, repeat_count=2, shuffle=False)
    out = list(s)
    assert out == [0, 0, 1, 1, 2, 2] * 2 + [3, 3, 4, 4, 5, 5] * 2  # index 6: incomplete chunk dropped
    assert len(s) == len(out)
    a = list(RepeatSampler(range(10), 1, 5, 1, seed=3))
    b = list(RepeatSampler(range(10), 1, 5, 1, seed=3))
    assert a == b and sorted(a) == list(range(10))


def test_selective_log_softmax_and_entropy():
    torch.manual_seed(0)
    logits = torch.randn(3, 5, 11)
    idx = torch.randint(0, 11, (3, 5))
    want = torch.log_softmax(logits, -1).gather(-1, idx[..., None]).squeeze(-1)
    assert torch.allclose(selective_log_softmax(logits, idx), want, atol=1e-6)
    assert torch.allclose(selective_log_softmax(logits.bfloat16(), idx).float(), want, atol=5e-2)
    k = torch.randint(0, 11, (3, 5, 2))
    assert selective_log_softmax(logits, k).shape == (3, 5, 2)
    lp = torch.log_softmax(logits, -1)
    assert torch.allclose(entropy_from_logits(logits, chunk_size=4), -(lp.exp() * lp).sum(-1), atol=1e-6)


def test_nan_helpers():
    t = torch.tensor([1.0, 2.0, float("nan"), 4.0])
    assert torch.isclose(nanstd(t), torch.tensor([1.0, 2.0, 4.0]).std())
    assert nanmin(t) == 1.0 and nanmax(t) == 4.0
    assert torch.isnan(nanstd(torch.tensor([float("nan"), 3.0])))
    g = torch.tensor([[1.0, 3.0], [float("nan"), 2.0]])
    out = nanstd(g, dim=1)
    assert torch.isclose(out[0], torch.tensor(math.sqrt(2.0))) and torch.isnan(out[1])


def test_split_and_shuffle_tensor_dict():
    d = {"a": torch.arange(12).reshape(6, 2), "b": torch.arange(6), "s": torch.tensor(3.0), "n": None,
         "l": list("uvwxyz")}
    parts = split_tensor_dict(d, 3)
    assert len(parts) == 3 and parts[1]["a"].tolist() == [[4, 5], [6, 7]] and parts[2]["l"] == ["y", "z"]
    assert parts[0]["s"] == 3.0 and parts[0]["n"] is None
    sh = shuffle_sequence_dict(d)
    perm = sh["b"].tolist()
    assert sorted(perm) == list(range(6)) and sh["a"][:, 0].tolist() == [2 * i for i in perm]
    assert sh["l"] == [d["l"][i] for i in perm]


@pytest.mark.parametrize("temp", [1.0, 0.7])
def test_chunked_logprob_forward_backward_vs_naive(temp):
    torch.manual_seed(0)
    N, H, V = 64, 32, 128
    h = torch.randn(N, H, requires_grad=True)
    w = torch.randn(V, H, requires_grad=True)
    y = torch.randint(0, V, (N,))
    lp, ent = F_.lm_head_logprobs(h, w, y, temp, chunk_tokens=16)
    g = torch.randn(N)
    (lp * g).sum().backward()
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    logits = (h2 @ w2.t()) / temp
    lp2 = torch.log_softmax(logits, -1).gather(-1, y[:, None]).squeeze(-1)
    (lp2 * g).sum().backward()
    p = torch.softmax(logits, -1)
    assert torch.allclose(lp, lp2, atol=1e-5) and torch.allclose(ent, -(p * torch.log(p)).sum(-1).detach(), atol=1e-4)
    assert torch.allclose(h.grad, h2.grad, atol=1e-5) and torch.allclose(w.grad, w2.grad, atol=1e-5)


def test_lm_head_ce_matches_cross_entropy_and_zero_valid():
    torch.manual_seed(0)
    h = torch.randn(20, 16, requires_grad=True)
    w = torch.randn(50, 16, requires_grad=True)
    y = torch.randint(0, 50, (20,))
    y[::3] = -100
    loss_sum, correct, ent_sum, n = F_.lm_head_ce(h, w, y)
    want = torch.nn.functional.cross_entropy(h @ w.t(), y, ignore_index=-100, reduction="sum")
    assert torch.allclose(loss_sum, want, atol=1e-5) and int(n) == int((y != -100).sum())
    z, c, e, n0 = F_.lm_head_ce(h, w, torch.full((20,), -100))
    assert float(z) == 0.0 and int(n0) == 0
    z.backward()  # the graph stays connected so every rank still runs backward
    assert h.grad is not None and float(h.grad.abs().sum()) == 0.0


def test_grpo_token_loss_reference_properties():
    lp = torch.tensor([[-1.0, -2.0]])
    loss, ratio, kl = ref.grpo_token_loss(lp, lp.clone(), lp - 0.5, torch.tensor([[2.0]]), 0.2, 0.2, 0.1)
    assert torch.allclose(ratio, torch.ones_like(ratio))
    assert torch.allclose(kl, torch.exp(torch.tensor(-0.5)) + 0.5 - 1)
    assert torch.allclose(loss, -2.0 + 0.1 * kl)


def test_flops_and_hash():
    from trl_b200.models.configuration import preset
    from trl_b200.models.decoder import CausalLM

    f = compute_flops_per_token(preset("qwen2.5-7b"), 1280)
    assert 4.0e10 < f < 6.0e10  # ~6 * 7.6e9 parameters
    m = CausalLM(preset("tiny-qwen2"))
    h1 = hash_module(m)
    with torch.no_grad():
        m.norm.add_(1)
    assert hash_module(m) != h1


def test_plumbing_modules(tmp_path):
    import trl_b200
    from trl_b200 import import_utils
    from trl_b200.cli.commands import CommandContext, TrainingCommand
    from trl_b200.distributed import DistributedBackend
    from trl_b200.models.utils import _ForwardRedirection
    from trl_b200.trainer.utils import generate_model_card

    assert import_utils.is_pydantic_available() and not import_utils.is_unsloth_available()
    assert CommandContext(["sft", "--x", "1"]).argv_after("sft") == ["--x", "1"]
    assert TrainingCommand("dpo").name == "dpo"
    be = DistributedBackend(None)
    assert not be.is_zero3
    with be.gather_params():
        pass
    text = generate_model_card(base_model="org/base", model_name="m", dataset_name="org/ds", trainer_name="DPO",
                               paper_title="Direct Preference Optimization", paper_id="2305.18290", tags=["dpo"])
    assert "org/base" in text and "2305.18290" in text and "- dpo" in text

    class Inner(torch.nn.Module):
        def forward(self, x):
            return x + 1

        def other(self, x):
            return x * 10

    class Wrapper(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m, self.calls = m, 0

        def forward(self, *a, **k):
            self.calls += 1
            return self.m(*a, **k)
    inner = Inner()
    w = Wrapper(inner)
    assert float(_ForwardRedirection()(w, inner, inner.other, torch.tensor(2.0))) == 20.0 and w.calls == 1
    assert float(inner(torch.tensor(2.0))) == 3.0
    assert trl_b200.__version__


# ---- streaming repetition, callable names, sampler variants -----------------------------------------------------------
@pytest.mark.parametrize("mini,bs,rep", [(1, 1, 1), (2, 3, 4), (3, 2, 2), (2, 2, 3)])
def test_repeat_iterable_dataset_follows_the_unshuffled_sampler(mini, bs, rep):
    from trl_b200.trainer.utils import RepeatSampler, repeat_iterable_dataset

    n = 12
    want = list(RepeatSampler(list(range(n)), mini_repeat_count=mini, batch_size=bs, repeat_count=rep, shuffle=False))
    got = [r["x"] for r in repeat_iterable_dataset(({"x": i} for i in range(n)), mini, bs, rep)]
    assert got == want


def test_repeat_iterable_dataset_defaults_tail_columns_and_independent_copies():
    from trl_b200.trainer.utils import repeat_iterable_dataset

    assert [r["x"] for r in repeat_iterable_dataset([{"x": i} for i in range(4)], mini_repeat_count=2)] == [0, 0, 1, 1, 2, 2, 3, 3]
    # seven rows in chunks of two: the seventh cannot fill a chunk and is dropped
    assert [r["x"] for r in repeat_iterable_dataset([{"x": i} for i in range(7)], 1, batch_size=2)] == [0, 1, 2, 3, 4, 5]
    rows = list(repeat_iterable_dataset([{"x": 0, "answer": "0"}, {"x": 1, "answer": "1"}], 2))
    assert rows == [{"x": 0, "answer": "0"}, {"x": 0, "answer": "0"}, {"x": 1, "answer": "1"}, {"x": 1, "answer": "1"}]
    a, b = list(repeat_iterable_dataset([{"prompt": [{"content": "hi"}]}], 2))
    a["prompt"][-1]["content"] += " there"  # editing one repeat must not leak into the other
    assert a is not b and b["prompt"][-1]["content"] == "hi"


def test_repeat_iterable_dataset_forwards_set_epoch_to_the_source():
    from trl_b200.trainer.utils import repeat_iterable_dataset

    class Shuffled:
        def __init__(self):
            self.epoch = 0

        def set_epoch(self, e):
            self.epoch = e

        def __iter__(self):
            g = torch.Generator().manual_seed(42 + self.epoch)
            return iter({"x": int(i)} for i in torch.randperm(8, generator=g))

    rep = repeat_iterable_dataset(Shuffled(), 1, batch_size=8)
    rep.set_epoch(0)
    e0 = [r["x"] for r in rep]
    rep.set_epoch(1)
    e1 = [r["x"] for r in rep]
    assert sorted(e0) == sorted(e1) == list(range(8)) and e0 != e1


def test_get_callable_name_for_functions_partials_instances_and_lambdas():
    import functools

    from trl_b200.trainer.utils import get_callable_name

    def reward(x, scale=1.0):
        return x

    class Scorer:
        def __call__(self, x):
            return x

    assert get_callable_name(reward) == "reward"
    assert get_callable_name(functools.partial(reward, scale=2.0)) == "reward"
    assert get_callable_name(functools.partial(functools.partial(reward, scale=2.0), 1)) == "reward"
    assert get_callable_name(Scorer()) == "Scorer"
    assert get_callable_name(lambda x: x) == "<lambda>"


def test_repeat_sampler_shapes_of_the_schedule():
    from trl_b200.trainer.utils import RepeatSampler

    data = ["a", "b", "c", "d", "e", "f", "g"]
    # every index exactly `mini_repeat_count` times when nothing is dropped
    out = list(RepeatSampler(data, mini_repeat_count=2, seed=0))
    assert len(out) == 14 and all(out[i] == out[i + 1] for i in range(0, 14, 2)) and sorted(set(out)) == list(range(7))
    assert list(RepeatSampler(data, mini_repeat_count=2, shuffle=False)) == [0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6]
    # chunks of three, the seventh item has no chunk
    out = list(RepeatSampler(data, mini_repeat_count=1, batch_size=3, shuffle=False))
    assert out == [0, 1, 2, 3, 4, 5]
    # 7 items, pairs of repeats, chunks of 3, every chunk 4 times: 2 chunks x 4 x 3 x 2
    out = list(RepeatSampler(data, mini_repeat_count=2, batch_size=3, repeat_count=4, shuffle=False))
    assert len(out) == 48 and out[:6] == [0, 0, 1, 1, 2, 2] and out[6:12] == out[:6] and out[24:30] == [3, 3, 4, 4, 5, 5]
    assert len(RepeatSampler(data, mini_repeat_count=2, batch_size=3, repeat_count=4)) == 48
    # the same seed gives the same permutation, and each epoch draws a new one
    s1, s2 = RepeatSampler(data, 1, seed=5), RepeatSampler(data, 1, seed=5)
    assert list(s1) == list(s2) and list(s1) != list(RepeatSampler(data, 1, seed=5))


def test_pad_variants():
    from trl_b200.trainer.utils import pad

    x, y = torch.tensor([1, 2, 3]), torch.tensor([4, 5])
    assert pad([x, y], padding_value=0, padding_side="left").tolist() == [[1, 2, 3], [0, 4, 5]]
    assert pad([x, y], padding_value=0, padding_side="right").tolist() == [[1, 2, 3], [4, 5, 0]]
    a, b = torch.tensor([[1, 2], [3, 4]]), torch.tensor([[5, 6]])
    assert pad([a, b], padding_value=0, padding_side="left").tolist() == [[[1, 2], [3, 4]], [[0, 0], [5, 6]]]
    assert pad([a, b], padding_value=0, padding_side="right").tolist() == [[[1, 2], [3, 4]], [[5, 6], [0, 0]]]
    assert pad([x, y], padding_value=0, pad_to_multiple_of=4).tolist() == [[1, 2, 3, 0], [4, 5, 0, 0]]
    assert pad([x, y], padding_value=0, padding_side="left", pad_to_multiple_of=4).tolist() == [[0, 1, 2, 3], [0, 0, 4, 5]]
    assert pad([torch.tensor([1, 2, 3, 4]), y], padding_value=0, pad_to_multiple_of=4).shape == (2, 4)  # already a multiple


def test_nanstd_and_hash_module_details():
    from trl_b200.trainer.utils import hash_module, nanstd

    t = torch.tensor([1.0, 2.0, 3.0, float("nan")])
    assert abs(float(nanstd(t)) - 1.0) < 1e-6
    m = torch.tensor([[1.0, 3.0], [float("nan"), 4.0], [5.0, float("nan")]])
    assert nanstd(m, dim=0, keepdim=True).shape == (1, 2)
    assert torch.isnan(nanstd(torch.tensor([float("nan"), float("nan")])))
    a, b = torch.nn.Linear(4, 3), torch.nn.Linear(4, 3)
    b.load_state_dict(a.state_dict())
    assert hash_module(a) == hash_module(b)
    with torch.no_grad():
        b.weight[0, 0] += 1e-3
    assert hash_module(a) != hash_module(b)
    assert hash_module(torch.nn.Linear(4, 3).half()) != hash_module(a)


def test_entropy_and_selective_log_softmax_in_chunks_and_dtypes():
    from trl_b200.oracle.ops import entropy_from_logits, selective_log_softmax

    g = torch.Generator().manual_seed(0)
    for shape in [(7, 33), (2, 5, 33)]:
        logits = torch.randn(*shape, generator=g)
        lp = torch.log_softmax(logits, -1)
        want = -(lp.exp() * lp).sum(-1)
        for chunk in (1, 3, 128):
            assert torch.allclose(entropy_from_logits(logits, chunk_size=chunk), want, atol=1e-5)
        idx = torch.randint(0, 33, shape[:-1], generator=g)
        assert torch.allclose(selective_log_softmax(logits, idx), lp.gather(-1, idx[..., None])[..., 0], atol=1e-5)
        multi = torch.randint(0, 33, shape[:-1] + (4,), generator=g)
        assert torch.allclose(selective_log_softmax(logits, multi), lp.gather(-1, multi), atol=1e-5)
        got16 = selective_log_softmax(logits.to(torch.bfloat16), idx)
        assert got16.dtype == torch.bfloat16 and (got16.float() - lp.gather(-1, idx[..., None])[..., 0]).abs().max() < 0.1


def test_small_compat_helpers():
    import asyncio

    from trl_b200.trainer import utils as U

    rows = [{"a": {"aa": None, "ab": 1}, "b": "my_string", "c": [{"x": None, "y": 2}, 3]}]
    assert U.remove_none_values(rows) == [{"a": {"ab": 1}, "b": "my_string", "c": [{"y": 2}, 3]}]
    with pytest.raises(TypeError):
        U.remove_none_values("text")
    assert U.identity(5) == 5 and U.get_config_model_id(object()) == ""
    t, loop, ready = U.start_event_loop_in_daemon("helper-loop")
    assert ready.wait(5) and t.daemon and t.name == "helper-loop"

    async def twice(x):
        return 2 * x

    assert asyncio.run_coroutine_threadsafe(twice(21), loop).result(5) == 42
    U.shutdown_event_loop_in_daemon(t, loop)
    assert not t.is_alive()
    U.shutdown_event_loop_in_daemon(None, None)  # no-op
    assert U.get_comet_experiment_url() is None and U.get_trackio_space_url() is None
    assert callable(U.selective_log_softmax) and callable(U.patch_chunked_lm_head) and callable(U.ensure_master_addr_port)


def test_split_and_unsplit_pixel_values_for_the_three_vision_layouts():
    from trl_b200.trainer.utils import split_pixel_values_by_grid, unsplit_pixel_values_by_grid

    # patches + grids: samples with 1, 0 and 2 images
    grid = torch.tensor([[1, 2, 2], [1, 2, 4], [1, 4, 2]])
    pv = torch.arange(20 * 3, dtype=torch.float32).view(20, 3)
    batch = {"pixel_values": pv, "image_grid_thw": grid, "num_images": [1, 0, 2], "input_ids": torch.zeros(3, 4)}
    sp = split_pixel_values_by_grid(batch)
    assert [t.shape[0] for t in sp["pixel_values"]] == [4, 0, 16]
    assert [t.tolist() for t in sp["image_grid_thw"]] == [[[1, 2, 2]], [], [[1, 2, 4], [1, 4, 2]]]
    assert sp["input_ids"] is batch["input_ids"]
    back = unsplit_pixel_values_by_grid(sp)
    assert torch.equal(back["pixel_values"], pv) and torch.equal(back["image_grid_thw"], grid)
    with pytest.raises(ValueError):
        split_pixel_values_by_grid({**batch, "pixel_values": pv[:-1]})
    # one row per image, positions travel with it
    b2 = {"pixel_values": torch.randn(3, 5, 7), "image_position_ids": torch.arange(3 * 4).view(3, 4), "num_images": [2, 1]}
    s2 = split_pixel_values_by_grid(b2)
    assert [t.shape[0] for t in s2["pixel_values"]] == [2, 1] and s2["image_position_ids"][1].tolist() == [[8, 9, 10, 11]]
    assert torch.equal(unsplit_pixel_values_by_grid(s2)["image_position_ids"], b2["image_position_ids"])
    # tiles: split by num_tiles, mask and shapes alongside
    b3 = {"pixel_values": torch.randn(5, 6), "pixel_attention_mask": torch.ones(5, 6), "spatial_shapes": torch.ones(5, 2),
          "num_tiles": [3, 2], "num_images": [1, 1]}
    s3 = split_pixel_values_by_grid(b3)
    assert [t.shape[0] for t in s3["pixel_values"]] == [3, 2] and [t.shape[0] for t in s3["spatial_shapes"]] == [3, 2]
    assert unsplit_pixel_values_by_grid(s3)["pixel_attention_mask"].shape == (5, 6)
    # nothing to split
    assert split_pixel_values_by_grid({"input_ids": 1}) == {"input_ids": 1}
    plain = {"pixel_values": torch.zeros(2, 3), "num_images": [1, 1]}
    assert split_pixel_values_by_grid(plain) is plain


def test_flops_per_token_and_mfu_properties():
    """Properties the reference tests for its MFU helpers (tests/test_utils.py:1462-1541), on native configurations."""
    import copy

    from trl_b200.models.configuration import preset
    from trl_b200.trainer.utils import adjusted_mfu, compute_mfu

    cfg = preset("tiny-qwen3")
    f8, f16, f32 = (compute_flops_per_token(cfg, n) for n in (8192, 16384, 32768))
    assert f32 - f16 == 2 * (f16 - f8)                      # only the attention scores depend on the length
    tied, untied = copy.deepcopy(cfg), copy.deepcopy(cfg)
    tied.tie_word_embeddings, untied.tie_word_embeddings = True, False
    assert compute_flops_per_token(untied, 16384) - compute_flops_per_token(tied, 16384) == 3 * 2 * cfg.vocab_size * cfg.hidden_size
    moe = preset("tiny-qwen3-moe")
    lo, hi = copy.deepcopy(moe), copy.deepcopy(moe)
    lo.num_experts_per_tok, hi.num_experts_per_tok = 1, 2
    per_expert = 2 * 3 * moe.hidden_size * moe.moe_intermediate_size
    assert compute_flops_per_token(hi, 16384) - compute_flops_per_token(lo, 16384) == 3 * moe.num_hidden_layers * per_expert
    # utilisation: 100 % when the job's tokens per second are exactly peak * devices / flops per token
    flops, peak, world = 100e9, 989.5e12, 8
    assert compute_mfu(flops, peak * world / flops, world, peak_flops_per_device=peak) == pytest.approx(100.0)
    # causal correction: multiplicative, consistent with the two formulas, stronger for longer sequences
    full = compute_flops_per_token(moe, 16384)
    hd = moe.head_dim or moe.hidden_size // moe.num_attention_heads
    half = moe.num_hidden_layers * 3 * 2 * moe.num_attention_heads * hd * 16384
    assert adjusted_mfu(100.0, moe, 16384) == pytest.approx(100.0 * (full - half) / full)
    assert adjusted_mfu(100.0, moe, 16384) == pytest.approx(2 * adjusted_mfu(50.0, moe, 16384))
    assert adjusted_mfu(100.0, moe, 4096) > adjusted_mfu(100.0, moe, 16384) > adjusted_mfu(100.0, moe, 65536)


@pytest.mark.parametrize("temperature", [1.0, 0.7])
def test_patched_chunked_lm_head_with_and_without_completion_mask(temperature):
    """With a completion mask the patched forward equals the unmasked one on completion positions and is zero on prompt
    positions; the lm_head gradient of a masked sum is the same either way; values equal a plain log-softmax
    (tests/test_utils.py:1321-1460 on the native decoder)."""
    from trl_b200.ops.chunked_lm_head import patch_chunked_lm_head
    from trl_b200.testing import make_tiny_model

    torch.manual_seed(42)
    B, S = 4, 16
    plain = make_tiny_model(seed=0)
    model = patch_chunked_lm_head(make_tiny_model(seed=0), chunk_size=32, temperature=temperature)
    ids = torch.randint(5, 1000, (B, S))
    am = torch.ones(B, S, dtype=torch.long)
    cm = torch.zeros(B, S)
    cm[:, S // 2:] = 1.0
    full = model(input_ids=ids, attention_mask=am)
    masked = model(input_ids=ids, attention_mask=am, completion_mask=cm)
    sm = cm[:, 1:].bool()
    assert torch.allclose(masked["log_probs"][sm], full["log_probs"][sm], atol=1e-5)
    assert torch.allclose(masked["entropy"][sm], full["entropy"][sm], atol=1e-5)
    assert (masked["log_probs"][~sm] == 0).all() and (masked["entropy"][~sm] == 0).all()
    # against explicit logits
    with torch.no_grad():
        logits = plain(input_ids=ids, attention_mask=am).logits[:, :-1].float() / temperature
    lsm = torch.log_softmax(logits, -1)
    want_lp = lsm.gather(-1, ids[:, 1:, None])[..., 0]
    want_ent = -(lsm.exp() * lsm).sum(-1)
    assert torch.allclose(full["log_probs"], want_lp, atol=1e-4) and torch.allclose(full["entropy"], want_ent, atol=1e-4)
    # gradients of a masked sum agree
    head = "lm_head"
    (full["log_probs"] * cm[:, 1:]).sum().backward()
    g_full = dict(model.named_parameters())[head].grad.clone()
    model.zero_grad()
    out2 = model(input_ids=ids, attention_mask=am, completion_mask=cm)
    (out2["log_probs"] * cm[:, 1:]).sum().backward()
    assert torch.allclose(dict(model.named_parameters())[head].grad, g_full, atol=1e-5)
    # padding on the right is excluded like a prompt position
    am2 = am.clone()
    am2[0, -3:] = 0
    out3 = model(input_ids=ids, attention_mask=am2, completion_mask=cm)
    assert (out3["log_probs"][0, -3:] == 0).all() and torch.allclose(out3["log_probs"][1:], masked["log_probs"][1:], atol=1e-5)


def test_print_prompt_completions_sample_tables(capsys):
    """Literal tables of the reference's tests (tests/test_utils.py:632-866): plain strings, extra columns after the
    advantage, chat messages with the role on its own line and reasoning before the answer, a random sub-sample."""
    import textwrap

    from trl_b200.trainer.utils import print_prompt_completions_sample

    rewards = {"Correctness": [0.123, 0.456], "Format": [0.789, 0.101]}
    print_prompt_completions_sample(["The sky is", "The sun is"], [" blue.", " in the sky."], rewards, [0.987, 0.654], 42)
    assert capsys.readouterr().out == textwrap.dedent("""\
        ╭──────────────────────────── Step 42 ─────────────────────────────╮
        │ ┏━━━━━━━━━━━━┳━━━━━━━━━━━━━━┳━━━━━━━━━━━━━┳━━━━━━━━┳━━━━━━━━━━━┓ │
        │ ┃ Prompt     ┃ Completion   ┃ Correctness ┃ Format ┃ Advantage ┃ │
        │ ┡━━━━━━━━━━━━╇━━━━━━━━━━━━━━╇━━━━━━━━━━━━━╇━━━━━━━━╇━━━━━━━━━━━┩ │
        │ │ The sky is │  blue.       │        0.12 │   0.79 │      0.99 │ │
        │ ├────────────┼──────────────┼─────────────┼────────┼───────────┤ │
        │ │ The sun is │  in the sky. │        0.46 │   0.10 │      0.65 │ │
        │ └────────────┴──────────────┴─────────────┴────────┴───────────┘ │
        ╰──────────────────────────────────────────────────────────────────╯
        """)
    print_prompt_completions_sample(["The sky is", "The sun is"], [" blue.", " in the sky."], rewards, [0.987, 0.654], 42,
                                    extra={"source": ["dataset_A", "dataset_B"]})
    assert capsys.readouterr().out == textwrap.dedent("""\
        ╭────────────────────────────────── Step 42 ───────────────────────────────────╮
        │ ┏━━━━━━━━━━━━┳━━━━━━━━━━━━━━┳━━━━━━━━━━━━━┳━━━━━━━━┳━━━━━━━━━━━┳━━━━━━━━━━━┓ │
        │ ┃ Prompt     ┃ Completion   ┃ Correctness ┃ Format ┃ Advantage ┃ source    ┃ │
        │ ┡━━━━━━━━━━━━╇━━━━━━━━━━━━━━╇━━━━━━━━━━━━━╇━━━━━━━━╇━━━━━━━━━━━╇━━━━━━━━━━━┩ │
        │ │ The sky is │  blue.       │        0.12 │   0.79 │      0.99 │ dataset_A │ │
        │ ├────────────┼──────────────┼─────────────┼────────┼───────────┼───────────┤ │
        │ │ The sun is │  in the sky. │        0.46 │   0.10 │      0.65 │ dataset_B │ │
        │ └────────────┴──────────────┴─────────────┴────────┴───────────┴───────────┘ │
        ╰──────────────────────────────────────────────────────────────────────────────╯
        """)
    prompts = [[{"role": "user", "content": "What color is the sky?"}]]
    for key in ("reasoning_content", "thinking"):
        completions = [[{"role": "assistant", key: "I think it is blue.", "content": "It is blue."}]]
        print_prompt_completions_sample(prompts, completions, {"Score": [0.5]}, [0.9], 1)
        assert capsys.readouterr().out == textwrap.dedent("""\
            ╭─────────────────────────────── Step 1 ───────────────────────────────╮
            │ ┏━━━━━━━━━━━━━━━━━━━━━━━━┳━━━━━━━━━━━━━━━━━━━━━┳━━━━━━━┳━━━━━━━━━━━┓ │
            │ ┃ Prompt                 ┃ Completion          ┃ Score ┃ Advantage ┃ │
            │ ┡━━━━━━━━━━━━━━━━━━━━━━━━╇━━━━━━━━━━━━━━━━━━━━━╇━━━━━━━╇━━━━━━━━━━━┩ │
            │ │ USER                   │ ASSISTANT           │  0.50 │      0.90 │ │
            │ │ What color is the sky? │ I think it is blue. │       │           │ │
            │ │                        │ It is blue.         │       │           │ │
            │ └────────────────────────┴─────────────────────┴───────┴───────────┘ │
            ╰──────────────────────────────────────────────────────────────────────╯
            """)
    # tool messages show as name(args); a sub-sample shows one of the rows
    print_prompt_completions_sample([[{"role": "user", "content": "Paris?"}]],
                                    [[{"role": "tool", "name": "get_temperature", "args": {"location": "Paris"}}]],
                                    {"Score": [0.5]}, [0.9], 1)
    out = capsys.readouterr().out
    assert "TOOL" in out and "get_temperature(" in out
    print_prompt_completions_sample(["A", "B"], ["1", "2"], {"Score": [0.1, 0.2]}, [0.3, 0.4], 10, num_samples=1)
    out = capsys.readouterr().out
    assert ("│ A      │ 1 " in out) != ("│ B      │ 2 " in out)


def test_model_card_fields_and_missing_values():
    """The assertions of the reference's model-card tests (tests/test_utils.py:334-381)."""
    from trl_b200.trainer.utils import generate_model_card

    text = str(generate_model_card(
        base_model="username/my_base_model", model_name="my_model", hub_model_id="username/my_hub_model",
        dataset_name="username/my_dataset", tags=["trl", "trainer-tag"], wandb_url="https://wandb.ai/username/project_id/runs/abcd1234",
        trackio_url="https://huggingface.co/spaces/username/space_id",
        comet_url="https://www.comet.com/username/project_id/experiment_id", trainer_name="My Trainer",
        trainer_citation="@article{my_trainer, ...}", paper_title="My Paper", paper_id="1234.56789"))
    for piece in ("[username/my_base_model](https://huggingface.co/username/my_base_model)", "my_model",
                  'pipeline("text-generation", model="username/my_hub_model", device="cuda")', "datasets: username/my_dataset",
                  "](https://wandb.ai/username/project_id/runs/abcd1234)", "](https://huggingface.co/spaces/username/space_id)",
                  "](https://www.comet.com/username/project_id/experiment_id", "My Trainer",
                  "```bibtex\n@article{my_trainer, ...}\n```", "[My Paper](https://huggingface.co/papers/1234.56789)",
                  "- trainer-tag"):
        assert piece in text, piece
    bare = str(generate_model_card(base_model=None, model_name="my_model", hub_model_id="username/my_hub_model", dataset_name=None,
                                   tags=[], wandb_url=None, trackio_url=None, comet_url=None, trainer_name="My Trainer",
                                   trainer_citation=None, paper_title=None, paper_id=None))
    assert "my_model" in bare and "My Trainer" in bare and "wandb" not in bare and "None" not in bare
    assert 'pipeline("text-generation", model="username/my_hub_model", device="cuda")' in bare
