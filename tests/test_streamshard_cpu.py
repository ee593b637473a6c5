"""Streamed full-shard engine, single process: construction from a meta-device model, training step, guards."""
import pytest
import torch

from trl_b200.models.configuration import preset
from trl_b200.models.decoder import CausalLM, SeqCtx
from trl_b200.ops import functional as ops
from trl_b200.parallel.streamshard import StreamShardEngine


def _loss(model, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 1024, (40,), generator=g)
    ctx = SeqCtx.from_lengths([15, 25], ids.device)
    h = model.forward_hidden(ids, ctx)
    s, _, _, n = ops.lm_head_ce(h, model.lm_head_weight, torch.roll(ids, -1))
    return s / n


def test_meta_model_is_initialised_inside_the_slots_and_trains():
    cfg = preset("tiny-qwen2", num_hidden_layers=3)
    engines = []
    for _ in range(2):
        m = CausalLM(cfg, device="meta")
        m.gradient_checkpointing_enable()
        m.train()
        engines.append((m, StreamShardEngine(m, device="cpu", init_seed=3)))
    (m1, e1), (m2, e2) = engines
    assert not any(p.is_meta for p in m1.parameters())
    sd1, sd2 = e1.streamed_hf_state_dict(), e2.streamed_hf_state_dict()
    for k in sd1:  # same seed, same weights (what makes the ranks of a job agree)
        assert torch.equal(sd1[k], sd2[k]), k
    assert torch.all(sd1["model.layers.0.input_layernorm.weight"] == 1)
    assert not torch.equal(sd1["model.layers.0.self_attn.o_proj.weight"], sd1["model.layers.2.self_attn.o_proj.weight"])
    assert abs(sd1["model.layers.1.mlp.down_proj.weight"].std().item() - 0.02) < 0.003
    # layers 0 and 2 share a slot and still keep their own weights through a step
    before = _loss(m1).item()
    for s in range(3):
        e1.zero_grad()
        e1.backward(_loss(m1))
        norm = e1.step(1e-2, 1.0)
        assert torch.isfinite(norm)
    assert _loss(m1).item() < before
    # loading a checkpoint into the slices
    e2.load_weights(e1.streamed_hf_state_dict())
    for k, v in e1.streamed_hf_state_dict().items():
        assert torch.equal(v, e2.streamed_hf_state_dict()[k]), k


def test_backward_refuses_to_run_without_checkpointing():
    m = CausalLM(preset("tiny-qwen2")).train()
    e = StreamShardEngine(m)
    with pytest.raises(RuntimeError, match="checkpointing"):
        e.backward(_loss(m))


def test_frozen_mode_streams_a_reference_model_without_optimizer_state():
    import copy

    torch.manual_seed(0)
    m = CausalLM(preset("tiny-qwen2", num_hidden_layers=3)).eval().requires_grad_(False)
    whole = copy.deepcopy(m)
    e = StreamShardEngine(m, frozen=True)
    assert e.gbuf is None and all(l.exp_avg is None for l in e.layers)
    with torch.no_grad():
        a, b = _loss(m, 3), _loss(whole, 3)
        c = _loss(m, 4)  # a second pass re-gathers the layers that were overwritten in their slots
    assert torch.allclose(a, b, atol=1e-6) and torch.allclose(c, _loss(whole, 4), atol=1e-6)


def test_frozen_meta_copy_starts_equal_to_the_policy():
    """A policy and its frozen reference, both built from meta models with the same seed, hold the same weights."""
    cfg = preset("tiny-qwen2", num_hidden_layers=2)
    pol = CausalLM(cfg, device="meta")
    pol.gradient_checkpointing_enable()
    ref = CausalLM(cfg, device="meta").eval().requires_grad_(False)
    StreamShardEngine(pol, device="cpu", init_seed=5)
    StreamShardEngine(ref, device="cpu", init_seed=5, frozen=True)
    assert not any(p.is_meta for p in ref.parameters()) and not any(p.requires_grad for p in ref.parameters())
    with torch.no_grad():
        assert torch.allclose(_loss(pol.eval(), 1), _loss(ref, 1), atol=1e-6)
