"""Activation offloading: pack / unpack bookkeeping on CPU tensors (streams off) and the checkpoint wrapper whose
saved layer input goes through the hooks.  Behaviours follow tests/test_activation_offloading.py of the reference:
same loss and gradients with and without the context, views and broadcasts restored exactly, parameters and small
tensors left alone, leaked state cleared on entry, the output head exempt."""
import pytest
import torch
import torch.nn as nn

from trl_b200.models.activation_offloading import (NoOpManager, OffloadActivations, get_act_offloading_ctx_manager,
                                                   no_offload, offload_checkpoint, offloading_active)


def _mlp():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(64, 128), nn.GELU(), nn.Linear(128, 64), nn.Tanh(), nn.Linear(64, 8))


def _run(model, x, ctx=None):
    model.zero_grad()
    if ctx is None:
        loss = model(x).pow(2).mean()
    else:
        with ctx:
            loss = model(x).pow(2).mean()
    loss.backward()
    return loss.detach(), [p.grad.clone() for p in model.parameters()]


def test_same_loss_and_gradients_with_offloading_and_everything_is_released():
    model, x = _mlp(), torch.randn(32, 64)
    l0, g0 = _run(model, x)
    ctx = OffloadActivations(use_streams=False, min_offload_size=16, model=model, _offload_cpu_tensors=True)
    for _ in range(2):  # the second pass reuses pooled host buffers
        l1, g1 = _run(model, x, ctx)
        assert torch.equal(l0, l1) and all(torch.equal(a, b) for a, b in zip(g0, g1))
        assert not ctx.tracker and not ctx.fwd_stash and not ctx.live_storage
    assert ctx.stats["offloaded"] > 0 and ctx.stats["restored"] == ctx.stats["offloaded"]


def test_parameters_small_tensors_and_param_views_stay_put():
    model = _mlp()
    ctx = OffloadActivations(use_streams=False, min_offload_size=1024, model=model, _offload_cpu_tensors=True)
    w = model[0].weight
    small, big = torch.randn(8), torch.randn(1024)
    assert not ctx._eligible(w) and not ctx._eligible(w.detach()[:4]) and not ctx._eligible(small)
    assert ctx._eligible(big) and not OffloadActivations(use_streams=False)._eligible(big)  # CPU tensors: test flag only


def test_views_offsets_and_broadcasts_are_restored_exactly():
    ctx = OffloadActivations(use_streams=False, min_offload_size=16, _offload_cpu_tensors=True)
    base = torch.arange(4 * 6 * 8, dtype=torch.float32).reshape(4, 6, 8)
    cases = [base, base[:, 1:3], base.transpose(0, 2), base[2], torch.randn(1, 8).expand(16, 8), base.view(-1)[5:77]]
    with ctx:
        ids = [ctx._pack(t) for t in cases]
    for t, i in zip(cases, ids):
        back = ctx._unpack(i)
        assert back.shape == t.shape and torch.equal(back, t)
        if 0 in t.stride():
            assert back.stride() == t.stride()  # a broadcast is not materialised
    assert not ctx.tracker
    with pytest.raises(ValueError):
        ctx._unpack(10_000)


def test_same_storage_saved_twice_is_copied_once_while_it_is_stashed():
    ctx = OffloadActivations(use_streams=False, min_offload_size=16, _offload_cpu_tensors=True)
    ctx.use_streams, ctx.max_fwd_stash_size = False, 5
    t = torch.randn(256)
    # emulate the stream path's stash (kept until the copy event): the second save finds the storage alive
    a = ctx._pack(t)
    ctx.fwd_stash[a] = (t, None)
    ctx.live_storage[(t.untyped_storage().data_ptr(), t.untyped_storage().nbytes())] = a
    b = ctx._pack(t.view(16, 16))
    assert ctx.tracker[b].kind == "keep" and ctx.stats["offloaded"] == 1
    assert torch.equal(ctx._unpack(b), t.view(16, 16)) and torch.equal(ctx._unpack(a), t)


def test_enter_clears_state_left_by_a_forward_without_backward():
    model, x = _mlp(), torch.randn(16, 64)
    ctx = OffloadActivations(use_streams=False, min_offload_size=16, model=model, _offload_cpu_tensors=True)
    with ctx:
        model(x).sum()  # no backward: entries leak
    assert ctx.tracker
    l0, g0 = _run(model, x)
    l1, g1 = _run(model, x, ctx)
    assert torch.equal(l0, l1) and all(torch.equal(a, b) for a, b in zip(g0, g1)) and not ctx.tracker


def test_noop_manager_and_no_offload_scope():
    ctx = OffloadActivations(use_streams=False, min_offload_size=16, _offload_cpu_tensors=True)
    lin = nn.Linear(64, 64)
    x = torch.randn(32, 64, requires_grad=True)
    assert not offloading_active()
    with ctx:
        assert offloading_active()
        with no_offload():
            y = lin(x).pow(2).sum()
        inside = ctx.stats["offloaded"]
        z = lin(x).pow(2).sum()
    assert inside == 0 and ctx.stats["offloaded"] > 0 and not offloading_active()
    (y + z).backward()
    assert isinstance(no_offload(), type(__import__("contextlib").nullcontext()))
    assert isinstance(NoOpManager(), torch.autograd.graph.saved_tensors_hooks)


def test_offload_checkpoint_matches_plain_backward_and_saves_only_the_layer_input():
    torch.manual_seed(1)
    layers = nn.ModuleList([nn.Sequential(nn.Linear(32, 32), nn.Tanh()) for _ in range(3)])
    x = torch.randn(8, 32)  # no grad on the input: the anchor keeps the graph connected

    def run(use_ckpt, ctx=None):
        layers.zero_grad()
        h = x
        with (ctx if ctx is not None else __import__("contextlib").nullcontext()):
            for l in layers:
                h = offload_checkpoint(l, h) if use_ckpt else l(h)
        loss = h.pow(2).mean()
        loss.backward()
        return loss.detach(), [p.grad.clone() for p in layers.parameters()]

    l0, g0 = run(False)
    ctx = OffloadActivations(use_streams=False, min_offload_size=16, _offload_cpu_tensors=True)
    l1, g1 = run(True, ctx)
    assert torch.allclose(l0, l1) and all(torch.allclose(a, b, atol=1e-6) for a, b in zip(g0, g1))
    assert ctx.stats["offloaded"] == 3  # one saved tensor per checkpointed layer: its input


def test_native_decoder_trains_identically_with_activation_offloading(tmp_path, tiny_tokenizer):
    from trl_b200 import SFTConfig, SFTTrainer
    from trl_b200.testing import make_dataset, make_tiny_model

    def losses(offload, sub):
        torch.manual_seed(0)
        model = make_tiny_model()
        args = SFTConfig(output_dir=str(tmp_path / sub), per_device_train_batch_size=4, max_steps=3, logging_steps=1,
                         learning_rate=1e-3, use_cpu=True, save_strategy="no", report_to="none", seed=3,
                         activation_offloading=offload, gradient_checkpointing=True)
        tr = SFTTrainer(model, args, train_dataset=make_dataset("standard_language_modeling", 24),
                        processing_class=tiny_tokenizer)
        tr.train()
        return [h["loss"] for h in tr.state.log_history if "loss" in h], tr

    a, _ = losses(False, "a")
    b, tr = losses(True, "b")
    assert a == b
    assert isinstance(tr.maybe_activation_offload_context, OffloadActivations)
    assert isinstance(get_act_offloading_ctx_manager(None), OffloadActivations)  # also without a GPU
