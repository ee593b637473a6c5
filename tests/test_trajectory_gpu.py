"""Training-invariant test for the GPU kernel path: the same model, data and optimizer run for 50 steps through the
bf16 kernels (tcgen05 attention, fused lm_head loss, RMSNorm / RoPE / SwiGLU kernels, fused AdamW with fp32 master
weights) and through the fp32 PyTorch oracle on the CPU; the loss and gradient-norm series must stay together, judged
like the reference's invariant suite by the largest deviation and by the mean residual
(tests/invariant/test_invariant.py:129-155 there)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _series(model, engine, batches, steps, lr):
    from trl_b200.models.decoder import SeqCtx
    from trl_b200.ops import functional as ops

    dev = model.device
    out = []
    for s in range(steps):
        ids, lens = batches[s % len(batches)]
        ids = ids.to(dev)
        engine.zero_grad()
        ctx = SeqCtx.from_lengths(lens, dev)
        h = model.forward_hidden(ids, ctx)
        labels = torch.roll(ids, -1)
        ends = torch.tensor(lens).cumsum(0) - 1
        labels[ends.to(dev)] = -100  # no target across a document boundary
        loss_sum, _, _, n = ops.lm_head_ce(h, model.lm_head_weight, labels)
        loss = loss_sum / n
        engine.backward(loss)
        gn = engine.step(lr, 1.0)
        out.append((float(loss.detach()), float(gn)))
    return out


@pytest.mark.parametrize("linear", ["cublas", "own"])
def test_fifty_steps_kernel_path_follows_the_fp32_oracle(linear):
    from trl_b200.ops import cuda as K
    from trl_b200.ops import functional as ops
    from trl_b200.parallel.engine import TrainEngine
    from trl_b200.testing import make_tiny_model

    base = make_tiny_model("tiny-qwen2", hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                           intermediate_size=512, num_hidden_layers=2, seed=0)
    g = torch.Generator().manual_seed(7)
    batches = []
    for _ in range(5):  # five packed batches, visited in turn: ten passes over each in fifty steps
        lens = [97, 160, 1, 254]  # odd lengths and a one-token document
        batches.append((torch.randint(0, 1024, (sum(lens),), generator=g), lens))
    m_ref = copy.deepcopy(base)
    ref = _series(m_ref, TrainEngine(m_ref, mode="ddp", weight_decay=0.01), batches, 50, 1e-3)
    m_gpu = copy.deepcopy(base).to(device="cuda", dtype=torch.bfloat16)
    was = ops.set_linear_impl(linear)
    try:
        got = _series(m_gpu, TrainEngine(m_gpu, mode="ddp", weight_decay=0.01), batches, 50, 1e-3)
    finally:
        ops.set_linear_impl(was)
    torch.cuda.synchronize()
    K.check_status(torch.device("cuda"))
    assert ref[-1][0] < ref[0][0] - 0.5 and got[-1][0] < got[0][0] - 0.5  # both learn the five batches
    d_loss = [abs(a[0] - b[0]) for a, b in zip(ref, got)]
    d_gn = [abs(a[1] - b[1]) / max(1.0, a[1]) for a, b in zip(ref, got)]
    mean_loss = abs(sum(a[0] - b[0] for a, b in zip(ref, got))) / len(ref)
    mean_gn = abs(sum((a[1] - b[1]) / max(1.0, a[1]) for a, b in zip(ref, got))) / len(ref)
    # bf16 compute against fp32: a few hundredths on a loss near 7 -> 5, a few percent on the gradient norm
    assert max(d_loss) < 0.08 and mean_loss < 0.03, (max(d_loss), mean_loss, ref[::10], got[::10])
    assert max(d_gn) < 0.12 and mean_gn < 0.04, (max(d_gn), mean_gn, ref[::10], got[::10])
