"""Fused GRPO / DPO loss kernels vs the PyTorch oracle (B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("beta,delta,use_old", [(0.0, None, False), (0.04, None, True), (0.04, 1.5, True)])
def test_grpo_loss_kernel(beta, delta, use_old):
    from trl_b200.ops import cuda as K
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    B, T = 16, 200
    logp = (-torch.rand(B, T, device="cuda") * 3).requires_grad_()
    old = (logp.detach() + 0.3 * torch.randn(B, T, device="cuda")) if use_old else None
    refl = logp.detach() + 0.2 * torch.randn(B, T, device="cuda")
    adv = torch.randn(B, device="cuda")
    mask = (torch.rand(B, T, device="cuda") > 0.3).float()
    row_scale = 1.0 / (mask.sum(-1).clamp(min=1) * B)
    ent = torch.rand(B, T, device="cuda")
    loss, stats = K.grpo_loss(logp, old, refl if beta else None, adv, mask, row_scale, ent, 0.2, 0.25, beta, delta)
    loss.backward()
    lp2 = logp.detach().clone().requires_grad_()
    tok, ratio, kl = ref.grpo_token_loss(lp2, old if use_old else lp2.detach(), refl if beta else None, adv[:, None],
                                         0.2, 0.25, beta, delta)
    rl = ((tok * mask).sum(-1) / mask.sum(-1).clamp(min=1)).mean()
    rl.backward()
    assert torch.allclose(loss, rl, atol=1e-5, rtol=1e-4), (loss, rl)
    assert torch.allclose(logp.grad, lp2.grad, atol=1e-6, rtol=1e-4)
    if beta:
        assert torch.allclose(stats[1] / stats[4], (kl * mask).sum() / mask.sum(), rtol=1e-4)
    assert torch.allclose(stats[7] / stats[4], (ent * mask).sum() / mask.sum(), rtol=1e-4)


def test_dpo_loss_kernel():
    from trl_b200.ops import cuda as K
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    P = 6
    lens = torch.randint(5, 60, (2 * P,))
    cu = torch.zeros(2 * P + 1, dtype=torch.int32)
    cu[1:] = lens.cumsum(0)
    Ttot = int(cu[-1])
    pol = (-torch.rand(Ttot, device="cuda") * 2).requires_grad_()
    rf = -torch.rand(Ttot, device="cuda") * 2
    mask = (torch.rand(Ttot, device="cuda") > 0.4).float()
    loss, out = K.dpo_loss(pol, rf, mask, cu.cuda(), 0.1, 0.0)
    loss.backward()
    p2 = pol.detach().clone().requires_grad_()
    seg = lambda x: torch.stack([(x * mask)[cu[i]:cu[i + 1]].sum() for i in range(2 * P)])
    ps, rs = seg(p2), seg(rf)
    l, rc, rr = ref.dpo_sigmoid_loss(ps[:P], ps[P:], rs[:P], rs[P:], 0.1)
    l.mean().backward()
    assert torch.allclose(loss, l.mean(), atol=1e-6, rtol=1e-5)
    assert torch.allclose(pol.grad, p2.grad, atol=1e-7, rtol=1e-4)
    assert torch.allclose(out[:, 1], rc.detach(), atol=1e-5) and torch.allclose(out[:, 2], rr.detach(), atol=1e-5)
