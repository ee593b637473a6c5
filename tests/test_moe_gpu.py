"""Grouped expert GEMM (tcgen05) and the MoE block built on it vs the fp32 expert loop (B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("E,I,H,T,k", [(8, 256, 512, 700, 2), (5, 96, 128, 37, 2), (16, 768, 2048, 1500, 4)])
def test_grouped_gemm_and_moe_forward_backward(E, I, H, T, k):
    from trl_b200.ops import cuda as K
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    dev = "cuda"
    hidden = (torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    gu = (torch.randn(E, 2 * I, H, device=dev) / H ** 0.5).to(torch.bfloat16).requires_grad_(True)
    dw = (torch.randn(E, H, I, device=dev) / I ** 0.5).to(torch.bfloat16).requires_grad_(True)
    logits = torch.randn(T, E, device=dev)
    if E > 2:
        logits[:, 1] = -1e9  # an expert without tokens
    topw, topi = torch.softmax(logits, -1).topk(k, -1)
    topw = (topw / topw.sum(-1, keepdim=True)).requires_grad_(True)

    # plain grouped GEMM against a per-expert loop
    flat = topi.reshape(-1)
    order = torch.argsort(flat, stable=True)
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=dev)
    offsets[1:] = torch.bincount(flat, minlength=E).cumsum(0)
    x_perm = hidden.detach()[order // k]
    got = K.grouped_gemm(x_perm, gu.detach(), offsets, 2 * I)
    offs = offsets.tolist()
    want = torch.cat([x_perm[offs[e]:offs[e + 1]].float() @ gu.detach()[e].float().t() for e in range(E)])
    assert (got.float() - want).abs().max().item() < 0.06 * max(1.0, want.abs().max().item())
    fused = K.grouped_gemm(x_perm, gu.detach(), offsets, I, swiglu=True)
    want_act = torch.nn.functional.silu(want[:, :I]) * want[:, I:]
    assert (fused.float() - want_act).abs().max().item() < 0.06 * max(1.0, want_act.abs().max().item())

    # input gradient form: the forward weight [E, 2I, H] read transposed, rows [R, 2I] -> [R, H]
    d_gu = (torch.randn(x_perm.shape[0], 2 * I, device=dev) * 0.5).to(torch.bfloat16)
    got_dx = K.grouped_gemm(d_gu, gu.detach(), offsets, H, w_transposed=True)
    want_dx = torch.cat([d_gu[offs[e]:offs[e + 1]].float() @ gu.detach()[e].float() for e in range(E)])
    assert (got_dx.float() - want_dx).abs().max().item() < 0.03 * max(1.0, want_dx.abs().max().item())
    # weight gradient: per expert d_gu^T @ x over the expert's rows (any row count, also none)
    got_dw = K.grouped_wgrad(d_gu, x_perm, offsets, E)
    want_dw = torch.stack([d_gu[offs[e]:offs[e + 1]].float().t() @ x_perm[offs[e]:offs[e + 1]].float() for e in range(E)])
    assert (got_dw.float() - want_dw).abs().max().item() < 0.03 * max(1.0, want_dw.abs().max().item())
    if E > 2:
        assert got_dw[1].abs().max().item() == 0.0
    K.check_status(torch.device(dev))

    out = K.moe_experts(hidden, gu, dw, topw, topi)
    out.float().square().sum().backward()
    grads = [t.grad.float().clone() for t in (hidden, gu, dw, topw)]
    for t in (hidden, gu, dw, topw):
        t.grad = None
    h32, g32, d32 = (t.detach().float().requires_grad_(True) for t in (hidden, gu, dw))
    w32 = topw.detach().clone().requires_grad_(True)
    out_ref = ref.moe_experts(h32, g32, d32, w32, topi).float()
    out_ref.square().sum().backward()
    K.check_status(torch.device(dev))
    scale = out_ref.abs().max().item()
    assert (out.float() - out_ref).abs().max().item() < 0.05 * max(1.0, scale)
    for got_g, ref_t in zip(grads, (h32, g32, d32, w32)):
        denom = ref_t.grad.abs().max().item() + 1e-6
        assert (got_g - ref_t.grad).abs().max().item() / denom < 0.08


@pytest.mark.parametrize("N,E,K,masked,dtype", [(1000, 128, 8, False, torch.float32), (77, 8, 2, True, torch.float32),
                                                (5000, 60, 4, True, torch.bfloat16), (3, 512, 8, False, torch.float32)])
def test_moe_aux_loss_kernel_matches_oracle_and_its_gradient(N, E, K, masked, dtype):
    from trl_b200.ops import functional as ops
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    logits = torch.randn(N, E, device="cuda")
    probs = torch.softmax(logits, -1).to(dtype).requires_grad_()
    idx = probs.detach().float().topk(K, -1).indices
    mask = (torch.rand(N, device="cuda") > 0.3).float() if masked else None
    for _ in range(2):  # the scratch accumulator must come back zeroed
        loss = ops.load_balancing_loss(probs, idx, E, K, mask)
        (g,) = torch.autograd.grad(loss, probs)
        p2 = probs.detach().float().requires_grad_()
        want = ref.load_balancing_loss(p2, idx, E, K, mask)
        (g2,) = torch.autograd.grad(want, p2)
        assert abs(float(loss) - float(want)) < 2e-3 * max(1.0, abs(float(want))), (float(loss), float(want))
        assert (g.float() - g2).abs().max().item() < 2e-3 * max(1e-3, g2.abs().max().item()) + 1e-6
