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
