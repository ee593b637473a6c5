"""tcgen05 GEMM family vs plain PyTorch fp32 references (runs on the B200 box)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (300, 520, 264), (1024, 3584, 3584), (77, 1000, 128)])
def test_gemm_bf16_tn_matches_fp32(M, N, K):
    from trl_b200.ops import cuda as K_

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    out = K_.gemm_bf16_tn(a, b, bias)
    K_.check_status()
    ref = a.float() @ b.float().t() + bias.float()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)


@pytest.mark.parametrize("M,V,K,temp", [(64, 128, 32 * 8, 1.0), (200, 1000, 64, 0.7), (1024, 4096, 256, 1.0), (513, 152064, 128, 1.0)])
def test_lmhead_forward_matches_oracle(M, V, K, temp):
    from trl_b200.ops import cuda as K_
    from trl_b200.oracle import ops as ref

    torch.manual_seed(1)
    h = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(V, K, device="cuda") * 0.1).to(torch.bfloat16)
    y = torch.randint(0, V, (M,), device="cuda")
    logp, ent, lse, amax = K_.lmhead_forward(h, w, y, 1.0 / temp, True, True)
    K_.check_status()
    rlogp, rent = ref.lm_head_logprobs(h, w, y, temp)
    assert torch.allclose(logp, rlogp, atol=2e-3, rtol=1e-3), (logp - rlogp).abs().max()
    assert torch.allclose(ent, rent, atol=2e-3, rtol=1e-3), (ent - rent).abs().max()
    logits = (h.float() @ w.float().t()) / temp
    assert (amax.long() == logits.argmax(-1)).float().mean() > 0.999


def test_lmhead_backward_matches_autograd():
    from trl_b200.ops import cuda as K_
    from trl_b200.oracle import ops as ref

    torch.manual_seed(2)
    M, V, K = 300, 2048, 128
    h = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, K, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    y = torch.randint(0, V, (M,), device="cuda")
    g = torch.randn(M, device="cuda")
    logp, _ = K_.lm_head_logprobs(h, w, y, 0.9, True)
    (logp * g).sum().backward()
    K_.check_status()
    h2, w2 = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    rl, _ = ref.lm_head_logprobs(h2, w2, y, 0.9)
    (rl * g).sum().backward()
    assert torch.allclose(h.grad.float(), h2.grad, atol=3e-2, rtol=3e-2), (h.grad.float() - h2.grad).abs().max()
    assert torch.allclose(w.grad.float(), w2.grad, atol=3e-2, rtol=3e-2), (w.grad.float() - w2.grad).abs().max()


@pytest.mark.parametrize("B,N,K", [(64, 3584, 18944), (7, 1000, 520), (33, 4608, 3584)])
def test_smallm_splitk_gemm_and_fp32_add_rmsnorm(B, N, K):
    from trl_b200.ops import cuda as Kc

    torch.manual_seed(0)
    x = (torch.randn(B, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    y = torch.zeros(B, N, device="cuda")
    Kc.smallm_gemm_accumulate(x, w, y, bias=bias)
    want = x.float() @ w.float().t() + bias.float()
    assert (y - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())
    Kc.smallm_gemm_accumulate(x, w, y)  # accumulates
    assert (y - (2 * want - bias.float())).abs().max().item() < 4e-2 * max(1.0, want.abs().max().item())
    if N % 8 == 0:
        res = torch.randn(B, N, device="cuda").to(torch.bfloat16)
        gamma = torch.randn(N, device="cuda").to(torch.bfloat16)
        r0, d0 = res.clone(), y.clone()
        out = Kc.add_rmsnorm_f32_infer(res, y, gamma, 1e-6)
        s = (r0.float() + d0).to(torch.bfloat16).float()
        ref = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float()
        assert (out.float() - ref).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item())
        assert float(y.abs().max()) == 0.0 and torch.equal(res.float(), s)
    torch.cuda.synchronize()
    Kc.check_status(torch.device("cuda"))
