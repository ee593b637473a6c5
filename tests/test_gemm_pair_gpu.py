"""CTA-pair GEMM (tcgen05 cta_group::2) vs plain PyTorch fp32 references (runs on the B200 box)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 256, 512), (512, 768, 256), (300, 520, 264), (1024, 3584, 3584),
                                   (77, 1000, 128), (4096, 4608, 1024)])
def test_pair_gemm_forward_matches_fp32(M, N, K):
    from trl_b200.ops import cuda as K_

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    out = K_.gemm_pair_bf16(a, b, bias)
    torch.cuda.synchronize()
    K_.check_status()
    ref = a.float() @ b.float().t() + bias.float()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)


@pytest.mark.parametrize("T,N,K", [(512, 512, 256), (1000, 776, 328), (2048, 4608, 3584)])
def test_pair_gemm_dgrad_and_wgrad_forms(T, N, K):
    """dX = dY W (W read MN-major) and dW = dY^T x (both operands MN-major), nothing transposed in memory."""
    from trl_b200.ops import cuda as K_

    torch.manual_seed(1)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    dy = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    dx = K_.gemm_pair_bf16(dy, w, b_mn=True)
    dw = K_.gemm_pair_bf16(dy, x, a_mn=True, b_mn=True)
    torch.cuda.synchronize()
    K_.check_status()
    rdx, rdw = dy.float() @ w.float(), dy.float().t() @ x.float()
    assert (dx.float() - rdx).abs().max().item() <= 1e-2 * rdx.abs().max().item() + 1e-2
    assert (dw.float() - rdw).abs().max().item() <= 1e-2 * rdw.abs().max().item() + 1e-2
