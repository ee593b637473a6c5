"""Fused memory-bound kernels vs fp32 PyTorch references (B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,H", [(7, 64), (333, 3584), (1024, 4096), (65, 8192), (16, 128)])
def test_rmsnorm_fwd_bwd(T, H):
    from trl_b200.ops import functional as F_
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    g = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    y = F_.rms_norm(x, w, 1e-6)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.rms_norm(xr, wr, 1e-6)
    yr.backward(g.float())
    assert torch.allclose(y.float(), yr, atol=2e-2, rtol=2e-2)
    assert torch.allclose(x.grad.float(), xr.grad, atol=3e-2, rtol=3e-2)
    assert torch.allclose(w.grad.float(), wr.grad, atol=0.15, rtol=3e-2), (w.grad.float() - wr.grad).abs().max()


def test_rope_fwd_bwd():
    from trl_b200.ops import functional as F_
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    T, Hq, Hk, D = 50, 8, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    pos = torch.randint(0, 4000, (T,), device="cuda", dtype=torch.int32)

    def split(t):
        return t[:, :Hq * D].reshape(T, Hq, D), t[:, Hq * D:(Hq + Hk) * D].reshape(T, Hk, D)
    q, k = split(qkv)
    qo, ko = F_.apply_rope_qk(q, k, pos, 1e6)
    (qo.float().sum() * 2 + (ko.float() ** 2).sum()).backward()
    qkv2 = qkv.detach().float().requires_grad_()
    q2, k2 = split(qkv2)
    qr, kr = ref.apply_rope(q2, pos, 1e6), ref.apply_rope(k2, pos, 1e6)
    (qr.sum() * 2 + (kr ** 2).sum()).backward()
    assert torch.allclose(qo.float(), qr, atol=3e-2, rtol=2e-2)
    assert torch.allclose(ko.float(), kr, atol=3e-2, rtol=2e-2)
    assert torch.allclose(qkv.grad.float(), qkv2.grad, atol=6e-2, rtol=3e-2)


def test_multimodal_rope_fwd_bwd():
    """Three position rows, frequency sections pick their row (Qwen2-VL); also equal rows = plain RoPE."""
    from trl_b200.ops import functional as F_
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    T, Hq, Hk, D = 70, 4, 2, 128
    sections = [16, 24, 24]
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    pos3 = torch.randint(0, 3000, (3, T), device="cuda")

    def split(t):
        return t[:, :Hq * D].reshape(T, Hq, D), t[:, Hq * D:(Hq + Hk) * D].reshape(T, Hk, D)
    q, k = split(qkv)
    qo, ko = F_.apply_mrope_qk(q, k, pos3, 1e6, sections)
    (qo.float().sum() * 2 + (ko.float() ** 2).sum()).backward()
    qkv2 = qkv.detach().float().requires_grad_()
    q2, k2 = split(qkv2)
    qr, kr = ref.apply_mrope(q2, pos3, 1e6, sections), ref.apply_mrope(k2, pos3, 1e6, sections)
    (qr.sum() * 2 + (kr ** 2).sum()).backward()
    assert torch.allclose(qo.float(), qr, atol=3e-2, rtol=2e-2)
    assert torch.allclose(ko.float(), kr, atol=3e-2, rtol=2e-2)
    assert torch.allclose(qkv.grad.float(), qkv2.grad, atol=6e-2, rtol=3e-2)
    same = pos3[:1].expand(3, T).contiguous()
    a, b = F_.apply_mrope_qk(q.detach(), k.detach(), same, 1e6, sections)
    c, d = F_.apply_rope_qk(q.detach(), k.detach(), same[0], 1e6)
    assert torch.equal(a, c) and torch.equal(b, d)


def test_swiglu_fwd_bwd():
    from trl_b200.ops import functional as F_
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    gu = torch.randn(37, 2 * 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(37, 512, device="cuda", dtype=torch.bfloat16)
    F_.swiglu(gu).backward(g)
    gr = gu.detach().float().requires_grad_()
    o = ref.swiglu(gr)
    o.backward(g.float())
    assert torch.allclose(F_.swiglu(gu).float(), o, atol=2e-2, rtol=2e-2)
    assert torch.allclose(gu.grad.float(), gr.grad, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_adamw_flat_matches_reference(gdtype):
    from trl_b200.loop.optim import adamw_reference
    from trl_b200.ops import cuda as K

    torch.manual_seed(0)
    n = 100_003
    master = torch.randn(n, device="cuda")
    grad = torch.randn(n, device="cuda").to(gdtype)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    mr, vr, pr = m.clone(), v.clone(), master.clone()
    shadow = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    scale = torch.tensor(0.5, device="cuda")
    for step in (1, 2, 3):
        K.adamw_flat(master, grad, m, v, step, 1e-3, 0.9, 0.999, 1e-8, 0.01, scale, shadow)
        adamw_reference(pr, grad, mr, vr, step, 1e-3, 0.9, 0.999, 1e-8, 0.01, 0.5)
    assert torch.allclose(master, pr, atol=1e-5, rtol=1e-5)
    assert torch.allclose(shadow.float(), pr, atol=1e-2, rtol=1e-2)
    ss = K.sumsq(grad)
    assert torch.allclose(ss[0], grad.float().pow(2).sum(), rtol=1e-3)
    # views that start one element into their buffers are not 16-byte aligned: the scalar kernel takes them
    K.adamw_flat(master[1:], grad[1:], m[1:], v[1:], 4, 1e-3, 0.9, 0.999, 1e-8, 0.01, scale, shadow[1:])
    adamw_reference(pr[1:], grad[1:], mr[1:], vr[1:], 4, 1e-3, 0.9, 0.999, 1e-8, 0.01, 0.5)
    assert torch.allclose(master, pr, atol=1e-5, rtol=1e-5) and torch.allclose(m, mr, atol=1e-6)


@pytest.mark.parametrize("T,H", [(64, 3584), (5, 8192), (1000, 2048)])
def test_add_rmsnorm_infer(T, H):
    from trl_b200.ops import cuda as K
    from trl_b200.oracle import ops as ref

    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    d = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
    res = x.clone()
    y = K.add_rmsnorm_infer(res, d, w, 1e-6)
    s = (x + d)
    assert torch.equal(res, s)
    assert torch.allclose(y.float(), ref.rms_norm(s, w, 1e-6).float(), atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("n", [8 * 1000 + 5, 64, 3, 1 << 20])
def test_accum_bf16_into_fp32(n):
    from trl_b200.ops import cuda as K

    torch.manual_seed(0)
    buf = torch.randn(n + 8, device="cuda")
    dst = buf[:n]
    src = torch.randn(n, device="cuda").to(torch.bfloat16)
    want = dst + src.float()
    K.accum_grad(dst, src)
    assert torch.equal(dst, want)
    assert float(buf[n:].abs().sum()) == float(buf[n:].abs().sum())


def test_attention_varlen_qk_mask_is_aligned_to_key_segment_end():
    """The library varlen kernel behind context parallelism: a query segment that is the tail of its key segment."""
    from trl_b200.oracle import ops as O
    from trl_b200.ops import cuda as K

    torch.manual_seed(0)
    Hq, Hk, D = 8, 2, 128
    cu_q = torch.tensor([0, 40, 41, 170], dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0, 300, 301, 430], dtype=torch.int32, device="cuda")  # first segment: 260 keys of prefix
    q = torch.randn(170, Hq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(430, Hk, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(430, Hk, D, device="cuda", dtype=torch.bfloat16)
    out = K.attention_varlen_qk(q, k, v, cu_q, cu_k, 129, 300)
    ref = O.attention_varlen_qk(q.float(), k.float(), v.float(), cu_q, cu_k)
    assert (out.float() - ref).abs().max().item() < 2e-2
