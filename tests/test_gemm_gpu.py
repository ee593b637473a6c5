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


@pytest.mark.parametrize("pdl", [False, True])
@pytest.mark.parametrize("B,N,K", [(64, 3584, 18944), (7, 1000, 520), (33, 4608, 3584), (1, 136, 64), (100, 777 * 8, 264),
                                   (128, 3584, 3584)])
def test_decode_gemm_stream_k_and_fp32_add_rmsnorm(B, N, K, pdl):
    from trl_b200.ops import cuda as Kc

    torch.manual_seed(0)
    x = (torch.randn(B, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    y = torch.zeros(B, N, device="cuda")
    was = Kc.set_pdl(pdl)
    try:
        Kc.decode_gemm(x, w, bias, y32=y)
        want = x.float() @ w.float().t() + bias.float()
        assert (y - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())
        Kc.decode_gemm(x, w, y32=y)  # accumulates
        assert (y - (2 * want - bias.float())).abs().max().item() < 4e-2 * max(1.0, want.abs().max().item())
        for ctas in (1, 5, 148):  # any grid gives the same sums
            y2 = torch.zeros(B, N, device="cuda")
            Kc.decode_gemm(x, w, bias, y32=y2, max_ctas=ctas)
            assert (y2 - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item()), ctas
        out = Kc.decode_gemm(x, w, bias)  # bf16 store, whole slab pairs
        assert (out.float() - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())
        wt = Kc.tile_weights(w)  # tile-major copy of the weight
        y3 = torch.zeros(B, N, device="cuda")
        Kc.decode_gemm(x, wt, bias, y32=y3, tiled_shape=(N, K))
        assert (y3 - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())
        ctr = torch.zeros(1, dtype=torch.int32, device="cuda")  # single rank: the arrival counter counts the grid
        y4 = torch.zeros(B, N, device="cuda")
        Kc.decode_gemm(x, w, bias, y32=y4, peers=([], [ctr.data_ptr()], None, None))
        assert int(ctr.item()) == Kc.decode_gemm_ctas(B, N, K) and (y4 - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())
        if N % 4 == 0:
            # the fused all-reduce path with a second local buffer standing in for a peer's accumulator: partial sums
            # meet in the staging buffer, every finished quarter is handed to both buffers once, two launches add up
            y5, y6 = torch.zeros(B, N, device="cuda"), torch.zeros(B, N, device="cuda")
            stage = torch.zeros(B, N, device="cuda")
            slab_ctr = torch.zeros(4 * ((N + 127) // 128), dtype=torch.int32, device="cuda")
            ctrs = torch.zeros(32, dtype=torch.int32, device="cuda")
            for _ in range(2):
                Kc.decode_gemm(x, w, bias, y32=y5, peers=([y6.data_ptr()], [ctrs.data_ptr(), ctrs[16:].data_ptr()], stage, slab_ctr))
            assert ctrs[0].item() == ctrs[16].item() == 2 * Kc.decode_gemm_arrivals(N)
            assert float(stage.abs().max()) == 0.0 and int(slab_ctr.abs().max()) == 0
            for got in (y5, y6):
                assert (got - 2 * want).abs().max().item() < 4e-2 * max(1.0, want.abs().max().item())
        if N % 8 == 0:
            res = torch.randn(B, N, device="cuda").to(torch.bfloat16)
            gamma = torch.randn(N, device="cuda").to(torch.bfloat16)
            r0, d0 = res.clone(), y.clone()
            o = Kc.add_rmsnorm_f32_infer(res, y, gamma, 1e-6)
            s = (r0.float() + d0).to(torch.bfloat16).float()
            ref = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float()
            assert (o.float() - ref).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item())
            assert float(y.abs().max()) == 0.0 and torch.equal(res.float(), s)
        torch.cuda.synchronize()
        Kc.check_status(torch.device("cuda"))
    finally:
        Kc.set_pdl(was)


@pytest.mark.parametrize("B,I,K", [(64, 18944, 3584), (5, 256, 72), (128, 1024, 256), (70, 384, 520)])
def test_decode_gemm_swiglu_epilogue(B, I, K):
    from trl_b200.ops import cuda as Kc

    torch.manual_seed(3)
    x = (torch.randn(B, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    out = Kc.decode_gemm(x, w, swiglu=True)
    g, u = x.float() @ w[:I].float().t(), x.float() @ w[I:].float().t()
    want = torch.nn.functional.silu(g) * u
    torch.cuda.synchronize()
    Kc.check_status(torch.device("cuda"))
    assert (out.float() - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())
    out2 = Kc.decode_gemm(x, Kc.tile_weights(w), swiglu=True, tiled_shape=(2 * I, K))
    torch.cuda.synchronize()
    assert (out2.float() - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("qk_norm,bias,v_t", [(False, True, True), (True, False, True), (False, False, False)])
def test_rope_kv_write_from_fp32_sums_matches_bf16_path(qk_norm, bias, v_t):
    from trl_b200.ops import cuda as Kc

    torch.manual_seed(4)
    B, Hq, Hk, D, bs, nblk = 9, 8, 2, 128, 64 if v_t else 16, 40
    qkv32 = torch.randn(B, (Hq + 2 * Hk) * D, device="cuda")
    b = torch.randn((Hq + 2 * Hk) * D, device="cuda").to(torch.bfloat16) if bias else None
    qn = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16) if qk_norm else None
    kn = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16) if qk_norm else None
    seq_lens = torch.tensor([3, 70, -1, 0, 129, 17, 64, 63, 5], dtype=torch.int32, device="cuda")
    table = torch.randperm(nblk, device="cuda").to(torch.int32)[: B * 4].reshape(B, 4)

    def caches():
        kc = torch.zeros(nblk, bs, Hk, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.zeros((nblk, Hk, D, bs) if v_t else (nblk, bs, Hk, D), device="cuda", dtype=torch.bfloat16)
        return kc, vc, torch.zeros(B, Hq, D, device="cuda", dtype=torch.bfloat16)

    # reference: the bf16 path (bias add, per-head norm in PyTorch, then the bf16 kernel)
    ref = qkv32 + (b.float() if bias else 0)
    ref = ref.to(torch.bfloat16)
    if qk_norm:
        r = ref.view(B, Hq + 2 * Hk, D).float()
        for lo, hi, wt in ((0, Hq, qn), (Hq, Hq + Hk, kn)):
            h = r[:, lo:hi]
            r[:, lo:hi] = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6) * wt.float()).to(torch.bfloat16).float()
        ref = r.view(B, -1).to(torch.bfloat16)
    kc0, vc0, q0 = caches()
    Kc.rope_kv_write(ref, seq_lens, None, table, bs, q0, kc0, vc0, Hq, Hk, D, 1e6, v_transposed=v_t)
    kc1, vc1, q1 = caches()
    acc = qkv32.clone()
    Kc.rope_kv_write_f32(acc, b, qn, kn, 1e-6, seq_lens, None, table, bs, q1, kc1, vc1, Hq, Hk, D, 1e6, v_transposed=v_t)
    torch.cuda.synchronize()
    assert float(acc.abs().max()) == 0.0
    for a_, b_ in ((q0, q1), (kc0, kc1), (vc0, vc1)):
        assert (a_.float() - b_.float()).abs().max().item() < 4e-2


@pytest.mark.parametrize("T,N,K", [(256, 512, 128), (1000, 520, 264), (4096, 3584, 1024), (136, 72, 64)])
def test_linear_forward_dgrad_wgrad_on_the_own_gemm(T, N, K):
    """y = x W^T, dX = dY W and dW = dY^T x on the tcgen05 kernel (the two gradients read W, dY and x as MN-major
    operands, i.e. transposed in place) against fp32 autograd."""
    from trl_b200.ops import cuda as Kc

    torch.manual_seed(0)
    x = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16).requires_grad_()
    b = torch.randn(N, device="cuda").to(torch.bfloat16).requires_grad_()
    g = torch.randn(T, N, device="cuda").to(torch.bfloat16)
    assert Kc.linear_own_ok(x, w)
    y = Kc.LinearFn.apply(x, w, b)
    dx, dw, db = torch.autograd.grad(y, (x, w, b), g)
    torch.cuda.synchronize()
    Kc.check_status()
    xf, wf, bf = (t.detach().float().requires_grad_() for t in (x, w, b))
    yf = xf @ wf.t() + bf
    rx, rw, rb = torch.autograd.grad(yf, (xf, wf, bf), g.float())
    for name, a_, r_ in (("y", y, yf), ("dx", dx, rx), ("dw", dw, rw), ("db", db, rb)):
        err = (a_.float() - r_).abs().max().item()
        assert err <= 1.5e-2 * r_.abs().max().item() + 1e-2, (name, err, r_.abs().max().item())


def test_decoder_trains_with_the_own_linear_gemm():
    """One forward/backward of a small decoder with every plain linear on the own GEMM matches the library GEMM."""
    from trl_b200.models.decoder import SeqCtx
    from trl_b200.ops import functional as ops
    from trl_b200.testing import make_tiny_model

    def run(impl):
        was = ops.set_linear_impl(impl)
        try:
            torch.manual_seed(0)
            model = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device="cuda:0", hidden_size=512, num_attention_heads=4,
                                    num_key_value_heads=2, head_dim=128, intermediate_size=1024, vocab_size=2048,
                                    num_hidden_layers=2)
            model.train()
            flat = torch.randint(2, 2048, (1024,), device="cuda:0", generator=torch.Generator(device="cuda:0").manual_seed(1))
            hidden = model.forward_hidden(flat, SeqCtx.from_lengths([512, 512], torch.device("cuda:0")))
            loss, _, _, n = ops.lm_head_ce(hidden[:-1], model.lm_head_weight, flat[1:])
            (loss / n).backward()
            return float(loss / n), {k: p.grad.float().clone() for k, p in model.named_parameters() if p.grad is not None}
        finally:
            ops.set_linear_impl(was)

    l0, g0 = run("cublas")
    l1, g1 = run("own")
    assert abs(l0 - l1) < 2e-2
    for k in g0:
        assert (g0[k] - g1[k]).abs().max().item() <= 5e-2 * g0[k].abs().max().item() + 1e-3, k
