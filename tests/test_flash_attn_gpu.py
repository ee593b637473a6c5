"""Varlen attention on tcgen05 vs the fp32 oracle (dense masked softmax): document boundaries, lengths that are not
multiples of the tile, length-1 documents, grouped-query heads, sliding window, end-aligned masks."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(lens, Hq, Hk, seed=0, strided=False):
    torch.manual_seed(seed)
    T = sum(lens)
    if strided:  # views into one fused projection, as the decoder produces them
        qkv = torch.randn(T, (Hq + 2 * Hk) * 128, device="cuda").to(torch.bfloat16)
        q = qkv[:, : Hq * 128].view(T, Hq, 128)
        k = qkv[:, Hq * 128:(Hq + Hk) * 128].view(T, Hk, 128)
        v = qkv[:, (Hq + Hk) * 128:].view(T, Hk, 128)
    else:
        q = torch.randn(T, Hq, 128, device="cuda").to(torch.bfloat16)
        k = torch.randn(T, Hk, 128, device="cuda").to(torch.bfloat16)
        v = torch.randn(T, Hk, 128, device="cuda").to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    return q, k, v, cu


@pytest.mark.parametrize("lens,Hq,Hk,window,strided", [
    ([128], 2, 2, None, False), ([256, 128], 4, 2, None, False), ([1, 130, 7, 300, 1, 129], 4, 1, None, True),
    ([700, 45], 14, 2, None, True), ([513, 64, 255], 2, 1, 100, False), ([1000], 2, 2, 257, True),
])
def test_fa_forward_matches_oracle(lens, Hq, Hk, window, strided):
    from trl_b200.ops import cuda as K
    from trl_b200.oracle import ops as ref

    q, k, v, cu = _mk(lens, Hq, Hk, strided=strided)
    out, lse = K.fa_varlen_fwd(q, k, v, cu, cu, causal=True, window=window)
    torch.cuda.synchronize()
    K.check_status()
    want = ref.attention_varlen(q.float(), k.float(), v.float(), cu, causal=True, window=window)
    err = (out.float() - want.float()).abs().max().item()
    assert err < 2e-2, err
    # log-sum-exp against the dense computation of one head
    T = q.shape[0]
    doc = torch.bucketize(torch.arange(T, device="cuda"), cu[1:].long(), right=True)
    idx = torch.arange(T, device="cuda")
    mask = (doc[:, None] == doc[None, :]) & (idx[:, None] >= idx[None, :])
    if window:
        mask &= idx[:, None] - idx[None, :] < window
    s = (q[:, 0].float() @ k[:, 0].float().t()) / 128 ** 0.5
    want_lse = torch.logsumexp(s.masked_fill(~mask, float("-inf")), -1)
    assert (lse[0] - want_lse).abs().max().item() < 2e-2


@pytest.mark.parametrize("causal", [True, False])
def test_fa_forward_when_the_reference_maximum_moves(causal):
    """Scores that keep growing along the keys (by far more than 2^8 from tile to tile) force the rows to move their
    reference maximum and rescale the output accumulated in TMEM many times; the result and the log-sum-exp must
    still match the dense fp32 computation."""
    from trl_b200.ops import cuda as K
    from trl_b200.oracle import ops as ref

    torch.manual_seed(3)
    lens, Hq, Hk = [640, 385], 4, 2
    T = sum(lens)
    q = torch.randn(T, Hq, 128, device="cuda")
    k = torch.randn(T, Hk, 128, device="cuda")
    ramp = torch.linspace(0.0, 8.0, T, device="cuda")  # later keys score higher for every query
    k = k + ramp[:, None, None]  # along the all-ones direction ...
    q = q + 1.0                  # ... which every query has a component of: score += ramp * (128 + noise) / sqrt(128)
    q, k = q.to(torch.bfloat16), k.to(torch.bfloat16)
    v = torch.randn(T, Hk, 128, device="cuda").to(torch.bfloat16)
    cu = torch.tensor([0, 640, 1025], dtype=torch.int32, device="cuda")
    out, lse = K.fa_varlen_fwd(q, k, v, cu, cu, causal=causal)
    torch.cuda.synchronize()
    K.check_status()
    want = ref.attention_varlen(q.float(), k.float(), v.float(), cu, causal=causal)
    assert (out.float() - want.float()).abs().max().item() < 3e-2
    idx = torch.arange(T, device="cuda")
    doc = torch.bucketize(idx, cu[1:].long(), right=True)
    mask = doc[:, None] == doc[None, :]
    if causal:
        mask &= idx[:, None] >= idx[None, :]
    sc = (q[:, 1].float() @ k[:, 0].float().t()) / 128 ** 0.5
    want_lse = torch.logsumexp(sc.masked_fill(~mask, float("-inf")), -1)
    spread = (sc.masked_fill(~mask, float("-inf")).max(-1).values - sc.masked_fill(~mask, float("inf")).min(-1).values)
    assert spread.max().item() > 40  # the ramp really spans many factors of 2^8
    assert (lse[1] - want_lse).abs().max().item() < 5e-2 * max(1.0, want_lse.abs().max().item() / 20)


def test_fa_forward_noncausal_and_end_aligned_segments():
    from trl_b200.ops import cuda as K
    from trl_b200.oracle import ops as ref

    torch.manual_seed(1)
    lq, lk = [40, 128, 3], [200, 128, 131]
    Tq, Tk, Hq, Hk = sum(lq), sum(lk), 4, 2
    q = torch.randn(Tq, Hq, 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(Tk, Hk, 128, device="cuda").to(torch.bfloat16)
    v = torch.randn(Tk, Hk, 128, device="cuda").to(torch.bfloat16)
    cq = torch.tensor([0, 40, 168, 171], dtype=torch.int32, device="cuda")
    ck = torch.tensor([0, 200, 328, 459], dtype=torch.int32, device="cuda")
    out, _ = K.fa_varlen_fwd(q, k, v, cq, ck, causal=True)
    want = ref.attention_varlen_qk(q.float(), k.float(), v.float(), cq, ck)
    torch.cuda.synchronize()
    K.check_status()
    assert (out.float() - want.float()).abs().max().item() < 2e-2
    cu = torch.tensor([0, 150, 300], dtype=torch.int32, device="cuda")
    q2 = torch.randn(300, 2, 128, device="cuda").to(torch.bfloat16)
    k2, v2 = k[:300, :2].contiguous(), v[:300, :2].contiguous()
    out2, _ = K.fa_varlen_fwd(q2, k2, v2, cu, cu, causal=False)
    want2 = ref.attention_varlen(q2.float(), k2.float(), v2.float(), cu, causal=False)
    torch.cuda.synchronize()
    assert (out2.float() - want2.float()).abs().max().item() < 2e-2


@pytest.mark.parametrize("lens,Hq,Hk,window,strided", [
    ([128], 2, 2, None, False), ([192, 64], 4, 2, None, False), ([1, 130, 7, 300, 1, 129], 4, 1, None, True),
    ([700, 45], 14, 2, None, True), ([513, 64, 255], 2, 1, 100, False),
])
def test_fa_backward_matches_autograd_of_the_oracle(lens, Hq, Hk, window, strided):
    from trl_b200.ops import cuda as K
    from trl_b200.oracle import ops as ref

    q, k, v, cu = _mk(lens, Hq, Hk, seed=2, strided=strided)
    q, k, v = (t.detach().clone().requires_grad_() if not strided else t.detach().requires_grad_() for t in (q, k, v))
    out = K.attention_varlen(q, k, v, cu, max(lens), True, window)
    g = torch.randn_like(out)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), g)
    torch.cuda.synchronize()
    K.check_status()
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    want = ref.attention_varlen(qf, kf, vf, cu, causal=True, window=window)
    rq, rk, rv = torch.autograd.grad(want, (qf, kf, vf), g.float())
    for name, a, b in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        err = (a.float() - b).abs().max().item()
        assert err < 3e-2 * max(1.0, b.abs().max().item()), (name, err, b.abs().max().item())


def test_fa_backward_end_aligned_segments():
    from trl_b200.ops import cuda as K
    from trl_b200.oracle import ops as ref

    torch.manual_seed(5)
    Hq, Hk = 4, 2
    cq = torch.tensor([0, 40, 168, 171], dtype=torch.int32, device="cuda")
    ck = torch.tensor([0, 200, 328, 459], dtype=torch.int32, device="cuda")
    q = torch.randn(171, Hq, 128, device="cuda").to(torch.bfloat16).requires_grad_()
    k = torch.randn(459, Hk, 128, device="cuda").to(torch.bfloat16).requires_grad_()
    v = torch.randn(459, Hk, 128, device="cuda").to(torch.bfloat16).requires_grad_()
    out = K.attention_varlen_qk(q, k, v, cq, ck, 128, 200)
    g = torch.randn_like(out)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), g)
    torch.cuda.synchronize()
    K.check_status()
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    rq, rk, rv = torch.autograd.grad(ref.attention_varlen_qk(qf, kf, vf, cq, ck), (qf, kf, vf), g.float())
    for a, b in ((dq, rq), (dk, rk), (dv, rv)):
        assert (a.float() - b).abs().max().item() < 3e-2 * max(1.0, b.abs().max().item())


def test_checkpointed_layers_reuse_the_attention_output_in_their_recompute():
    """With activation checkpointing the recompute of a layer takes the attention output of the first pass instead of
    launching the forward kernel again: same gradients, one attention forward per layer instead of two."""
    from trl_b200.models.decoder import SeqCtx
    from trl_b200.ops import cuda as K
    from trl_b200.ops import functional as ops
    from trl_b200.testing import make_tiny_model

    model = make_tiny_model("tiny-qwen2", dtype=torch.bfloat16, device="cuda", hidden_size=256, num_attention_heads=2,
                            num_key_value_heads=1, head_dim=128, intermediate_size=512, num_hidden_layers=3, seed=0)
    model.gradient_checkpointing_enable()
    model.train()
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 1024, (400,), generator=g).cuda()
    lens = [150, 250]

    def run():
        for p in model.parameters():
            p.grad = None
        before = K.LAUNCHES[0]
        h = model.forward_hidden(ids, SeqCtx.from_lengths(lens, ids.device))
        loss_sum, _, _, n = ops.lm_head_ce(h, model.lm_head_weight, torch.roll(ids, -1))
        (loss_sum / n).backward()
        torch.cuda.synchronize()
        return K.LAUNCHES[0] - before, {k: p.grad.clone() for k, p in model.named_parameters()}

    was = K.AttnKeep.enabled
    try:
        K.AttnKeep.enabled = True
        n_keep, g_keep = run()
        assert not K.AttnKeep.store  # every kept output was taken back by its recompute
        K.AttnKeep.enabled = False
        n_plain, g_plain = run()
    finally:
        K.AttnKeep.enabled = was
    assert n_plain - n_keep == 3, (n_plain, n_keep)  # one forward attention launch less per layer
    for k in g_keep:
        assert torch.equal(g_keep[k], g_plain[k]), k
    K.check_status()
