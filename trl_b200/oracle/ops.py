"""Pure-PyTorch reference implementations of every hot op.

These are the numerical oracles for the sm_100a kernels and also the execution
path on CPU (fp32, gloo).  All functions are differentiable through autograd and
do their arithmetic in fp32 regardless of the input dtype.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * weight.float()).to(x.dtype)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, dtype=torch.float32):
    """cos/sin tables [T, head_dim/2] for integer ``positions`` [T]."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half RoPE on ``x`` [T, H, D] (HF Llama/Qwen convention)."""
    d = x.shape[-1]
    cos, sin = rope_cos_sin(positions, d, theta)
    xf = x.float()
    x1, x2 = xf[..., : d // 2], xf[..., d // 2:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def apply_mrope(x: torch.Tensor, positions3: torch.Tensor, theta: float, sections) -> torch.Tensor:
    """Multimodal rotary embedding on ``x`` [T, H, D]: ``positions3`` [3, T] holds a temporal, a height and a width
    position per token; the D/2 rotary frequencies are cut into ``sections`` (their sizes sum to D/2) and section i
    turns with position set i mod 3.  With three equal position rows this is ordinary RoPE
    (Qwen2-VL; transformers modeling_qwen2_vl.py ``apply_multimodal_rotary_pos_emb`` is the behaviour matched)."""
    d = x.shape[-1]
    half = d // 2
    if sum(sections) != half:
        raise ValueError(f"mrope_section {list(sections)} must sum to head_dim / 2 = {half}")
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))  # [half]
    ang = positions3.float()[:, :, None] * inv[None, None, :]                                  # [3, T, half]
    which = torch.cat([torch.full((n,), i % 3, dtype=torch.long) for i, n in enumerate(sections)]).to(x.device)
    ang = ang.gather(0, which[None, None, :].expand(1, ang.shape[1], half))[0]                 # [T, half]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dim."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def attention_varlen(q, k, v, cu_seqlens, max_seqlen=None, causal=True, scale=None, window=None):
    """Causal GQA attention over packed documents.

    q [T, Hq, D]; k, v [T, Hkv, D]; ``cu_seqlens`` int tensor [n_docs + 1].
    A dense block-diagonal mask is built: fine for an oracle, O(T^2) memory.
    """
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    doc = torch.bucketize(torch.arange(T, device=q.device), cu_seqlens[1:].to(q.device), right=True)
    mask = doc[:, None] == doc[None, :]
    if causal:
        idx = torch.arange(T, device=q.device)
        mask = mask & (idx[:, None] >= idx[None, :])
    if window:
        idx = torch.arange(T, device=q.device)
        mask = mask & (idx[:, None] - idx[None, :] < window)
        if not causal:
            mask = mask & (idx[None, :] - idx[:, None] < window)
    rep = Hq // Hkv
    qf = q.float().transpose(0, 1)  # [Hq, T, D]
    kf = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf)  # [Hq, T, D]
    return o.transpose(0, 1).to(q.dtype).contiguous()


def attention_varlen_qk(q, k, v, cu_q, cu_k, scale=None):
    """Causal GQA attention, query segment i (``cu_q``) against key segment i (``cu_k``), mask aligned to the end of the
    key segment: query j of a segment with lq queries and lk keys sees keys 0 .. j + lk - lq.  Dense mask, oracle only."""
    Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[0], k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    cq, ck = cu_q.to(q.device).long(), cu_k.to(q.device).long()
    iq, ik = torch.arange(Tq, device=q.device), torch.arange(Tk, device=q.device)
    sq = torch.bucketize(iq, cq[1:], right=True)
    sk = torch.bucketize(ik, ck[1:], right=True)
    # position of every query / key counted from the END of its segment
    q_from_end = cq[1:][sq] - iq
    k_from_end = ck[1:][sk] - ik
    mask = (sq[:, None] == sk[None, :]) & (k_from_end[None, :] >= q_from_end[:, None])
    rep = Hq // Hkv
    qf = q.float().transpose(0, 1)
    kf = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf).transpose(0, 1).to(q.dtype).contiguous()


def lm_head_logprobs(hidden, weight, labels, temperature=1.0, bias=None, softcap=None,
                     compute_entropy=True, entropy_grad=False):
    """Per-token log p(label) and entropy from ``hidden[N,H] @ weight[V,H]^T``.

    Entropy carries no gradient (matches trl/trainer/utils.py:1291-1424) unless ``entropy_grad``
    (the differentiable entropy of the GRPO bonus, trl/trainer/grpo_trainer.py:3155-3175).
    """
    logits = hidden.float() @ weight.float().t()
    if bias is not None:
        logits = logits + bias.float()
    if softcap:
        logits = torch.tanh(logits / softcap) * softcap
    logits = logits / temperature
    lse = torch.logsumexp(logits, dim=-1)
    tgt = logits.gather(-1, labels.long().clamp_min(0)[:, None]).squeeze(-1)
    logp = tgt - lse
    ent = None
    if compute_entropy:
        with torch.set_grad_enabled(bool(entropy_grad) and torch.is_grad_enabled()):
            p = torch.softmax(logits, dim=-1)
            ent = (lse if entropy_grad else lse.detach()) - (p * logits).sum(-1)
    return logp, ent


def lm_head_ce(hidden, weight, labels, ignore_index=-100, bias=None):
    """Sum of token NLL over valid labels plus (correct, entropy_sum, n_valid).

    Mirrors the quantities of trl/trainer/sft_trainer.py:117-234.  When no label
    is valid the loss is ``(hidden.sum() + weight.sum()) * 0`` so that backward
    and gradient synchronisation still run on every rank.
    """
    valid = labels != ignore_index
    n_valid = valid.sum()
    if int(n_valid) == 0:
        z = (hidden.sum() + weight.sum()).float() * 0.0
        zero = torch.zeros((), device=hidden.device)
        return z, zero, zero, n_valid
    h = hidden[valid]
    y = labels[valid]
    logits = h.float() @ weight.float().t()
    if bias is not None:
        logits = logits + bias.float()
    logp = torch.log_softmax(logits, dim=-1)
    nll = -logp.gather(-1, y[:, None]).squeeze(-1)
    with torch.no_grad():
        correct = (logits.argmax(-1) == y).sum()
        ent = -(logp.exp() * logp).sum(-1).sum()
    return nll.sum(), correct, ent, n_valid


def selective_log_softmax(logits, index):
    """log_softmax(logits).gather(index); index [...] or [..., K] (utils.py:479-523)."""
    squeeze = index.ndim == logits.ndim - 1
    if squeeze:
        index = index.unsqueeze(-1)
    if logits.dtype in (torch.float32, torch.float64):
        sel = torch.gather(logits, dim=-1, index=index)
        lse = torch.stack([torch.logsumexp(l, dim=-1) for l in logits])
        out = sel - lse.unsqueeze(-1)
    else:
        out = torch.stack([F.log_softmax(rl, dim=-1).gather(-1, ri) for rl, ri in zip(logits, index)])
    return out.squeeze(-1) if squeeze else out


def entropy_from_logits(logits: torch.Tensor, chunk_size: int = 128) -> torch.Tensor:
    """Shannon entropy (nats) row-chunked (utils.py:526-560)."""
    shp = logits.shape[:-1]
    flat = logits.reshape(-1, logits.shape[-1])
    outs = []
    for c in flat.split(chunk_size, dim=0):
        lp = F.log_softmax(c, dim=-1)
        outs.append(-(lp.exp() * lp).sum(-1))
    return torch.cat(outs, 0).reshape(shp) if outs else flat.new_zeros(shp)


def moe_router(hidden, gate_weight, top_k, norm_topk_prob):
    """softmax(fp32) -> top-k -> optional renormalise.  Returns (probs, idx, full_probs)."""
    logits = hidden.float() @ gate_weight.float().t()
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    return w, idx, probs


def moe_experts(hidden, gate_up_w, down_w, topk_w, topk_idx):
    """Dense loop over experts.  gate_up_w [E, 2I, H]; down_w [E, H, I]."""
    out = torch.zeros_like(hidden, dtype=torch.float32)
    E = gate_up_w.shape[0]
    for e in range(E):
        tok, slot = (topk_idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        x = hidden[tok].float()
        gu = x @ gate_up_w[e].float().t()
        act = swiglu(gu)
        y = act @ down_w[e].float().t()
        out.index_add_(0, tok, y * topk_w[tok, slot].float()[:, None])
    return out.to(hidden.dtype)


def load_balancing_loss(router_probs, topk_idx, num_experts, top_k, token_mask=None):
    """Switch-style aux loss ``E * sum_e f_e * P_e`` over all layers' tokens.

    router_probs [L*T, E] are post-softmax probabilities; topk_idx [L*T, K].
    """
    onehot = F.one_hot(topk_idx, num_experts).float()  # [N, K, E]
    if token_mask is None:
        f = onehot.mean(0)  # [K, E]
        p = router_probs.float().mean(0)
    else:
        m = token_mask.float().reshape(-1)
        f = (onehot * m[:, None, None]).sum(0) / m.sum().clamp_min(1)
        p = (router_probs.float() * m[:, None]).sum(0) / m.sum().clamp_min(1)
    return (f * p[None, :]).sum() * num_experts


def grpo_token_loss(logp, old_logp, ref_logp, adv, eps_low, eps_high, beta, delta=None):
    """Token-level clipped surrogate + k3 KL (grpo_trainer.py:3054-3121)."""
    ratio = torch.exp(logp - old_logp)
    clipped = torch.clamp(ratio, 1 - eps_low, 1 + eps_high)
    r1 = ratio if delta is None else torch.clamp(ratio, max=delta)
    loss = -torch.min(r1 * adv, clipped * adv)
    kl = None
    if beta != 0.0 and ref_logp is not None:
        d = ref_logp - logp
        kl = torch.exp(d) - d - 1
        loss = loss + beta * kl
    return loss, ratio, kl


def dpo_sigmoid_loss(pol_c, pol_r, ref_c, ref_r, beta, label_smoothing=0.0):
    d = (pol_c - ref_c) - (pol_r - ref_r)
    loss = -F.logsigmoid(beta * d) * (1 - label_smoothing) - F.logsigmoid(-beta * d) * label_smoothing
    return loss, beta * (pol_c - ref_c), beta * (pol_r - ref_r)
