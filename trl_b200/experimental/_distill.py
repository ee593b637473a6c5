"""Shared pieces of the distillation trainers: divergences between a student's and a teacher's next-token
distributions computed chunk by chunk from hidden states (the [tokens, vocab] logits of both models exist only for one
chunk at a time), and on-policy completion sampling from either model.

Divergence definitions follow trl/experimental/gkd/gkd_trainer.py:193-262 (generalised JSD) and the forward / reverse
KL used by trl/experimental/minillm and trl/experimental/distillation."""
from __future__ import annotations

import torch


def generalized_jsd_loss(student_logits, teacher_logits, labels=None, beta: float = 0.5, temperature: float = 1.0,
                         reduction: str = "batchmean", num_items_in_batch=None):
    """JSD(beta) per position, then reduced.  beta = 0: KL(teacher || student) (forward KL); beta = 1: KL(student ||
    teacher) (reverse KL); otherwise beta * KL(teacher || M) + (1 - beta) * KL(student || M) with the mixture
    M = beta * teacher + (1 - beta) * student.  ``labels == -100`` positions are left out."""
    from .sdft.loss_utils import compute_divergence

    per_pos = compute_divergence(torch.log_softmax(student_logits / temperature, -1),
                                 torch.log_softmax(teacher_logits / temperature, -1), float(beta))
    if labels is not None:
        keep = labels != -100
        per_pos = per_pos[keep]
        count = keep.sum()
    else:
        count = per_pos.numel()
    if num_items_in_batch is not None:
        return per_pos.sum() / num_items_in_batch
    if reduction == "batchmean":
        return per_pos.sum() / count
    if reduction == "sum":
        return per_pos.sum()
    if reduction == "mean":
        return per_pos.mean()
    return per_pos


def chunked_token_divergence(h_student, w_student, h_teacher, w_teacher, beta: float = 0.5, temperature: float = 1.0,
                             chunk: int = 2048, weights=None, softcap=None):
    """Sum over rows of JSD(beta) between softmax(h_s W_s^T / T) and softmax(h_t W_t^T / T); rows may carry weights.
    Returns (sum, per-row divergence detached)."""
    total = h_student.new_zeros((), dtype=torch.float32)
    per_row = []
    for s in range(0, h_student.shape[0], chunk):
        sl = slice(s, s + chunk)
        zs = h_student[sl].float() @ w_student.float().t()
        with torch.no_grad():
            zt = h_teacher[sl].float() @ w_teacher.float().t()
        if softcap:
            zs, zt = torch.tanh(zs / softcap) * softcap, torch.tanh(zt / softcap) * softcap
        d = generalized_jsd_loss(zs, zt, beta=beta, temperature=temperature, reduction="none")
        per_row.append(d.detach())
        total = total + (d * weights[sl] if weights is not None else d).sum()
    return total, (torch.cat(per_row) if per_row else h_student.new_zeros(0))


_GENERATORS: dict = {}


def generator_for(model):
    """Rollout engine on CUDA (paged KV, CUDA-graph decode; weights read in place), eager generator on CPU."""
    from ..rollout.engine import EagerGenerator

    key = id(model)
    if key not in _GENERATORS:
        _GENERATORS[key] = EagerGenerator(model) if model.device.type != "cuda" else None
    return _GENERATORS[key]


def sample_completions(model, prompts, max_new_tokens, temperature=1.0, top_p=1.0, top_k=0, eos_token_id=None, seed=0,
                       engine_cache=None):
    """prompts: list of id lists -> list of completion id lists sampled from ``model``."""
    from ..rollout.sampling import SamplingParams

    sp = SamplingParams(n=1, max_tokens=max_new_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                        eos_token_id=eos_token_id, seed=seed)
    if model.device.type == "cuda":
        from ..rollout.engine import RolloutEngine

        cache = engine_cache if engine_cache is not None else _GENERATORS
        need = max(len(p) for p in prompts) + max_new_tokens + 8
        eng = cache.get(("engine", id(model)))
        if eng is None or eng.max_len < need or eng.max_seqs < len(prompts):
            eng = RolloutEngine(model, max_num_seqs=max(len(prompts), 8), max_model_len=(need + 63) // 64 * 64)
            cache[("engine", id(model))] = eng
        outs = eng.generate(prompts, sp)
    else:
        outs = generator_for(model).generate(prompts, sp)
    return [o.token_ids for o in outs]
