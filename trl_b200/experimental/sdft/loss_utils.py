"""Divergences for token-level self-distillation.

One routine, ``support_divergence``, scores a student against a teacher on a chosen *support* of the vocabulary:
the whole vocabulary, the student's top-k tokens (renormalised, or completed with one bucket that holds the rest of
the probability mass), or just the sampled token.  ``alpha`` picks the direction: 0 -> KL(teacher || student),
1 -> KL(student || teacher), in between the skewed Jensen-Shannon mixture.  The public names below are the ones the
reference exposes (trl/experimental/sdft/loss_utils.py:21-135)."""
from __future__ import annotations

import torch


def _kl(log_p, log_q):
    """sum_i p_i (log p_i - log q_i) along the last dim, from log-probabilities."""
    return (log_p.exp() * (log_p - log_q)).sum(-1)


def compute_divergence(student_log_probs, teacher_log_probs, alpha: float):
    s, t = student_log_probs, teacher_log_probs
    if alpha == 0.0:
        return _kl(t, s)
    if alpha == 1.0:
        return _kl(s, t)
    a = torch.as_tensor(alpha, dtype=s.dtype, device=s.device)
    mix = torch.logaddexp(s + torch.log1p(-a), t + torch.log(a))
    return (1 - alpha) * _kl(s, mix) + alpha * _kl(t, mix)


def add_tail_bucket(log_probs):
    """log-probs of a subset (their mass is at most 1) -> one more entry with the log of the missing mass."""
    mass = torch.logsumexp(log_probs, dim=-1, keepdim=True).clamp(max=-1e-7)
    rest = torch.log1p(-mass.exp())
    return torch.cat([log_probs, rest], dim=-1)


def _on_support(logits, index):
    return logits.gather(-1, index) - torch.logsumexp(logits, dim=-1, keepdim=True)


def support_divergence(student_logits, teacher_logits, alpha, topk=None, add_tail=False):
    if topk is None or topk >= student_logits.shape[-1]:
        return compute_divergence(torch.log_softmax(student_logits, -1), torch.log_softmax(teacher_logits, -1), alpha)
    index = student_logits.topk(topk, dim=-1).indices  # the student's own most likely tokens define the support
    s, t = _on_support(student_logits, index), _on_support(teacher_logits, index)
    if add_tail:
        s, t = add_tail_bucket(s), add_tail_bucket(t)
    else:
        s, t = torch.log_softmax(s, -1), torch.log_softmax(t, -1)
    return compute_divergence(s, t, alpha)


def compute_topk_self_distillation_loss(student_logits, teacher_logits, *, distillation_topk, distillation_alpha,
                                        distillation_add_tail):
    return support_divergence(student_logits, teacher_logits, distillation_alpha, distillation_topk, distillation_add_tail)


def compute_full_logit_self_distillation_loss(student_logits, teacher_logits, *, distillation_alpha):
    return support_divergence(student_logits, teacher_logits, distillation_alpha)


def compute_sampled_token_self_distillation_loss(student_logits, teacher_logits, completion_ids, *, distillation_alpha):
    """Reverse KL estimated on the sampled token: (log p_s - log p_t), detached, times log p_s (score function)."""
    if distillation_alpha != 1.0:
        raise ValueError("Only reverse KL (alpha=1.0) is supported for token-level distillation when "
                         f"`distillation_mode='sampled_token'`, got alpha={distillation_alpha}")
    idx = completion_ids[..., None]
    s, t = _on_support(student_logits, idx).squeeze(-1), _on_support(teacher_logits, idx).squeeze(-1)
    return (s - t).detach() * s


def apply_importance_sampling_clipping(per_token_loss, student_log_probs, old_log_probs, clip_coeff: float):
    """Weights the loss by min(pi / pi_old, clip) with the ratio treated as a constant."""
    log_w = (student_log_probs - old_log_probs).detach().clamp(-20.0, 20.0)
    return per_token_loss * log_w.exp().clamp(max=clip_coeff)
