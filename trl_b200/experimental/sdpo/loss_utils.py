"""Self-distillation losses used by SDPO (trl/experimental/sdpo/loss_utils.py:21-135); same definitions as the SDFT
module: divergence on the student top-k support, on the full vocabulary, or a reverse-KL surrogate on sampled tokens."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def compute_divergence(student_log_probs, teacher_log_probs, alpha: float):
    """alpha = 0: KL(teacher || student); alpha = 1: KL(student || teacher); else JSD(alpha).  Summed over the support."""
    if alpha == 0.0:
        kl = F.kl_div(student_log_probs, teacher_log_probs, reduction="none", log_target=True)
    elif alpha == 1.0:
        kl = F.kl_div(teacher_log_probs, student_log_probs, reduction="none", log_target=True)
    else:
        a = torch.tensor(alpha, dtype=student_log_probs.dtype, device=student_log_probs.device)
        mix = torch.logsumexp(torch.stack([student_log_probs + torch.log(1 - a), teacher_log_probs + torch.log(a)]), dim=0)
        kl = torch.lerp(F.kl_div(mix, student_log_probs, reduction="none", log_target=True),
                        F.kl_div(mix, teacher_log_probs, reduction="none", log_target=True), alpha)
    return kl.sum(-1)


def add_tail_bucket(log_probs):
    """Top-k log-probs sum to the captured mass <= 1: append log(1 - mass) as one more category."""
    log_s = torch.logsumexp(log_probs, dim=-1, keepdim=True).clamp(max=-1e-7)
    return torch.cat([log_probs, torch.log(-torch.expm1(log_s))], dim=-1)


def apply_importance_sampling_clipping(per_token_loss, student_log_probs, old_log_probs, clip_coeff: float):
    neg_kl = (student_log_probs - old_log_probs).detach().clamp(min=-20.0, max=20.0)
    return per_token_loss * torch.exp(neg_kl).clamp(max=clip_coeff)


def compute_topk_self_distillation_loss(student_logits, teacher_logits, *, distillation_topk, distillation_alpha,
                                        distillation_add_tail):
    s_lse = torch.logsumexp(student_logits, dim=-1, keepdim=True)
    top_s, idx = torch.topk(student_logits, k=min(distillation_topk, student_logits.shape[-1]), dim=-1)
    s = top_s - s_lse
    t = torch.gather(teacher_logits, -1, idx) - torch.logsumexp(teacher_logits, dim=-1, keepdim=True)
    if distillation_add_tail:
        s, t = add_tail_bucket(s), add_tail_bucket(t)
    else:
        s, t = s - torch.logsumexp(s, -1, keepdim=True), t - torch.logsumexp(t, -1, keepdim=True)
    return compute_divergence(s, t, distillation_alpha)


def compute_full_logit_self_distillation_loss(student_logits, teacher_logits, *, distillation_alpha):
    return compute_divergence(torch.log_softmax(student_logits, -1), torch.log_softmax(teacher_logits, -1),
                              distillation_alpha)


def compute_sampled_token_self_distillation_loss(student_logits, teacher_logits, completion_ids, *, distillation_alpha):
    if distillation_alpha != 1.0:
        raise ValueError("Only reverse KL (alpha=1.0) is supported for token-level distillation when "
                         f"`distillation_mode='sampled_token'`, got alpha={distillation_alpha}")
    s = torch.log_softmax(student_logits, -1).gather(-1, completion_ids[..., None]).squeeze(-1)
    t = torch.log_softmax(teacher_logits, -1).gather(-1, completion_ids[..., None]).squeeze(-1)
    return (s - t).detach() * s
