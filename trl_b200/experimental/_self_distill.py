"""Token-level self-distillation between the student under its own prompt and a teacher under a privileged prompt, on
completions sampled by the student.  Shared by SDFT and SDPO."""
from __future__ import annotations

import torch


class SelfDistillMixin:
    """Needs ``self._get_per_token_logps_and_entropies`` (online trainer), ``self.teacher`` (module or None) and the
    config fields distillation_{mode,alpha,topk,add_tail,is_clip}, num_loss_tokens_to_skip."""

    def _selected(self, model, prompt_ids, completion_ids, grad: bool):
        self._keep_selected_hidden = True
        try:
            with torch.enable_grad() if grad else torch.no_grad():
                lp, _ = self._get_per_token_logps_and_entropies(model, prompt_ids, completion_ids)
            hidden, r, c = self._selected_hidden[:3]
        finally:
            self._keep_selected_hidden, self._selected_hidden = False, None
        return lp, hidden, r, c

    def self_distillation_loss(self, model, prompt_ids, teacher_prompt_ids, completion_ids, old_logps=None,
                               row_weight=None, chunk: int = 1024):
        """Mean over completion tokens (of rows with weight > 0) of the configured divergence."""
        from .sdft.loss_utils import (apply_importance_sampling_clipping, compute_full_logit_self_distillation_loss,
                                      compute_sampled_token_self_distillation_loss, compute_topk_self_distillation_loss)

        a = self.args
        lp, h_s, r, c = self._selected(model, prompt_ids, completion_ids, grad=True)
        teacher = self.teacher if self.teacher is not None else model
        _, h_t, _, _ = self._selected(teacher, teacher_prompt_ids, completion_ids, grad=False)
        tgt = torch.tensor([t for ids in completion_ids for t in ids], dtype=torch.long, device=h_s.device)
        w_s, w_t = model.lm_head_weight, teacher.lm_head_weight
        per_tok = []
        for s in range(0, h_s.shape[0], chunk):
            sl = slice(s, s + chunk)
            zs = h_s[sl].float() @ w_s.float().t()
            with torch.no_grad():
                zt = h_t[sl].float() @ w_t.float().t()
            if a.distillation_mode == "topk_logits":
                d = compute_topk_self_distillation_loss(zs, zt, distillation_topk=a.distillation_topk,
                                                        distillation_alpha=a.distillation_alpha,
                                                        distillation_add_tail=a.distillation_add_tail)
            elif a.distillation_mode == "full_logits":
                d = compute_full_logit_self_distillation_loss(zs, zt, distillation_alpha=a.distillation_alpha)
            else:
                d = compute_sampled_token_self_distillation_loss(zs, zt, tgt[sl], distillation_alpha=a.distillation_alpha)
            per_tok.append(d)
        per_tok = torch.cat(per_tok) if per_tok else h_s.new_zeros(0)
        if old_logps is not None and a.distillation_is_clip is not None:
            per_tok = apply_importance_sampling_clipping(per_tok, lp[r, c], old_logps[r, c], a.distillation_is_clip)
        w = torch.ones_like(per_tok)
        if a.num_loss_tokens_to_skip:
            w = w * (c >= a.num_loss_tokens_to_skip).float()
        if row_weight is not None:
            w = w * row_weight[r]
        return (per_tok * w).sum() / w.sum().clamp(min=1.0), per_tok.detach()
