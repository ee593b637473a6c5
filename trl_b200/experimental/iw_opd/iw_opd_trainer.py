"""Importance-weighted on-policy distillation (trl/experimental/iw_opd/iw_opd_trainer.py: loss :1231-1286).

Sampled-token objective on the student's own completions: per-token advantage A_t = log p_teacher(y_t) - log p_rollout(y_t)
(detached), position weights w_t = 1 + gamma * (1 - sum_{s<t}|A_s| / sum_s|A_s|) so early tokens, whose errors condition
everything after them, count more; loss = -sum_t w_t A_t log p_student(y_t) / #tokens."""
from __future__ import annotations

import torch

from ...ops import functional as ops
from ...parallel import dist as D
from ..distillation.distillation_trainer import DistillationTrainer
from .iw_opd_config import IWOPDConfig


def iw_opd_weights(a_opd: torch.Tensor, mask: torch.Tensor, gamma: float, eps: float) -> torch.Tensor:
    """a_opd, mask: [B, T].  Weight of token t from the share of |A| mass that lies before it."""
    ab = a_opd.abs() * mask
    prefix = ab.cumsum(1) - ab
    total = ab.sum(1, keepdim=True).clamp_min(eps)
    return 1.0 + gamma * (1.0 - prefix / total)


class IWOPDTrainer(DistillationTrainer):
    _tag_names = ["trl", "iw-opd"]
    _name = "IWOPD"

    def __init__(self, model=None, teacher_model=None, args: IWOPDConfig | None = None, **kw):
        super().__init__(model, teacher_model, args or IWOPDConfig("model-IWOPD"), **kw)

    def _teacher_token_logps(self, flat, ctx, sel, tgt):
        with torch.no_grad():
            h = self.teacher_model.forward_hidden(flat, ctx)
            return ops.lm_head_logprobs(h[sel], self.teacher_model.lm_head_weight, tgt[sel], self.temperature,
                                        compute_entropy=False)[0]

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        if self.args.distillation_objective == "jsd":
            return super().compute_loss(model, inputs, return_outputs, num_items_in_batch)
        flat, ctx, tgt = self._flat_labels(model, inputs)
        hidden = model.forward_hidden(flat, ctx)
        sel = (tgt != -100).nonzero().flatten()
        s_lp, _ = ops.lm_head_logprobs(hidden[sel], model.lm_head_weight, tgt[sel], self.temperature, compute_entropy=False)
        t_lp = self._teacher_token_logps(flat, ctx, sel, tgt)
        # [B, T] layout for the per-sequence prefix sums
        seq_id = torch.repeat_interleave(torch.arange(ctx.cu_seqlens.numel() - 1, device=flat.device),
                                         (ctx.cu_seqlens[1:] - ctx.cu_seqlens[:-1]).long())[sel]
        n_seq = ctx.cu_seqlens.numel() - 1
        counts = torch.bincount(seq_id, minlength=n_seq)
        start = torch.cumsum(counts, 0) - counts
        col = torch.arange(sel.numel(), device=flat.device) - start[seq_id]
        T = int(counts.max()) if sel.numel() else 1
        a_pad = torch.zeros(n_seq, T, device=flat.device)
        mask = torch.zeros(n_seq, T, device=flat.device)
        a_opd = (t_lp - s_lp).detach()
        a_pad[seq_id, col], mask[seq_id, col] = a_opd, 1.0
        w = iw_opd_weights(a_pad, mask, self.args.iw_opd_gamma, self.args.iw_opd_epsilon)[seq_id, col]
        adv = (w * a_opd).detach()
        loss_sum = -(s_lp * adv).sum()
        denom = num_items_in_batch if num_items_in_batch is not None else max(1, sel.numel())
        loss = loss_sum / denom
        m = self._metrics["train" if model.training else "eval"]
        if sel.numel():
            st = torch.stack([adv.mean(), a_opd.abs().mean(), w.mean(), w.min(), w.max()])
            for k, v in zip(["iw_opd/mean_advantage", "iw_opd/mean_abs_advantage", "iw_opd/mean_weight",
                             "iw_opd/min_weight", "iw_opd/max_weight"], st):
                m[k].append(v)
        return (loss, None) if return_outputs else loss
