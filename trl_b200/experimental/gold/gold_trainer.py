"""GOLD: general on-policy logit distillation, also across tokenizers (trl/experimental/gold/gold_trainer.py:
ULDLoss :250-900, trainer :1000-2900).

With the same tokenizer this is the on-policy JSD distillation of ``DistillationTrainer``.  With
``use_uld_loss`` the teacher may use another vocabulary: the completion text is re-tokenised for the teacher, student
and teacher tokens are grouped into spans that cover the same characters, per-span distributions are merged, and the
distance is the L1 difference of the *sorted* probability vectors (zero-padded to the larger vocabulary), which needs
no token correspondence.  The hybrid variant adds a JSD over the token strings both vocabularies share."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .._distill import generalized_jsd_loss
from ..distillation.distillation_trainer import DistillationTrainer
from .gold_config import GOLDConfig


def align_spans(student_pieces: list[str], teacher_pieces: list[str]) -> list[tuple[list[int], list[int]]]:
    """Greedy grouping of two tokenisations of one text into spans ending at common character offsets."""
    spans, i, j, ls, lt = [], 0, 0, 0, 0
    cs, ct = [], []
    while i < len(student_pieces) or j < len(teacher_pieces):
        if (ls <= lt and i < len(student_pieces)) or j >= len(teacher_pieces):
            ls += len(student_pieces[i])
            cs.append(i)
            i += 1
        else:
            lt += len(teacher_pieces[j])
            ct.append(j)
            j += 1
        if ls == lt and cs and ct:
            spans.append((cs, ct))
            cs, ct = [], []
    if cs and ct:
        spans.append((cs, ct))
    return spans


class ULDLoss:
    def __init__(self, config: GOLDConfig, student_tokenizer, teacher_tokenizer):
        self.cfg, self.s_tok, self.t_tok = config, student_tokenizer, teacher_tokenizer
        self._matched = None

    def _merge(self, probs: torch.Tensor, groups: list[list[int]]) -> torch.Tensor:
        how = self.cfg.uld_token_merge_strategy
        rows = []
        for g in groups:
            p = probs[g]
            rows.append(p.mean(0) if how == "mean" else (p[0] if how == "first" else p[-1]))
        return torch.stack(rows) if rows else probs[:0]

    def _matched_ids(self):
        if self._matched is None:
            sv, tv = self.s_tok.get_vocab(), self.t_tok.get_vocab()
            common = sorted(set(sv) & set(tv))
            self._matched = (torch.tensor([sv[k] for k in common], dtype=torch.long),
                             torch.tensor([tv[k] for k in common], dtype=torch.long))
        return self._matched

    def __call__(self, student_logits, teacher_logits, student_ids, teacher_ids):
        """One sequence: logits [Ts, Vs] / [Tt, Vt] on the completion positions, ids of the completion tokens."""
        c = self.cfg
        ps = torch.softmax(student_logits.float() / c.uld_student_temperature, -1)
        pt = torch.softmax(teacher_logits.float() / c.uld_teacher_temperature, -1)
        if c.uld_skip_student_eos and len(student_ids) and student_ids[-1] == self.s_tok.eos_token_id:
            ps, student_ids = ps[:-1], student_ids[:-1]
        if c.uld_skip_teacher_eos and len(teacher_ids) and teacher_ids[-1] == self.t_tok.eos_token_id:
            pt, teacher_ids = pt[:-1], teacher_ids[:-1]
        if c.use_extended_uld:
            sp = [self.s_tok.decode([t]) for t in student_ids]
            tp = [self.t_tok.decode([t]) for t in teacher_ids]
            spans = align_spans(sp, tp)
            ps, pt = self._merge(ps, [a for a, _ in spans]), self._merge(pt, [b for _, b in spans])
        n = min(ps.shape[0], pt.shape[0])
        if n == 0:
            return student_logits.sum() * 0.0
        ps, pt = ps[:n], pt[:n]
        loss = 0.0
        if c.uld_use_hybrid_loss:
            ms, mt = self._matched_ids()
            ms, mt = ms.to(ps.device), mt.to(pt.device)
            if ms.numel():
                qs, qt = ps[:, ms], pt[:, mt]
                matched_mass = 0.5 * (qs.sum(-1) + qt.sum(-1)).detach()
                jsd = generalized_jsd_loss(torch.log(qs.clamp_min(1e-12)), torch.log(qt.clamp_min(1e-12)), beta=c.beta,
                                           reduction="none")
                wm = c.uld_hybrid_matched_weight if c.uld_hybrid_matched_weight is not None else matched_mass
                wu = c.uld_hybrid_unmatched_weight if c.uld_hybrid_unmatched_weight is not None else 1 - matched_mass
                keep_s = torch.ones(ps.shape[1], dtype=torch.bool, device=ps.device)
                keep_t = torch.ones(pt.shape[1], dtype=torch.bool, device=pt.device)
                keep_s[ms], keep_t[mt] = False, False
                l1 = self._sorted_l1(ps[:, keep_s], pt[:, keep_t])
                return ((wm * jsd).mean() + (wu * l1).mean()) * c.uld_distillation_weight
        loss = self._sorted_l1(ps, pt).mean() * c.uld_distillation_weight
        return loss

    @staticmethod
    def _sorted_l1(ps, pt):
        ss, st = torch.sort(ps, -1, descending=True).values, torch.sort(pt, -1, descending=True).values
        v = max(ss.shape[1], st.shape[1])
        return (F.pad(ss, (0, v - ss.shape[1])) - F.pad(st, (0, v - st.shape[1]))).abs().sum(-1)


class GOLDTrainer(DistillationTrainer):
    _tag_names = ["trl", "gold"]
    _name = "GOLD"

    def __init__(self, model=None, teacher_model=None, args: GOLDConfig | None = None, teacher_processing_class=None, **kw):
        args = args or GOLDConfig("model-GOLD")
        super().__init__(model, teacher_model, args, **kw)
        self.teacher_tokenizer = teacher_processing_class
        if self.teacher_tokenizer is None and args.teacher_tokenizer_name_or_path:
            from transformers import AutoTokenizer

            self.teacher_tokenizer = AutoTokenizer.from_pretrained(args.teacher_tokenizer_name_or_path)
        self.use_uld = bool(args.use_uld_loss and self.teacher_tokenizer is not None)
        if args.use_uld_loss and not self.use_uld:
            raise ValueError("use_uld_loss needs the teacher's tokenizer (teacher_processing_class or "
                             "teacher_tokenizer_name_or_path)")
        self.uld = ULDLoss(args, self.processing_class, self.teacher_tokenizer) if self.use_uld else None

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        if not self.use_uld:
            return super().compute_loss(model, inputs, return_outputs, num_items_in_batch)
        from ...models.decoder import SeqCtx

        ids, am, labels = inputs["input_ids"], inputs["attention_mask"], inputs["labels"]
        dev = ids.device
        s_tok, t_tok = self.processing_class, self.teacher_tokenizer
        total, n_seq, ce_sum, ce_n = 0.0, 0, 0.0, 0
        for row, m, lab in zip(ids.tolist(), am.tolist(), labels.tolist()):
            n = sum(m)
            first = next((i for i in range(n) if lab[i] != -100), n)
            p_ids, c_ids = row[:first], row[first:n]
            if not c_ids or not p_ids:
                continue
            tp = t_tok(s_tok.decode(p_ids), add_special_tokens=False)["input_ids"] or [t_tok.eos_token_id]
            tc = t_tok(s_tok.decode(c_ids), add_special_tokens=False)["input_ids"]
            if not tc:
                continue
            sf = torch.tensor(p_ids + c_ids, device=dev)
            hs = model.forward_hidden(sf, SeqCtx.from_lengths([len(sf)], dev))[len(p_ids) - 1:-1]
            zs = hs.float() @ model.lm_head_weight.float().t()
            with torch.no_grad():
                tf = torch.tensor(tp + tc, device=dev)
                ht = self.teacher_model.forward_hidden(tf, SeqCtx.from_lengths([len(tf)], dev))[len(tp) - 1:-1]
                zt = ht.float() @ self.teacher_model.lm_head_weight.float().t()
            total = total + self.uld(zs, zt, c_ids, tc)
            n_seq += 1
            if self.args.uld_crossentropy_weight:
                ce_sum = ce_sum + F.cross_entropy(zs, torch.tensor(c_ids, device=dev), reduction="sum")
                ce_n += len(c_ids)
        loss = total / max(1, n_seq)
        if self.args.uld_crossentropy_weight and ce_n:
            loss = loss + self.args.uld_crossentropy_weight * ce_sum / ce_n
        if not torch.is_tensor(loss):
            loss = model.lm_head_weight.sum() * 0.0
        self._metrics["train" if model.training else "eval"]["uld_loss"].append(loss.detach())
        return (loss, None) if return_outputs else loss
