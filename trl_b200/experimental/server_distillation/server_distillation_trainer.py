"""Distillation against a teacher behind a generation server (trl/experimental/server_distillation/
server_distillation_trainer.py:60-545).

The teacher is never loaded here: per-token teacher log-probs of the student's completions come from the server's
``/get_sequence_logprobs/`` route, so the divergence lives on a sparse support: the sampled token plus one tail
bucket holding the remaining mass.  beta = 1 gives the reverse-KL surrogate on that two-point support, beta = 0 the
forward KL, values in between the JSD."""
from __future__ import annotations

import torch

from ...generation.client import VLLMClient
from ...ops import functional as ops
from ..distillation.distillation_trainer import DistillationTrainer
from ..gkd.gkd_trainer import GKDTrainer
from ..sdft.loss_utils import add_tail_bucket, compute_divergence
from .server_distillation_config import ServerDistillationConfig


def build_teacher_request_inputs(input_ids: torch.Tensor, attention_mask: torch.Tensor,
                                 prompt_attention_mask: torch.Tensor | None = None, labels: torch.Tensor | None = None):
    """Padded batch -> what a teacher-server request needs: (unpadded token rows, prompt lengths, completion lengths).
    The prompt length of a row comes from ``prompt_attention_mask`` or, without it, from the number of unmasked
    ``labels`` (server_distillation_trainer.py:84-127)."""
    if input_ids.shape != attention_mask.shape:
        raise ValueError(f"input_ids and attention_mask must have the same shape, got {tuple(input_ids.shape)} and "
                         f"{tuple(attention_mask.shape)}.")
    ids, keep = input_ids.detach().cpu(), attention_mask.detach().cpu().bool()
    if prompt_attention_mask is not None:
        p_len = prompt_attention_mask.detach().cpu().sum(1).long()
    else:
        if labels is None:
            raise ValueError("labels are required when prompt_attention_mask is not provided.")
        if labels.shape != input_ids.shape:
            raise ValueError(f"labels must match input_ids shape, got {tuple(labels.shape)} and {tuple(input_ids.shape)}.")
        p_len = keep.sum(1).long() - (labels.detach().cpu() != -100).sum(1).long()
    rows, plens, clens = [], [], []
    for row, m, pl in zip(ids, keep, p_len.tolist()):
        r = row[m].tolist()
        if pl < 0 or pl > len(r):
            raise ValueError(f"Invalid prompt length {pl} for trimmed sequence of length {len(r)}.")
        rows.append(r)
        plens.append(int(pl))
        clens.append(len(r) - int(pl))
    return rows, plens, clens


class ServerDistillationTrainer(DistillationTrainer):
    _tag_names = ["trl", "server-distillation"]
    _name = "ServerDistillation"

    def __init__(self, model=None, args: ServerDistillationConfig | None = None, teacher_client=None, **kw):
        # skip GKDTrainer's teacher loading: go straight to the SFT constructor, then set the shared fields
        from ...trainer.sft_trainer import SFTTrainer
        import random

        SFTTrainer.__init__(self, model, args, **kw)
        self.teacher_model = None
        self.lmbda, self.beta, self.temperature, self.seq_kd = args.lmbda, args.beta, args.temperature, False
        self._rng = random.Random(args.seed)
        self._gen_cache: dict = {}
        self.teacher_client = teacher_client or VLLMClient(base_url=args.teacher_model_server_url)

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        ids, am, labels = inputs["input_ids"], inputs["attention_mask"], inputs["labels"]
        seqs, plens = [], []
        for row, m, lab in zip(ids.tolist(), am.tolist(), labels.tolist()):
            n = sum(m)
            seqs.append(row[:n])
            plens.append(next((i for i in range(n) if lab[i] != -100), n))
        t_rows = self.teacher_client.get_sequence_logprobs(seqs, plens, temperature=self.temperature)
        flat, ctx, tgt = self._flat_labels(model, inputs)
        hidden = model.forward_hidden(flat, ctx)
        sel = (tgt != -100).nonzero().flatten()
        s_lp, _ = ops.lm_head_logprobs(hidden[sel], model.lm_head_weight, tgt[sel], self.temperature, compute_entropy=False)
        t_lp = torch.tensor([x for r in t_rows for x in r], dtype=torch.float32, device=s_lp.device)
        if t_lp.numel() != s_lp.numel():
            raise ValueError(f"teacher server returned {t_lp.numel()} log-probs for {s_lp.numel()} completion tokens")
        s2, t2 = s_lp[:, None].clamp(max=-1e-7), t_lp[:, None].clamp(max=-1e-7)
        if self.args.loss_add_tail:
            s2, t2 = add_tail_bucket(s2), add_tail_bucket(t2)
        if self.beta == 1.0 and not self.args.loss_add_tail:
            per = (s_lp - t_lp).detach() * s_lp  # single-point support: the score-function surrogate
        else:
            per = compute_divergence(s2, t2, self.beta)
        denom = num_items_in_batch if num_items_in_batch is not None else max(1, sel.numel())
        loss = per.sum() / denom
        self._metrics["train" if model.training else "eval"]["jsd"].append(per.detach().mean())
        return (loss, None) if return_outputs else loss
