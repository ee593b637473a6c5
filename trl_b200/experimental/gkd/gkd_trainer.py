"""Generalised knowledge distillation (trl/experimental/gkd/gkd_trainer.py: JSD :193-262, compute_loss :264-310,
on-policy generation :312-360, training_step :491-531).

SFT data pipeline; every step trains the student against a frozen teacher with JSD(beta) on the completion tokens.
With probability ``lmbda`` the completions of the batch are first replaced by samples from the student (on-policy),
else with ``seq_kd`` by samples from the teacher."""
from __future__ import annotations

import random

import torch

from ...parallel import dist as D
from ...trainer.sft_trainer import SFTTrainer
from ...trainer.utils import create_model_from_path, disable_dropout_in_model, pad
from .._distill import chunked_token_divergence, generalized_jsd_loss, sample_completions
from .gkd_config import GKDConfig


class GKDTrainer(SFTTrainer):
    _tag_names = ["trl", "gkd"]
    _name = "GKD"
    generalized_jsd_loss = staticmethod(generalized_jsd_loss)

    def __init__(self, model=None, teacher_model=None, args: GKDConfig | None = None, **kw):
        args = args or GKDConfig("model-GKD")
        if args.padding_free or args.packing:
            raise ValueError("GKD regenerates completions per example: packing / padding_free batches are not supported")
        super().__init__(model, args, **kw)
        teacher_model = teacher_model or args.teacher_model_name_or_path
        if teacher_model is None:
            raise ValueError("GKDTrainer needs a teacher_model")
        if isinstance(teacher_model, str):
            teacher_model = create_model_from_path(teacher_model, **dict(args.teacher_model_init_kwargs or {}))
        if args.disable_dropout:
            disable_dropout_in_model(self.model)
        self.teacher_model = teacher_model.to(self.args.device, dtype=self.model.dtype).eval().requires_grad_(False)
        self.lmbda, self.beta, self.temperature, self.seq_kd = args.lmbda, args.beta, args.temperature, args.seq_kd
        self._rng = random.Random(args.seed)
        self._gen_cache: dict = {}

    # ---- on-policy data ------------------------------------------------------------------------------------------
    def _prompts_of(self, inputs):
        ids, labels, am = inputs["input_ids"], inputs["labels"], inputs["attention_mask"]
        prompts = []
        for row, lab, m in zip(ids.tolist(), labels.tolist(), am.tolist()):
            n = sum(m)
            first = next((i for i in range(n) if lab[i] != -100), n)
            prompts.append(row[:max(first, 1)])
        return prompts

    def generate_on_policy_outputs(self, model, inputs):
        tok = self.processing_class
        prompts = self._prompts_of(inputs)
        comps = sample_completions(model, prompts, self.args.max_new_tokens, temperature=self.temperature,
                                   eos_token_id=tok.eos_token_id, seed=self._rng.randrange(1 << 30),
                                   engine_cache=self._gen_cache)
        dev = inputs["input_ids"].device
        seqs = [torch.tensor(p + c, dtype=torch.long) for p, c in zip(prompts, comps)]
        labs = [torch.tensor([-100] * len(p) + c, dtype=torch.long) for p, c in zip(prompts, comps)]
        return (pad(seqs, tok.pad_token_id, "right").to(dev), pad([torch.ones_like(s) for s in seqs], 0, "right").to(dev),
                pad(labs, -100, "right").to(dev))

    def training_step(self, model, inputs, num_items_in_batch=None):
        src = None
        if self._rng.random() <= self.lmbda:
            src = model
        elif self.seq_kd:
            src = self.teacher_model
        if src is not None:
            inputs = self._prepare_inputs(inputs)
            was = model.training
            ids, am, lab = self.generate_on_policy_outputs(src, inputs)
            model.train(was)
            inputs = dict(inputs, input_ids=ids, attention_mask=am, labels=lab)
            inputs.pop("position_ids", None)
            num_items_in_batch = None  # the count of the loader's labels no longer applies
        return super().training_step(model, inputs, num_items_in_batch)

    # ---- loss --------------------------------------------------------------------------------------------------------
    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        flat, ctx, tgt = self._flat_labels(model, inputs)
        hidden = model.forward_hidden(flat, ctx)
        with torch.no_grad():
            t_hidden = self.teacher_model.forward_hidden(flat, ctx)
        sel = (tgt != -100).nonzero().flatten()
        total, per_row = chunked_token_divergence(hidden[sel], model.lm_head_weight, t_hidden[sel],
                                                  self.teacher_model.lm_head_weight, beta=self.beta,
                                                  temperature=self.temperature,
                                                  softcap=model.config.final_logit_softcapping)
        denom = num_items_in_batch if num_items_in_batch is not None else max(1, sel.numel())
        loss = total / denom
        m = self._metrics["train" if model.training else "eval"]
        n = torch.tensor(float(sel.numel()), device=flat.device)
        s = torch.stack([per_row.sum(), n])
        if D.world_size() > 1:
            D.all_reduce(s, "sum")
        m["jsd"].append(s[0] / s[1].clamp(min=1))
        if model.training:
            m["_num_tokens"].append(torch.tensor(float(flat.numel()), device=flat.device))
        return (loss, None) if return_outputs else loss
