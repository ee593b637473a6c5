"""Kahneman-Tversky Optimization on unpaired preference data.

Behaviour of trl/trainer/kto_trainer.py: paired data is unpaired first, the KL estimate uses
mismatched (prompt, completion) pairs built by rotating completions by one inside every
per-device batch (:1096-1111), loss (:1552-1592)

    kl      = clamp(mean over ranks of mean(KL_logps - ref_KL_logps), min=0)      (detached)
    chosen  : 1 - sigmoid(beta * (logratio - kl))      rejected : 1 - sigmoid(beta * (kl - logratio))
    loss    = nanmean(cat(desirable_weight * chosen, undesirable_weight * rejected))

and ``apo_zero_unpaired`` (no KL term).  Sequential sampling is the default because the KL
pairs are tied to batch composition (kto_config.py:119-120).
"""
from __future__ import annotations

import copy
import os
import warnings
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.nn.functional as F

from ..data_utils import (_map, is_conversational, maybe_apply_chat_template, maybe_extract_prompt,
                          maybe_unpair_preference_dataset)
from ..loop.trainer import Trainer
from ..ops import functional as ops
from ..parallel import dist as D
from .base_config import _BaseConfig
from .utils import create_model_from_path, disable_dropout_in_model, pad, use_adapter


@dataclass
class KTOConfig(_BaseConfig):
    _VALID_DICT_FIELDS = _BaseConfig._VALID_DICT_FIELDS + ["model_init_kwargs"]
    _LOSS_TYPES = ("kto", "apo_zero_unpaired")

    learning_rate: float = 1e-6
    train_sampling_strategy: str = "sequential"
    model_init_kwargs: Optional[Any] = None
    trust_remote_code: bool = False
    disable_dropout: bool = True
    dataset_num_proc: Optional[int] = None
    max_length: Optional[int] = 1024
    pad_to_multiple_of: Optional[int] = None
    precompute_ref_log_probs: bool = False
    precompute_ref_batch_size: Optional[int] = None
    loss_type: str = "kto"
    beta: float = 0.1
    desirable_weight: float = 1.0
    undesirable_weight: float = 1.0
    activation_offloading: bool = False
    sync_ref_model: bool = False
    ref_model_mixup_alpha: float = 0.6
    ref_model_sync_steps: int = 512
    router_aux_loss_coef: float = 0.001

    def __post_init__(self):
        super().__post_init__()
        if self.loss_type not in self._LOSS_TYPES:
            raise ValueError(f"loss_type must be one of {self._LOSS_TYPES}")


@dataclass
class DataCollatorForUnpairedPreference:
    """``prompt_ids / completion_ids / label`` (+ ``KL_completion_ids``) -> padded batch with
    ``input_ids, attention_mask, completion_mask, label`` and the ``KL_*`` twins."""

    pad_token_id: int
    max_length: Optional[int] = None
    pad_to_multiple_of: Optional[int] = None

    def _build(self, examples, key):
        seqs, masks = [], []
        for ex in examples:
            ids = list(ex["prompt_ids"]) + list(ex[key])
            cm = [0] * len(ex["prompt_ids"]) + [1] * len(ex[key])
            if self.max_length is not None:
                ids, cm = ids[:self.max_length], cm[:self.max_length]
            seqs.append(torch.tensor(ids, dtype=torch.long))
            masks.append(torch.tensor(cm, dtype=torch.long))
        return (pad(seqs, self.pad_token_id, "right", self.pad_to_multiple_of),
                pad([torch.ones_like(s) for s in seqs], 0, "right", self.pad_to_multiple_of),
                pad(masks, 0, "right", self.pad_to_multiple_of))

    def __call__(self, examples: list[dict[str, Any]]) -> dict[str, Any]:
        ids, am, cm = self._build(examples, "completion_ids")
        out = {"input_ids": ids, "attention_mask": am, "completion_mask": cm,
               "label": torch.tensor([bool(ex["label"]) for ex in examples])}
        if "KL_completion_ids" in examples[0]:
            kids, kam, kcm = self._build(examples, "KL_completion_ids")
            out.update(KL_input_ids=kids, KL_attention_mask=kam, KL_completion_mask=kcm)
        for k in ("ref_logps", "ref_KL_logps"):
            if k in examples[0]:
                out[k] = torch.tensor([ex[k] for ex in examples])
        return out


class KTOTrainer(Trainer):
    _tag_names = ["trl", "kto"]
    _name = "KTO"

    def __init__(self, model, ref_model=None, args: KTOConfig | None = None, train_dataset=None, eval_dataset=None,
                 processing_class=None, data_collator=None, callbacks=None, optimizers=(None, None), peft_config=None,
                 compute_metrics=None):
        if args is None:
            name = model if isinstance(model, str) else getattr(model, "name_or_path", "model")
            args = KTOConfig(f"{os.path.basename(str(name).rstrip('/'))}-KTO")
        if isinstance(model, str):
            model_id = model
            model = create_model_from_path(model, **dict(args.model_init_kwargs or {}))
        else:
            model_id = getattr(model, "name_or_path", "")
        if isinstance(ref_model, str):
            ref_model = create_model_from_path(ref_model, **dict(args.model_init_kwargs or {}))
        if processing_class is None:
            from transformers import AutoTokenizer

            processing_class = AutoTokenizer.from_pretrained(model_id)
        tok = processing_class
        if tok.pad_token is None:
            tok.pad_token = tok.eos_token
        if peft_config is not None:
            from ..models.lora import get_peft_model

            model = get_peft_model(model, peft_config)
        if args.disable_dropout:
            disable_dropout_in_model(model)
        self.loss_type, self.beta = args.loss_type, args.beta
        self.desirable_weight, self.undesirable_weight = args.desirable_weight, args.undesirable_weight
        self.calculate_KL = self.loss_type == "kto"
        if self.calculate_KL:
            if args.train_sampling_strategy != "sequential":
                raise ValueError("loss_type='kto' estimates the KL from batch-mates: train_sampling_strategy must be "
                                 "'sequential'")
            if args.per_device_train_batch_size <= 1:
                raise ValueError("Actual (not effective) batch size must be > 1. KTO will not work properly because the "
                                 "KL term will be equivalent to the implied reward.")
        if data_collator is None:
            data_collator = DataCollatorForUnpairedPreference(tok.pad_token_id, args.max_length, args.pad_to_multiple_of)
        with D.main_process_first():
            if train_dataset is not None:
                train_dataset = self._prepare_dataset(train_dataset, tok, args, args.per_device_train_batch_size, True)
            if isinstance(eval_dataset, dict):
                eval_dataset = {k: self._prepare_dataset(v, tok, args, args.per_device_eval_batch_size, False)
                                for k, v in eval_dataset.items()}
            elif eval_dataset is not None:
                eval_dataset = self._prepare_dataset(eval_dataset, tok, args, args.per_device_eval_batch_size, False)
        super().__init__(optimizers=optimizers, model=model, args=args, data_collator=data_collator, train_dataset=train_dataset,
                         eval_dataset=eval_dataset, processing_class=tok, callbacks=callbacks,
                         compute_metrics=compute_metrics)
        self.model_accepts_loss_kwargs = False
        self._ref_adapter_off = False
        if ref_model is not None:
            self.ref_model = ref_model.to(self.args.device, dtype=self.model.dtype).eval().requires_grad_(False)
        elif getattr(self.model, "peft_config", None) is not None:
            self.ref_model, self._ref_adapter_off = None, True
        elif args.precompute_ref_log_probs:
            self.ref_model = None  # the policy before training is the reference; its log-probs are computed below
        else:
            self.ref_model = copy.deepcopy(self.model).eval().requires_grad_(False)
        self.precompute_ref_log_probs = args.precompute_ref_log_probs
        if self.precompute_ref_log_probs:  # the reference is evaluated once over the datasets, before any update
            if args.sync_ref_model:
                raise ValueError("sync_ref_model and precompute_ref_log_probs cannot both be enabled")
            self.train_dataset = self._precompute_ref_logps(self.train_dataset, args.per_device_train_batch_size)
            if isinstance(self.eval_dataset, dict):
                self.eval_dataset = {k: self._precompute_ref_logps(v, args.per_device_eval_batch_size)
                                     for k, v in self.eval_dataset.items()}
            elif self.eval_dataset is not None:
                self.eval_dataset = self._precompute_ref_logps(self.eval_dataset, args.per_device_eval_batch_size)
        if args.sync_ref_model and self.ref_model is not None:
            from .callbacks import SyncRefModelCallback

            self.add_callback(SyncRefModelCallback(ref_model=self.ref_model))
        self._num_tokens = 0.0

    def _prepare_given_eval_dataset(self, dataset):
        ds = self._prepare_dataset(dataset, self.processing_class, self.args, self.args.per_device_eval_batch_size, False)
        if self.precompute_ref_log_probs and "ref_logps" not in next(iter(ds)):
            if self.ref_model is None and not self._ref_adapter_off and self.state.global_step > 0:
                raise ValueError("Cannot compute reference log-probs for a dataset passed to `evaluate()` after training "
                                 "has started: with `precompute_ref_log_probs=True` and no `ref_model` the reference is the "
                                 "policy before training.")
            ds = self._precompute_ref_logps(ds, self.args.per_device_eval_batch_size)
        return ds

    def _precompute_ref_logps(self, dataset, batch_size):
        """Adds ``ref_logps`` (and ``ref_KL_logps`` for the KL estimate) computed with the reference model in batches of
        ``batch_size`` rows, the rows in dataset order so the KL rotation stays inside its batch
        (kto_trainer.py ``precompute_ref_log_probs``)."""
        if dataset is None or not hasattr(dataset, "__len__"):
            raise ValueError("precompute_ref_log_probs needs a map-style dataset (its length must be known)")
        ref = self.ref_model if self.ref_model is not None else self.model
        was_training = ref.training
        ref.eval()
        rows = [dataset[i] for i in range(len(dataset))]
        lps, kls = [], []
        with torch.no_grad():
            for s in range(0, len(rows), batch_size):
                b = self._prepare_inputs(self.data_collator(rows[s:s + batch_size]))
                lp, _, _ = self._seq_logps(ref, b["input_ids"], b["attention_mask"], b["completion_mask"],
                                           adapter_off=self._ref_adapter_off)
                lps.append(lp.float().cpu())
                if self.calculate_KL and "KL_input_ids" in b:
                    kl, _, _ = self._seq_logps(ref, b["KL_input_ids"], b["KL_attention_mask"], b["KL_completion_mask"],
                                               adapter_off=self._ref_adapter_off)
                    kls.append(kl.float().cpu())
        ref.train(was_training)
        cols = {"ref_logps": torch.cat(lps).tolist()}
        if kls:
            cols["ref_KL_logps"] = torch.cat(kls).tolist()
        if hasattr(dataset, "add_column"):
            for k, v in cols.items():
                dataset = dataset.add_column(k, v)
            return dataset
        return [{**r, **{k: v[i] for k, v in cols.items()}} for i, r in enumerate(rows)]

    def _prepare_dataset(self, dataset, tok, args, batch_size, is_train):
        first = next(iter(dataset))
        if "prompt_ids" in first:
            ds = dataset
        else:
            ds = _map(dataset, maybe_extract_prompt) if "chosen" in first else dataset
            ds = maybe_unpair_preference_dataset(ds)
            conv = is_conversational(next(iter(ds)))
            ds = _map(ds, lambda ex: maybe_apply_chat_template(
                {k: ex[k] for k in ("prompt", "completion", "label") if k in ex}, tok))
            eos = tok.eos_token

            def tokenize(ex):
                comp = ex["completion"]
                if not conv and not comp.endswith(eos):
                    comp = comp + eos
                return {"prompt_ids": tok(text=ex["prompt"], add_special_tokens=not conv)["input_ids"],
                        "completion_ids": tok(text=comp, add_special_tokens=False)["input_ids"]}
            ds = _map(ds, tokenize)
            keep = {"prompt_ids", "completion_ids", "label"}
            if hasattr(ds, "remove_columns"):
                ds = ds.remove_columns([c for c in ds.column_names if c not in keep])
            else:
                ds = [{k: v for k, v in r.items() if k in keep} for r in ds]
        if args.max_length is not None:
            if hasattr(ds, "filter"):
                ds = ds.filter(lambda ex: len(ex["prompt_ids"]) < args.max_length)
            else:
                ds = [r for r in ds if len(r["prompt_ids"]) < args.max_length]
        if self.calculate_KL and "KL_completion_ids" not in next(iter(ds)):
            rows = [dict(r) for r in ds]
            for s in range(0, len(rows), batch_size):
                chunk = rows[s:s + batch_size]
                comps = [r["completion_ids"] for r in chunk]
                rot = [comps[-1]] + comps[:-1]
                for r, k in zip(chunk, rot):
                    r["KL_completion_ids"] = k
            try:
                from datasets import Dataset

                ds = Dataset.from_list(rows) if hasattr(ds, "column_names") else rows
            except Exception:
                ds = rows
        if is_train:
            labels = [bool(r["label"]) for r in ds]
            nd, nu = sum(labels), len(labels) - sum(labels)
            if nd and nu and nd != nu:
                des_lo, des_hi = round(nu * self.undesirable_weight / nd * 1, 2), round(nu * self.undesirable_weight / nd * 1.33, 2)
                und_lo, und_hi = round(nd * self.desirable_weight / nu / 1.33, 2), round(nd * self.desirable_weight / nu / 1, 2)
                if not (des_lo <= self.desirable_weight <= des_hi or und_lo <= self.undesirable_weight <= und_hi):
                    warnings.warn(
                        "You have different amounts of desirable/positive and undesirable/negative examples but the weights "
                        f"on the desirable and undesirable losses don't seem to be in an ideal range. Based on your data, we "
                        f"recommend EITHER desirable_weight in [{des_lo}, {des_hi}] or undesirable_weight in "
                        f"[{und_lo}, {und_hi}] (but NOT BOTH).", UserWarning)
        return ds

    def _seq_logps(self, model, ids, am, cm, need_entropy=False, adapter_off=False):
        flat, ctx, _ = model.pack_inputs(ids, am)
        mflat = am.reshape(-1).bool()
        tgt = torch.zeros_like(ids)
        tgt[:, :-1] = ids[:, 1:]
        pred = torch.zeros_like(cm)
        pred[:, :-1] = cm[:, 1:] * am[:, 1:]
        tgt_f, pred_f = tgt.reshape(-1)[mflat], pred.reshape(-1)[mflat].bool()
        if adapter_off:
            with use_adapter(model, None):
                hidden = model.forward_hidden(flat, ctx)
        else:
            hidden = model.forward_hidden(flat, ctx)
        sel = pred_f.nonzero().flatten()
        lp, ent = ops.lm_head_logprobs(hidden[sel], model.lm_head_weight, tgt_f[sel], 1.0, compute_entropy=need_entropy)
        seq_id = torch.repeat_interleave(torch.arange(ids.shape[0], device=ids.device), am.sum(1))[sel]
        out = torch.zeros(ids.shape[0], device=ids.device, dtype=lp.dtype).index_add(0, seq_id, lp)
        return out, ent, model.aux_loss(ctx) if getattr(model.config, "is_moe", False) and torch.is_grad_enabled() else None

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        mode = "train" if model.training else "eval"
        m = self._metrics[mode]
        label = inputs["label"].bool()
        logps, ent, aux = self._seq_logps(model, inputs["input_ids"], inputs["attention_mask"], inputs["completion_mask"],
                                          need_entropy=True)
        ref = self.ref_model if self.ref_model is not None else model
        with torch.no_grad():
            if "ref_logps" in inputs:
                ref_logps = inputs["ref_logps"].to(logps)
            else:
                ref_logps, _, _ = self._seq_logps(ref, inputs["input_ids"], inputs["attention_mask"],
                                                  inputs["completion_mask"], adapter_off=self._ref_adapter_off)
            if self.calculate_KL and "KL_input_ids" in inputs:
                kl_lp, _, _ = self._seq_logps(model, inputs["KL_input_ids"], inputs["KL_attention_mask"],
                                              inputs["KL_completion_mask"])
                if "ref_KL_logps" in inputs:
                    ref_kl = inputs["ref_KL_logps"].to(kl_lp)
                else:
                    ref_kl, _, _ = self._seq_logps(ref, inputs["KL_input_ids"], inputs["KL_attention_mask"],
                                                   inputs["KL_completion_mask"], adapter_off=self._ref_adapter_off)
                kl = (kl_lp - ref_kl).mean().detach()
                kl = D.gather(kl.reshape(1)).mean().clamp(min=0)
            else:
                kl = torch.zeros((), device=logps.device)
        logratio = logps - ref_logps
        c_lr, r_lr = logratio[label], logratio[~label]
        c_loss, r_loss = self._unpaired_losses(c_lr, r_lr, kl, mode)
        losses = torch.cat([self.desirable_weight * c_loss, self.undesirable_weight * r_loss], 0)
        loss = losses.nanmean() if losses.numel() else (logps.sum() * 0.0)
        if aux is not None:
            loss = loss + self.args.router_aux_loss_coef * aux
        with torch.no_grad():
            lf = label.float()
            s = torch.stack([(self.beta * logratio.detach() * lf).sum(), lf.sum(),
                             (self.beta * logratio.detach() * (1 - lf)).sum(), (1 - lf).sum(),
                             (logps.detach() * lf).sum(), (logps.detach() * (1 - lf)).sum(),
                             ent.sum(), torch.tensor(float(ent.numel()), device=ent.device),
                             inputs["attention_mask"].sum().float()])
            if D.world_size() > 1:
                D.all_reduce(s, "sum")
            if s[1] > 0:
                m["rewards/chosen"].append(float(s[0] / s[1]))
                m["logps/chosen"].append(float(s[4] / s[1]))
            if s[3] > 0:
                m["rewards/rejected"].append(float(s[2] / s[3]))
                m["logps/rejected"].append(float(s[5] / s[3]))
            if s[1] > 0 and s[3] > 0:
                m["rewards/margins"].append(float(s[0] / s[1] - s[2] / s[3]))
            m["kl"].append(float(kl))
            m["entropy"].append(float(s[6] / s[7].clamp(min=1)))
            if mode == "train":
                self._num_tokens += float(s[8])
            m["num_tokens"].append(self._num_tokens)
        return (loss, None) if return_outputs else loss

    def _unpaired_losses(self, c_lr, r_lr, kl, mode):
        """Per-example losses of the desirable / undesirable completions from their policy-vs-reference log-ratios."""
        if self.loss_type == "kto":
            return 1 - torch.sigmoid(self.beta * (c_lr - kl)), 1 - torch.sigmoid(self.beta * (kl - r_lr))
        return 1 - torch.sigmoid(self.beta * c_lr), torch.sigmoid(self.beta * r_lr)

    def prediction_step(self, model, inputs, prediction_loss_only=True, ignore_keys=None):
        inputs = self._prepare_inputs(inputs)
        with torch.no_grad():
            loss = self.compute_loss(model, inputs)
        return loss.detach(), None, None
