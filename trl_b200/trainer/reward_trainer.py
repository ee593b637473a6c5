"""Outcome reward-model training (Bradley-Terry).

Behaviour of trl/trainer/reward_trainer.py: collator (:137-224, batch = [chosen..., rejected...],
optional ``margin``), over-long pairs filtered (:693-701), loss
``-logsigmoid(r_c - r_r - margin) + coef * mean((r_c + r_r)^2)`` (:739-778), metrics
``min/mean/max_reward, accuracy, margin, num_tokens``.  The model is the native decoder with a
one-logit score head read at each sequence's last token.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.nn.functional as F

from ..data_utils import _map, is_conversational, maybe_extract_prompt
from ..loop.trainer import Trainer
from ..parallel import dist as D
from .base_config import _BaseConfig
from .utils import create_model_from_path, disable_dropout_in_model, pad


@dataclass
class RewardConfig(_BaseConfig):
    _VALID_DICT_FIELDS = _BaseConfig._VALID_DICT_FIELDS + ["model_init_kwargs"]

    learning_rate: float = 1e-4
    model_init_kwargs: Optional[Any] = None
    trust_remote_code: bool = False
    chat_template_path: Optional[str] = None
    disable_dropout: bool = True
    dataset_num_proc: Optional[int] = None
    eos_token: Optional[str] = None
    pad_token: Optional[str] = None
    max_length: Optional[int] = 1024
    pad_to_multiple_of: Optional[int] = None
    center_rewards_coefficient: Optional[float] = None
    activation_offloading: bool = False


@dataclass
class DataCollatorForPreference:
    pad_token_id: int
    pad_to_multiple_of: Optional[int] = None
    return_tensors: str = "pt"

    def __call__(self, examples: list[dict[str, Any]]) -> dict[str, Any]:
        seqs = [torch.tensor(ex["chosen_ids"], dtype=torch.long) for ex in examples] + \
               [torch.tensor(ex["rejected_ids"], dtype=torch.long) for ex in examples]
        out = {"input_ids": pad(seqs, self.pad_token_id, "right", self.pad_to_multiple_of),
               "attention_mask": pad([torch.ones_like(s) for s in seqs], 0, "right", self.pad_to_multiple_of)}
        if "margin" in examples[0]:
            out["margin"] = torch.tensor([ex["margin"] for ex in examples], dtype=torch.float)
        return out

    torch_call = __call__


class RewardTrainer(Trainer):
    _tag_names = ["trl", "reward-trainer"]
    _name = "Reward"

    def __init__(self, model, args: RewardConfig | None = None, data_collator=None, train_dataset=None,
                 eval_dataset=None, processing_class=None, compute_metrics=None, callbacks=None,
                 optimizers=(None, None), peft_config=None):
        if args is None:
            name = model if isinstance(model, str) else getattr(model, "name_or_path", "model")
            args = RewardConfig(f"{os.path.basename(str(name).rstrip('/'))}-Reward")
        if isinstance(model, str):
            model_id = model
            model = create_model_from_path(model, num_labels=1, **dict(args.model_init_kwargs or {}))
        else:
            model_id = getattr(model, "name_or_path", "")
            if not getattr(model.config, "num_labels", 0):
                raise ValueError("RewardTrainer needs a model with a score head (num_labels=1)")
        if processing_class is None:
            from transformers import AutoTokenizer

            processing_class = AutoTokenizer.from_pretrained(model_id)
        tok = processing_class
        if args.eos_token is not None:
            tok.eos_token = args.eos_token
        if tok.pad_token is None:
            tok.pad_token = args.pad_token or tok.eos_token
        model.config.pad_token_id = tok.pad_token_id
        if args.chat_template_path is not None:
            with open(args.chat_template_path, encoding="utf-8") as f:
                tok.chat_template = f.read()
        if peft_config is not None:
            from ..models.lora import get_peft_model

            if not getattr(peft_config, "modules_to_save", None):
                peft_config.modules_to_save = ["score"]
            model = get_peft_model(model, peft_config)
        if args.disable_dropout:
            disable_dropout_in_model(model)
        if data_collator is None:
            data_collator = DataCollatorForPreference(tok.pad_token_id, args.pad_to_multiple_of)
        with D.main_process_first():
            if train_dataset is not None:
                train_dataset = self._prepare_dataset(train_dataset, tok, args)
            if eval_dataset is not None:
                if isinstance(eval_dataset, dict):
                    eval_dataset = {k: self._prepare_dataset(v, tok, args) for k, v in eval_dataset.items()}
                else:
                    eval_dataset = self._prepare_dataset(eval_dataset, tok, args)
        super().__init__(optimizers=optimizers, model=model, args=args, data_collator=data_collator, train_dataset=train_dataset,
                         eval_dataset=eval_dataset, processing_class=tok, compute_metrics=compute_metrics,
                         callbacks=callbacks)
        self.model_accepts_loss_kwargs = False
        self._num_tokens = 0.0

    def _prepare_given_eval_dataset(self, dataset):
        return self._prepare_dataset(dataset, self.processing_class, self.args)

    def _prepare_dataset(self, dataset, tok, args):
        first = next(iter(dataset))
        if "chosen_ids" in first:
            return dataset
        ds = dataset
        conv = is_conversational(first)
        eos = tok.eos_token

        def tokenize(ex):
            out = {}
            if conv:
                for k in ("chosen", "rejected"):
                    msgs = (ex.get("prompt") or []) + ex[k] if "prompt" in ex else ex[k]
                    ids = tok.apply_chat_template(msgs, tokenize=True, return_dict=True)["input_ids"]
                    out[f"{k}_ids"] = ids[0] if ids and isinstance(ids[0], list) else ids
            else:
                for k in ("chosen", "rejected"):
                    text = (ex.get("prompt") or "") + ex[k]
                    if not text.endswith(eos):
                        text += eos
                    out[f"{k}_ids"] = tok(text=text)["input_ids"]
            return out
        ds = _map(ds, tokenize)
        keep = {"chosen_ids", "rejected_ids", "margin"}
        if hasattr(ds, "remove_columns"):
            ds = ds.remove_columns([c for c in ds.column_names if c not in keep])
            if args.max_length is not None:
                ds = ds.filter(lambda ex: len(ex["chosen_ids"]) <= args.max_length and len(ex["rejected_ids"]) <= args.max_length)
        else:
            ds = [{k: v for k, v in r.items() if k in keep} for r in ds]
            if args.max_length is not None:
                ds = [r for r in ds if len(r["chosen_ids"]) <= args.max_length and len(r["rejected_ids"]) <= args.max_length]
        return ds

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        mode = "train" if model.training else "eval"
        out = model(input_ids=inputs["input_ids"], attention_mask=inputs["attention_mask"])
        rewards = out.logits[:, 0].float()
        rc, rr = rewards.chunk(2)
        diff = rc - rr
        if "margin" in inputs:
            diff = diff - inputs["margin"].to(diff)
        loss = -F.logsigmoid(diff).mean()
        if self.args.center_rewards_coefficient is not None:
            loss = loss + self.args.center_rewards_coefficient * torch.mean((rc + rr) ** 2)
        if out.aux_loss is not None:
            loss = loss + getattr(self.args, "router_aux_loss_coef", 0.001) * out.aux_loss
        with torch.no_grad():
            allr = D.gather(rewards.detach())
            acc = D.gather((rc > rr).float().detach())
            mar = D.gather((rc - rr).detach())
            nt = inputs["attention_mask"].sum().float().reshape(1)
            if mode == "train":
                self._num_tokens += float(D.gather(nt).sum())
            m = self._metrics[mode]
            m["num_tokens"].append(self._num_tokens)
            m["min_reward"].append(float(allr.min()))
            m["mean_reward"].append(float(allr.mean()))
            m["max_reward"].append(float(allr.max()))
            m["accuracy"].append(float(acc.mean()))
            m["margin"].append(float(mar.mean()))
        return (loss, out) if return_outputs else loss
