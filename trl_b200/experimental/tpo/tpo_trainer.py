"""Triple preference optimisation (trl/experimental/tpo/tpo_trainer.py: collator :78-200, loss :628-700).

Rows carry a third, gold response (``reference``): the pair loss is reference-model-free on (chosen, rejected) and
the NLL term is taken on the gold response.  Batches are ``[chosen..., rejected..., reference...]``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.nn.functional as F

from ...data_utils import is_conversational
from ...trainer.utils import pad
from .._pairwise import PairwiseTrainer
from .tpo_config import TPOConfig


@dataclass
class DataCollatorForTriplePreference:
    pad_token_id: int
    max_length: Optional[int] = None
    truncation_mode: str = "keep_start"
    pad_to_multiple_of: Optional[int] = None
    include_reference: bool = True
    return_tensors: str = "pt"

    def __call__(self, examples: list[dict[str, Any]]) -> dict[str, Any]:
        seqs, masks = [], []
        keys = ("chosen_ids", "rejected_ids", "reference_ids") if self.include_reference else ("chosen_ids", "rejected_ids")
        for key in keys:
            for ex in examples:
                ids = list(ex["prompt_ids"]) + list(ex[key])
                cm = [0] * len(ex["prompt_ids"]) + [1] * len(ex[key])
                if self.max_length is not None and len(ids) > self.max_length:
                    sl = slice(0, self.max_length) if self.truncation_mode == "keep_start" else slice(-self.max_length, None)
                    ids, cm = ids[sl], cm[sl]
                seqs.append(torch.tensor(ids, dtype=torch.long))
                masks.append(torch.tensor(cm, dtype=torch.long))
        return {"input_ids": pad(seqs, self.pad_token_id, "right", self.pad_to_multiple_of),
                "attention_mask": pad([torch.ones_like(s) for s in seqs], 0, "right", self.pad_to_multiple_of),
                "completion_mask": pad(masks, 0, "right", self.pad_to_multiple_of)}


class TPOTrainer(PairwiseTrainer):
    _tag_names = ["trl", "tpo"]
    _name = "TPO"

    def __init__(self, model, args: TPOConfig | None = None, data_collator=None, processing_class=None, **kw):
        args = args or TPOConfig("model-TPO")
        self._average_logps = args.loss_type in ("ipo", "tpo-l")
        self._branches = 3 if args.tpo_alpha != 0.0 else 2
        if data_collator is None and processing_class is not None:
            if processing_class.pad_token is None:
                processing_class.pad_token = processing_class.eos_token
            data_collator = DataCollatorForTriplePreference(processing_class.pad_token_id, args.max_length,
                                                            args.truncation_mode, args.pad_to_multiple_of,
                                                            include_reference=args.tpo_alpha != 0.0)
        super().__init__(model, args, data_collator=data_collator, processing_class=processing_class, **kw)

    def _prepare_dataset(self, dataset, tok, args, name):
        first = next(iter(dataset))
        if "prompt_ids" in first:
            return dataset
        from ...data_utils import apply_chat_template, maybe_extract_prompt

        examples = [dict(ex) for ex in dataset]
        base = super()._prepare_dataset([{k: v for k, v in ex.items() if k != "reference"} for ex in examples], tok, args,
                                        name)
        rows = []
        for b, ex in zip(base, examples):
            ref = ex["reference"]
            if isinstance(ref, list):  # conversational: render the gold completion after the (possibly implicit) prompt
                prompt = ex.get("prompt")
                if prompt is None:
                    prompt = maybe_extract_prompt({"chosen": ex["chosen"], "rejected": ex["rejected"]})["prompt"]
                    ref = ref[len(prompt):]
                text = apply_chat_template({"prompt": prompt, "completion": ref}, tok)["completion"]
            else:
                prompt = ex.get("prompt")
                if prompt is not None and ref.startswith(prompt):
                    ref = ref[len(prompt):]
                text = ref if ref.endswith(tok.eos_token) else ref + tok.eos_token
            rows.append({**dict(b), "reference_ids": tok(text=text, add_special_tokens=False)["input_ids"]})
        return rows

    def pair_loss(self, pc, pr, nll, ex, P):
        beta, ls = self.args.beta, self.args.label_smoothing
        delta = pc - pr
        if self.loss_type == "sigmoid":
            per = -F.logsigmoid(beta * delta) * (1 - ls) - F.logsigmoid(-beta * delta) * ls
        elif self.loss_type == "hinge":
            per = torch.relu(1 - beta * delta)
        elif self.loss_type == "ipo":
            per = (delta - 1 / (2 * beta)) ** 2
        else:  # tpo-l
            d = delta - self.args.tpo_l_gamma / beta
            per = -F.logsigmoid(beta * d) * (1 - ls) - F.logsigmoid(-beta * d) * ls
        if self._branches == 3:
            gold = ex["seq_id"] >= 2 * P
            gold_nll = -(ex["tok_logps"] * gold).sum() / gold.sum().clamp(min=1)
            return per, self.args.tpo_alpha * gold_nll, {"gold_nll_loss": gold_nll}
        return per, nll * 0.0, {}
