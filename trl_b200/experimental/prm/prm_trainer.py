"""Process reward model training (trl/experimental/prm/prm_trainer.py: tokenize_row :258-330, token-classification
loss through the model's 2-label head).

Stepwise-supervision rows ``{"prompt", "completions": [step...], "labels": [bool...]}``: every step is followed by the
separator, the label sits on the separator's last token, everything else is ignored.  The model is the native decoder
with a 2-row score head applied to every token (no shift: the label of a position is predicted from that position)."""
from __future__ import annotations

from dataclasses import dataclass
from itertools import chain
from typing import Any, Optional

import torch
import torch.nn.functional as F

from ...loop.trainer import Trainer
from ...parallel import dist as D
from ...trainer.utils import create_model_from_path, disable_dropout_in_model, pad
from .prm_config import PRMConfig


@dataclass
class DataCollatorForTokenClassification:
    pad_token_id: int
    label_pad_token_id: int = -100
    pad_to_multiple_of: Optional[int] = None

    def __call__(self, examples: list[dict[str, Any]]) -> dict[str, Any]:
        ids = [torch.tensor(e["input_ids"], dtype=torch.long) for e in examples]
        labels = [torch.tensor(e["labels"], dtype=torch.long) for e in examples]
        return {"input_ids": pad(ids, self.pad_token_id, "right", self.pad_to_multiple_of),
                "attention_mask": pad([torch.ones_like(x) for x in ids], 0, "right", self.pad_to_multiple_of),
                "labels": pad(labels, self.label_pad_token_id, "right", self.pad_to_multiple_of)}


class PRMTrainer(Trainer):
    _tag_names = ["trl", "prm"]
    _name = "PRM"

    def __init__(self, model=None, args: PRMConfig | None = None, data_collator=None, train_dataset=None,
                 eval_dataset=None, processing_class=None, compute_metrics=None, callbacks=None, peft_config=None, **kw):
        args = args or PRMConfig("model-PRM")
        if isinstance(model, str):
            model = create_model_from_path(model, num_labels=2)
        if getattr(model.config, "num_labels", 0) != 2:
            raise ValueError("PRMTrainer needs a token-classification model with num_labels=2")
        if peft_config is not None:
            from ...models.lora import get_peft_model

            model = get_peft_model(model, peft_config)
        if args.disable_dropout:
            disable_dropout_in_model(model)
        tok = processing_class
        if tok.pad_token is None:
            tok.pad_token = tok.eos_token
        if data_collator is None:
            data_collator = DataCollatorForTokenClassification(tok.pad_token_id)

        def prep(ds, is_eval):
            if ds is None or "input_ids" in next(iter(ds)):
                return ds
            return [self.tokenize_row(ex, tok, args.step_separator, args.max_length, args.max_completion_length,
                                      args.train_on_last_step_only, is_eval) for ex in ds]
        with D.main_process_first():
            train_dataset, eval_dataset = prep(train_dataset, False), prep(eval_dataset, True)
        super().__init__(model=model, args=args, data_collator=data_collator, train_dataset=train_dataset,
                         eval_dataset=eval_dataset, processing_class=tok, compute_metrics=compute_metrics,
                         callbacks=callbacks)

    @staticmethod
    def tokenize_row(features, tokenizer, step_separator, max_length, max_completion_length, train_on_last_step_only,
                     is_eval):
        prompt_ids = tokenizer(features["prompt"], add_special_tokens=False)["input_ids"]
        steps = [tokenizer(c, add_special_tokens=False)["input_ids"] for c in features["completions"]]
        if train_on_last_step_only and not is_eval:
            labels = [-100] * (len(features["labels"]) - 1) + [int(features["labels"][-1])]
        else:
            labels = [int(x) for x in features["labels"]]
        sep = tokenizer.encode(step_separator, add_special_tokens=False)
        steps = [s + sep for s in steps]
        labels = [[-100] * (len(s) - 1) + [l] for s, l in zip(steps, labels, strict=True)]
        completion_ids, labels = list(chain(*steps)), list(chain(*labels))
        if getattr(tokenizer, "bos_token_id", None) is not None:
            prompt_ids = [tokenizer.bos_token_id] + prompt_ids
        if max_completion_length is not None:
            completion_ids, labels = completion_ids[:max_completion_length], labels[:max_completion_length]
        input_ids = prompt_ids + completion_ids
        labels = [-100] * len(prompt_ids) + labels
        if max_length is not None:
            input_ids, labels = input_ids[:max_length], labels[:max_length]
        return {"input_ids": input_ids, "labels": labels}

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        ids, am, labels = inputs["input_ids"], inputs["attention_mask"], inputs["labels"]
        flat, ctx, _ = model.pack_inputs(ids, am)
        hidden = model.forward_hidden(flat, ctx)
        lab = labels.reshape(-1)[am.reshape(-1).bool()]
        sel = (lab != -100).nonzero().flatten()
        logits = hidden[sel].float() @ model.score.float().t()
        loss = F.cross_entropy(logits, lab[sel]) if sel.numel() else hidden.sum() * 0.0
        with torch.no_grad():
            s = torch.stack([(logits.argmax(-1) == lab[sel]).float().sum(), torch.tensor(float(sel.numel()), device=flat.device)])
            if D.world_size() > 1:
                D.all_reduce(s, "sum")
            self._metrics["train" if model.training else "eval"]["accuracy"].append(s[0] / s[1].clamp(min=1))
        return (loss, logits) if return_outputs else loss
