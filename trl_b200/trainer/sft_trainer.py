"""Supervised fine-tuning.

API and behaviour follow trl/trainer/sft_trainer.py (collator :394-534, dataset
preparation :1375-1625, loss/metrics :1700-1832).  The forward is always
padding-free inside the model; the loss is the fused lm-head + cross-entropy op
(`ops.lm_head_ce`), so `chunked_nll` and `nll` are the same kernel here and no
``[tokens, vocab]`` logits tensor exists.
"""
from __future__ import annotations

import os
import warnings
from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

from ..data_utils import (is_conversational, is_conversational_from_value, maybe_convert_to_chatml, pack_dataset,
                          _map, _tokenize, get_dataset_column_names)
from ..loop.trainer import Trainer
from ..ops import functional as ops
from ..parallel import dist as D
from .sft_config import SFTConfig
from .utils import create_model_from_path, pad


@dataclass
class DataCollatorForLanguageModeling:
    """Pads to the longest row, or with ``padding_free`` flattens the batch into one row whose
    ``position_ids`` restart at every document (and ``labels`` are ``-100`` at document starts)."""

    pad_token_id: int
    completion_only_loss: bool = True
    padding_free: bool = False
    pad_to_multiple_of: Optional[int] = None
    return_tensors: str = "pt"

    def __call__(self, examples: list[dict[str, Any]]) -> dict[str, Any]:
        ids = [torch.as_tensor(e["input_ids"], dtype=torch.long) for e in examples]
        labels = [torch.as_tensor(e.get("labels", e["input_ids"]), dtype=torch.long).clone() for e in examples]
        given = "labels" in examples[0]  # labels that come with the rows are final: mask columns beside them are ignored
        if not given and self.completion_only_loss and "completion_mask" in examples[0]:
            for l, e in zip(labels, examples):
                l[torch.as_tensor(e["completion_mask"]) == 0] = -100
        if not given and "assistant_masks" in examples[0]:
            for l, e in zip(labels, examples):
                l[torch.as_tensor(e["assistant_masks"]) == 0] = -100
        out = {}
        if self.padding_free:
            if "seq_lengths" in examples[0]:
                pos = self.get_position_ids_from_packed_seq_lengths([e["seq_lengths"] for e in examples])
            else:
                pos = [torch.arange(len(x)) for x in ids]
            ids, labels, pos = [torch.cat(ids)], [torch.cat(labels)], [torch.cat(pos)]
        out["input_ids"] = pad(ids, self.pad_token_id, "right", self.pad_to_multiple_of)
        out["labels"] = pad(labels, -100, "right", self.pad_to_multiple_of)
        if self.padding_free:
            out["position_ids"] = pad(pos, 0, "right", self.pad_to_multiple_of)
            out["labels"][out["position_ids"] == 0] = -100
        else:
            out["attention_mask"] = pad([torch.ones_like(x) for x in ids], 0, "right", self.pad_to_multiple_of)
        return out

    torch_call = __call__

    @staticmethod
    def get_position_ids_from_packed_seq_lengths(batch_seq_lengths: list[list[int]]) -> list[torch.Tensor]:
        return [torch.cat([torch.arange(int(n)) for n in lens]) for lens in batch_seq_lengths]


class DataCollatorForVisionLanguageModeling:
    """Tokenises text and converts images on the fly, batch by batch (image conversion is too heavy to do for the
    whole dataset up front).  Examples carry ``images`` (list) or ``image`` plus either ``messages`` / a text field
    (language modelling) or ``prompt`` + ``completion``.  Output: ``input_ids``, ``attention_mask``, ``pixel_values``,
    ``labels`` (padding masked; with ``completion_only_loss`` the prompt too) and whatever else the processor returns.
    ``processor`` is a transformers ``ProcessorMixin`` or ``models.vision_processing.VisionProcessor``
    (trl/trainer/sft_trainer.py:538-760)."""

    def __init__(self, processor, max_length: int | None = None, completion_only_loss: bool = False,
                 pad_to_multiple_of: int | None = None, dataset_text_field: str = "text", return_tensors: str = "pt"):
        self.processor = processor
        self.max_length = max_length
        self.completion_only_loss = completion_only_loss
        self.pad_to_multiple_of = pad_to_multiple_of
        self.dataset_text_field = dataset_text_field
        self.return_tensors = return_tensors

    @staticmethod
    def _images(examples):
        examples = [dict(e) for e in examples]
        for e in examples:
            if "image" in e:
                e["images"] = [e.pop("image")]
            e.setdefault("images", [])
        imgs = [list(e["images"]) for e in examples]
        return examples, (None if all(not i for i in imgs) else imgs)  # processors reject an all-empty image batch

    def __call__(self, examples):
        first = examples[0]
        if "messages" in first or self.dataset_text_field in first:
            if self.completion_only_loss:
                raise ValueError("The `completion_only_loss` argument is not supported for language modeling datasets.")
            return self._language_modeling(examples)
        if "prompt" in first and "completion" in first:
            return self._prompt_completion(examples)
        raise KeyError(f"Unexpected input keys in examples: {list(first.keys())}.")

    torch_call = __call__

    def _language_modeling(self, examples):
        from ..data_utils import prepare_multimodal_messages

        examples, images = self._images(examples)
        if "messages" in examples[0]:
            msgs = [prepare_multimodal_messages(e["messages"], images=e["images"]) for e in examples]
            texts = self.processor.apply_chat_template(msgs, tokenize=False)
        else:
            texts = [e[self.dataset_text_field] for e in examples]
        out = dict(self.processor(images=images, text=texts, padding=True, padding_side="right",
                                  pad_to_multiple_of=self.pad_to_multiple_of, truncation=self.max_length is not None,
                                  max_length=self.max_length, return_tensors=self.return_tensors,
                                  add_special_tokens=False))
        labels = out["input_ids"].clone()
        labels[out["attention_mask"] == 0] = -100
        out["labels"] = labels
        return out

    def _prompt_completion(self, examples):
        from ..data_utils import apply_chat_template, is_conversational, prepare_multimodal_messages
        from .utils import flush_left

        if self.pad_to_multiple_of is not None:
            raise NotImplementedError("Padding to a multiple of a value is not yet implemented for vision-language "
                                      "modeling and prompt-completion data.")
        examples, images = self._images(examples)
        if is_conversational(examples[0]):
            rendered = []
            for e in examples:
                e = {**e, "prompt": prepare_multimodal_messages(e["prompt"], images=e["images"]),
                     "completion": prepare_multimodal_messages(e["completion"])}
                rendered.append(apply_chat_template({k: e[k] for k in ("prompt", "completion")}, self.processor))
            examples = rendered
        kw = dict(return_tensors=self.return_tensors, add_special_tokens=False, padding=True)
        pp = self.processor(images=images, text=[e["prompt"] for e in examples], padding_side="left", **kw)
        pc = self.processor(text=[e["completion"] for e in examples], padding_side="right", **kw)
        ids = torch.cat([pp["input_ids"], pc["input_ids"]], dim=1)
        am = torch.cat([pp["attention_mask"], pc["attention_mask"]], dim=1)
        cm = torch.cat([torch.zeros_like(pp["attention_mask"]), pc["attention_mask"]], dim=1)
        extras = {}
        for k in ("token_type_ids", "mm_token_type_ids"):
            if k in pp:
                tail = pc[k] if k in pc else torch.zeros_like(pc["input_ids"])
                extras[k] = torch.cat([pp[k], tail], dim=1)
        am, ids, cm, *rest = flush_left(am, ids, cm, *extras.values())
        extras = dict(zip(extras.keys(), rest))
        if self.max_length is not None:
            ids, am, cm = ids[:, :self.max_length], am[:, :self.max_length], cm[:, :self.max_length]
            extras = {k: v[:, :self.max_length] for k, v in extras.items()}
        labels = ids.clone()
        labels[am == 0] = -100
        if self.completion_only_loss:
            labels[cm == 0] = -100
        out = {k: v for k, v in pp.items() if k not in ("input_ids", "attention_mask", "token_type_ids", "mm_token_type_ids")}
        out.update(input_ids=ids, attention_mask=am, labels=labels, **extras)
        return out


def dft_loss(logp: torch.Tensor, valid: torch.Tensor, num_items_in_batch=None) -> torch.Tensor:
    """Dynamic fine-tuning: ``-stopgrad(p_y) * log p_y`` (sft_trainer.py:773-787)."""
    per_tok = -(logp.detach().exp() * logp) * valid
    denom = num_items_in_batch if num_items_in_batch is not None else valid.sum().clamp_min(1)
    return per_tok.sum() / denom


def shift_labels_flat(labels: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Next-token targets on a flat packed stream: position t predicts t+1 unless t+1 starts a document."""
    nxt = torch.full_like(labels, -100)
    nxt[:-1] = labels[1:]
    starts_next = torch.ones_like(positions, dtype=torch.bool)
    starts_next[:-1] = positions[1:] == 0
    nxt[starts_next] = -100
    return nxt


class SFTTrainer(Trainer):
    _tag_names = ["trl", "sft"]
    _name = "SFT"

    def __init__(self, model, args: SFTConfig | None = None, data_collator=None, train_dataset=None, eval_dataset=None,
                 processing_class=None, compute_loss_func=None, compute_metrics=None, callbacks=None,
                 optimizers=(None, None), optimizer_cls_and_kwargs=None, preprocess_logits_for_metrics=None,
                 peft_config=None, formatting_func: Callable | None = None):
        if args is None:
            name = model if isinstance(model, str) else getattr(model, "name_or_path", "model")
            args = SFTConfig(f"{os.path.basename(str(name).rstrip('/'))}-SFT")
        if isinstance(model, str):
            model_id = model
            kw = dict(args.model_init_kwargs or {})
            model = create_model_from_path(model, **kw)
        else:
            model_id = getattr(model, "name_or_path", "")
            if args.model_init_kwargs is not None:
                warnings.warn("model_init_kwargs is ignored when the model is already instantiated.")
        if processing_class is None:
            from transformers import AutoTokenizer

            if not os.path.isdir(model_id):
                raise ValueError("processing_class is required when the model is not a local checkpoint directory")
            processing_class = AutoTokenizer.from_pretrained(model_id)
        # a processor (vision-language models) wraps the text tokenizer
        tok = getattr(processing_class, "tokenizer", processing_class)
        if args.eos_token is not None:
            if tok.convert_tokens_to_ids(args.eos_token) is None:
                raise ValueError(f"eos_token {args.eos_token!r} is not in the vocabulary")
            tok.eos_token = args.eos_token
        if args.chat_template_path is not None:
            if os.path.isfile(args.chat_template_path) and args.chat_template_path.endswith((".jinja", ".j2")):
                with open(args.chat_template_path, encoding="utf-8") as f:
                    tok.chat_template = f.read()
            else:
                from ..chat_template_utils import clone_chat_template

                model, tok, _ = clone_chat_template(model, tok, args.chat_template_path)
        if tok.pad_token is None:
            tok.pad_token = args.pad_token or tok.eos_token
        if peft_config is not None:
            from ..models.lora import get_peft_model

            model = get_peft_model(model, peft_config)
        self.padding_free = args.padding_free or (args.packing and args.packing_strategy in ("bfd", "bfd_split"))
        first = next(iter(train_dataset)) if train_dataset is not None else {}
        self._is_vlm = "images" in first or "image" in first
        if args.completion_only_loss is None:
            self.completion_only_loss = "prompt" in first and "completion" in first or "completion_mask" in first
        else:
            self.completion_only_loss = args.completion_only_loss
        if data_collator is None:
            if self._is_vlm:
                if not hasattr(processing_class, "tokenizer"):
                    raise ValueError("a dataset with images needs a processor (image processor + tokenizer) as "
                                     "processing_class, e.g. models.vision_processing.VisionProcessor")
                if self.padding_free or args.packing:
                    raise ValueError("packing / padding_free are not supported for vision-language datasets")
                data_collator = DataCollatorForVisionLanguageModeling(
                    processing_class, max_length=args.max_length, completion_only_loss=bool(self.completion_only_loss),
                    pad_to_multiple_of=args.pad_to_multiple_of, dataset_text_field=args.dataset_text_field)
                args.remove_unused_columns = False  # the collator reads the raw columns
            else:
                data_collator = DataCollatorForLanguageModeling(tok.pad_token_id, self.completion_only_loss,
                                                                self.padding_free, args.pad_to_multiple_of)
        if args.packing and args.packing_strategy == "wrapped" and args.padding_free:
            warnings.warn("'wrapped' packing has no document boundaries: padding_free has no effect on attention.")
        skip = (args.dataset_kwargs or {}).get("skip_prepare_dataset", False) or self._is_vlm
        self._skip_prepare, self._formatting_func = skip, formatting_func
        if not skip:
            with D.main_process_first():
                if train_dataset is not None:
                    train_dataset = self._prepare_dataset(train_dataset, tok, args, args.packing, formatting_func, "train")
                if eval_dataset is not None:
                    ep = args.packing if args.eval_packing is None else args.eval_packing
                    if isinstance(eval_dataset, dict):
                        eval_dataset = {k: self._prepare_dataset(v, tok, args, ep, formatting_func, k) for k, v in eval_dataset.items()}
                    else:
                        eval_dataset = self._prepare_dataset(eval_dataset, tok, args, ep, formatting_func, "eval")
        self._total_train_tokens = 0
        self.aux_loss_enabled = getattr(getattr(model, "config", None), "is_moe", False)
        super().__init__(optimizers=optimizers, optimizer_cls_and_kwargs=optimizer_cls_and_kwargs, model=model, args=args, data_collator=data_collator, train_dataset=train_dataset,
                         eval_dataset=eval_dataset, processing_class=processing_class if self._is_vlm else tok,
                         compute_loss_func=compute_loss_func,
                         compute_metrics=compute_metrics, callbacks=callbacks,
                         preprocess_logits_for_metrics=preprocess_logits_for_metrics)
        self.model_accepts_loss_kwargs = True
        if args.activation_offloading:
            from ..models.activation_offloading import get_act_offloading_ctx_manager

            self.maybe_activation_offload_context = get_act_offloading_ctx_manager(self.model)
            self._own_offload_scope = True  # compute_loss wraps the decoder forward itself
        else:
            import contextlib

            self.maybe_activation_offload_context = contextlib.nullcontext()

    # ---- dataset ---------------------------------------------------------------------------------
    def _prepare_given_eval_dataset(self, dataset):
        if self._skip_prepare:
            return dataset
        a = self.args
        tok = getattr(self.processing_class, "tokenizer", self.processing_class)
        return self._prepare_dataset(dataset, tok, a, a.packing if a.eval_packing is None else a.eval_packing,
                                     self._formatting_func, "eval")

    def _prepare_dataset(self, dataset, tok, args: SFTConfig, packing: bool, formatting_func, name: str):
        fmt = getattr(dataset, "format", None)
        if isinstance(fmt, dict) and fmt.get("type") == "custom":
            # map() would read through the transform and freeze a random or stateful transform into the token columns
            raise ValueError("SFTTrainer cannot prepare a dataset that uses `Dataset.with_transform()`. Pass "
                             "`dataset_kwargs={'skip_prepare_dataset': True}` and make the transform return trainer-ready "
                             "examples (tokenized fields included), or materialize the transform with `Dataset.map()`.")
        cols = get_dataset_column_names(dataset)
        first = next(iter(dataset))
        if "input_ids" in cols:  # already tokenised
            ds = dataset
        else:
            ds = dataset
            if formatting_func is not None:
                ds = _map(ds, lambda ex: {"text": formatting_func(ex)})
                first = next(iter(ds))
            if is_conversational_from_value(first):
                ds = _map(ds, maybe_convert_to_chatml, remove_columns=["conversations"] if "conversations" in cols else None)
                first = next(iter(ds))
            conv = is_conversational(first)
            if not conv:  # append EOS to plain-text examples
                eos = tok.eos_token

                def add_eos(ex):
                    out = {}
                    for k in ("text", "completion"):
                        if k in ex and not ("text" == k and "completion" in ex) and not ex[k].endswith(eos):
                            out[k] = ex[k] + eos
                    return out
                tf = args.dataset_text_field
                if tf != "text" and tf in cols:
                    ds = _map(ds, lambda ex: {"text": ex[tf]})
                ds = _map(ds, add_eos)

            def tokenize(ex):
                tools = ex.get("tools")
                ckw = ex.get("chat_template_kwargs") or {}
                if "prompt" in ex:
                    if is_conversational(ex):
                        p_ids = _tokenize(tok, ex["prompt"], tools=tools, add_generation_prompt=True, **ckw)["input_ids"]
                        full = _tokenize(tok, ex["prompt"] + ex["completion"], tools=tools,
                                         return_assistant_tokens_mask=args.assistant_only_loss, **ckw)
                    else:
                        p_ids = _tokenize(tok, ex["prompt"])["input_ids"]
                        full = _tokenize(tok, ex["prompt"] + ex["completion"])
                    ids = full["input_ids"]
                    if ids[:len(p_ids)] != p_ids:
                        warnings.warn("Mismatch between tokenized prompt and the start of tokenized prompt+completion.")
                    out = {"input_ids": ids, "completion_mask": [0] * len(p_ids) + [1] * (len(ids) - len(p_ids))}
                    if "assistant_masks" in full:
                        out["assistant_masks"] = full["assistant_masks"]
                    return out
                if is_conversational(ex):
                    full = _tokenize(tok, ex["messages"], tools=tools, return_assistant_tokens_mask=args.assistant_only_loss, **ckw)
                    out = {"input_ids": full["input_ids"]}
                    if "assistant_masks" in full:
                        if 1 not in full["assistant_masks"]:
                            raise RuntimeError("assistant_only_loss=True but the chat template marks no assistant tokens "
                                               "({% generation %} block missing).")
                        out["assistant_masks"] = full["assistant_masks"]
                    return out
                return {"input_ids": _tokenize(tok, ex["text"])["input_ids"]}
            ds = _map(ds, tokenize)
        keep = [c for c in ("input_ids", "completion_mask", "assistant_masks", "labels", "seq_lengths")
                if c in get_dataset_column_names(ds)]
        drop = [c for c in get_dataset_column_names(ds) if c not in keep]
        if drop and hasattr(ds, "remove_columns"):
            ds = ds.remove_columns(drop)
        elif drop:
            ds = [{k: r[k] for k in keep} for r in ds]
        if args.max_length is not None and not (packing and args.packing_strategy != "wrapped"):
            ml = args.max_length

            def trunc(ex):
                sl = slice(0, ml) if args.truncation_mode == "keep_start" else slice(-ml, None)
                return {k: ex[k][sl] for k in keep if k != "seq_lengths"}
            ds = _map(ds, trunc)
        if packing:
            if args.max_length is None:
                raise ValueError("packing requires max_length")
            sel = [c for c in ("input_ids", "completion_mask", "assistant_masks") if c in keep]
            if hasattr(ds, "select_columns"):
                ds = ds.select_columns(sel)
            ds = pack_dataset(ds, args.max_length, args.packing_strategy)
        if args.shuffle_dataset and hasattr(ds, "shuffle"):
            ds = ds.shuffle(seed=args.seed)
        return ds

    # ---- loss --------------------------------------------------------------------------------------
    def _flat_labels(self, model, inputs):
        """(flat_ids, ctx, shifted flat labels) for either batch layout."""
        ids, labels = inputs["input_ids"], inputs.get("shift_labels")
        am, pos = inputs.get("attention_mask"), inputs.get("position_ids")
        flat, ctx, _ = model.pack_inputs(ids, am, pos)
        if labels is not None:  # pre-shifted by a sequence-parallel loader
            tgt = labels
        else:
            lab = inputs["labels"]
            tgt = torch.full_like(lab, -100)
            tgt[:, :-1] = lab[:, 1:]
        if am is not None and not bool(am.all()):
            tgt = tgt.reshape(-1)[am.reshape(-1).bool()]
        else:
            tgt = tgt.reshape(-1)
            if pos is not None:
                nxt_start = torch.ones_like(ctx.positions, dtype=torch.bool)
                nxt_start[:-1] = ctx.positions[1:] == 0
                tgt = tgt.masked_fill(nxt_start, -100)
        return flat, ctx, tgt

    def loss_from_hidden(self, model, hidden, ctx, targets, num_items_in_batch=None):
        a = self.args
        mode = "train" if model.training else "eval"
        W = model.lm_head_weight
        valid = targets != -100
        if a.loss_type == "dft":
            logp, ent = ops.lm_head_logprobs(hidden, W, targets.clamp_min(0), compute_entropy=True)
            n_valid = valid.sum()
            denom = num_items_in_batch if num_items_in_batch is not None else n_valid.clamp_min(1)
            loss = dft_loss(logp, valid, denom)
            ent_sum = (ent * valid).sum()
            correct = None
        else:
            loss_sum, correct, ent_sum, n_valid = ops.lm_head_ce(hidden, W, targets)
            denom = num_items_in_batch if num_items_in_batch is not None else n_valid.clamp_min(1)
            loss = loss_sum / denom
        if a.average_tokens_across_devices and num_items_in_batch is not None:
            loss = loss * D.world_size()
        aux = None
        if self.aux_loss_enabled:
            aux = model.aux_loss(ctx)
            if aux is not None:
                loss = loss + a.router_aux_loss_coef * aux
        m = self._metrics[mode]
        stats = [ent_sum.detach().float(), n_valid.detach().float()]
        stats.append(correct.detach().float() if correct is not None else torch.zeros_like(stats[0]))
        m["_stats"].append(torch.stack(stats))
        if aux is not None:
            m["aux_loss"].append(aux.detach())
        return loss

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        flat, ctx, tgt = self._flat_labels(model, inputs)
        sp = self.sp_info()
        if sp is not None:  # Ulysses: this rank keeps one chunk of the packed stream
            from ..parallel.ulysses import shard_sequence

            flat, tgt, ctx = shard_sequence(flat, tgt, ctx, sp, self.processing_class.pad_token_id or 0)
        if model.training:
            n_tok = torch.tensor(float(flat.numel()), device=flat.device)
            self._metrics["train"]["_num_tokens"].append(n_tok)
        extra = {}
        if getattr(model, "is_vlm", False):
            extra["pixel_values"] = inputs.get("pixel_values")
            if inputs.get("image_grid_thw") is not None:  # towers that take flat patches of images of any size
                extra["image_grid_thw"] = inputs["image_grid_thw"]
            tgt = tgt.masked_fill(tgt == model.config.image_token_index, -100)  # placeholders carry no target
        with self.maybe_activation_offload_context:
            hidden = model.forward_hidden(flat, ctx, **extra)
        loss = self.loss_from_hidden(model, hidden, ctx, tgt, num_items_in_batch)
        return (loss, None) if return_outputs else loss

    def prediction_step(self, model, inputs, prediction_loss_only=True, ignore_keys=None):
        inputs = self._prepare_inputs(inputs)
        with torch.no_grad():
            loss = self.compute_loss(model, inputs)
            if prediction_loss_only or getattr(model, "is_vlm", False):
                return loss.detach(), None, None
            # metrics on predictions (``compute_metrics``): this is the one place where [batch, length, vocab] logits
            # are materialised, as the reference does in evaluation; training never does
            kw = {k: inputs[k] for k in ("attention_mask", "position_ids") if inputs.get(k) is not None}
            logits = model(input_ids=inputs["input_ids"], **kw).logits
        return loss.detach(), logits, inputs.get("labels")

    def log(self, logs: dict, start_time: float | None = None):
        mode = "train" if self.model.training else "eval"
        m = self._metrics[mode]
        stats = m.pop("_stats", None)
        ntok = m.pop("_num_tokens", None)
        if stats:
            s = torch.stack(stats).sum(0)
            if ntok:
                s = torch.cat([s, torch.stack(ntok).sum()[None]])
            if D.world_size() > 1:
                D.all_reduce(s, "sum")
            ent, nv, cor = float(s[0]), max(float(s[1]), 1.0), float(s[2])
            m["entropy"].append(ent / nv)
            if self.args.loss_type != "dft":
                m["mean_token_accuracy"].append(cor / nv)
            if ntok:
                self._total_train_tokens += int(s[3])
                m["num_tokens"].append(float(self._total_train_tokens))
        for k in list(m.keys()):
            m[k] = [float(v) for v in m[k]]
        super().log(logs, start_time)
