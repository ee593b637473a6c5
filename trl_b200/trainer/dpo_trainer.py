"""Direct Preference Optimization.

Behaviour of trl/trainer/dpo_trainer.py: preference collator (:92-213), tokenisation into
``prompt_ids / chosen_ids / rejected_ids`` (:1019-1071), reference handling (explicit model,
frozen copy, adapter-off, precomputed log-probs :1107-1176), the 15 loss types with
f-divergences, LD-DPO and WPO weighting (:1396-1578) and the metric names (:1585-1653).

Forward: chosen and rejected sequences go through the model as one packed, padding-free stream;
completion-token log-probabilities come from the fused lm_head kernel, and for the default sigmoid
loss the masked per-sequence sums, the loss, its gradient and the reward metrics are one kernel.
"""
from __future__ import annotations

import copy
import os
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.nn.functional as F

from ..data_utils import _map, is_conversational, maybe_apply_chat_template, maybe_extract_prompt
from ..loop.trainer import Trainer
from ..models.decoder import SeqCtx
from ..ops import functional as ops
from ..parallel import dist as D
from .dpo_config import DPOConfig
from .utils import (DeferredMetric, create_model_from_path, defer_mean, defer_ratio, disable_dropout_in_model, hash_module, pad,
                    resolve_deferred_metrics, use_adapter)


@dataclass
class DataCollatorForPreference:
    """Rows ``prompt_ids / chosen_ids / rejected_ids`` -> batch ``[chosen..., rejected...]`` with
    ``input_ids, attention_mask, completion_mask`` (+ ``ref_chosen_logps / ref_rejected_logps``)."""

    pad_token_id: int
    max_length: Optional[int] = None
    truncation_mode: str = "keep_start"
    pad_to_multiple_of: Optional[int] = None
    return_tensors: str = "pt"

    def __call__(self, examples: list[dict[str, Any]]) -> dict[str, Any]:
        seqs, masks = [], []
        for key in ("chosen_ids", "rejected_ids"):
            for ex in examples:
                ids = list(ex["prompt_ids"]) + list(ex[key])
                cm = [0] * len(ex["prompt_ids"]) + [1] * len(ex[key])
                if self.max_length is not None and len(ids) > self.max_length:
                    sl = slice(0, self.max_length) if self.truncation_mode == "keep_start" else slice(-self.max_length, None)
                    ids, cm = ids[sl], cm[sl]
                seqs.append(torch.tensor(ids, dtype=torch.long))
                masks.append(torch.tensor(cm, dtype=torch.long))
        out = {
            "input_ids": pad(seqs, self.pad_token_id, "right", self.pad_to_multiple_of),
            "attention_mask": pad([torch.ones_like(s) for s in seqs], 0, "right", self.pad_to_multiple_of),
            "completion_mask": pad(masks, 0, "right", self.pad_to_multiple_of),
        }
        if "ref_chosen_logps" in examples[0]:
            out["ref_chosen_logps"] = torch.tensor([ex["ref_chosen_logps"] for ex in examples])
            out["ref_rejected_logps"] = torch.tensor([ex["ref_rejected_logps"] for ex in examples])
        return out

    torch_call = __call__


class DataCollatorForVisionPreference:
    """Tokenises and converts images batch by batch.  Examples: ``images`` (or ``image``) + ``prompt`` / ``chosen`` /
    ``rejected`` (text or conversations).  Output rows are [all chosen; all rejected] with ``completion_mask`` and the
    images repeated for both halves (trl/trainer/dpo_trainer.py:217-370)."""

    def __init__(self, processor, max_length: int | None = None, pad_to_multiple_of: int | None = None,
                 return_tensors: str = "pt"):
        self.processor = processor
        self.max_length = max_length
        self.pad_to_multiple_of = pad_to_multiple_of
        self.return_tensors = return_tensors

    def __call__(self, examples):
        from ..data_utils import apply_chat_template, prepare_multimodal_messages
        from .utils import flush_left

        if self.pad_to_multiple_of is not None:
            raise NotImplementedError("Padding to a multiple of a value is not yet implemented for vision-language "
                                      "modeling and prompt-completion data.")
        examples = [dict(e) for e in examples]
        for e in examples:
            if "image" in e:
                e["images"] = [e.pop("image")]
            e.setdefault("images", [])
        images = [list(e["images"]) for e in examples] * 2  # chosen rows, then rejected rows
        if all(not i for i in images):
            images = None
        if is_conversational(examples[0]):
            rendered = []
            for e in examples:
                e = {"prompt": prepare_multimodal_messages(e["prompt"], images=e["images"]),
                     "chosen": prepare_multimodal_messages(e["chosen"]),
                     "rejected": prepare_multimodal_messages(e["rejected"])}
                rendered.append(apply_chat_template(e, self.processor))
            examples = rendered
        kw = dict(return_tensors=self.return_tensors, add_special_tokens=False, padding=True)
        pp = self.processor(images=images, text=[e["prompt"] for e in examples] * 2, padding_side="left", **kw)
        pc = self.processor(text=[e["chosen"] for e in examples] + [e["rejected"] for e in examples],
                            padding_side="right", **kw)
        ids = torch.cat([pp["input_ids"], pc["input_ids"]], dim=1)
        am = torch.cat([pp["attention_mask"], pc["attention_mask"]], dim=1)
        cm = torch.cat([torch.zeros_like(pp["attention_mask"]), pc["attention_mask"]], dim=1)
        am, ids, cm = flush_left(am, ids, cm)
        if self.max_length is not None:
            ids, am, cm = ids[:, :self.max_length], am[:, :self.max_length], cm[:, :self.max_length]
        out = {k: v for k, v in pp.items() if k not in ("input_ids", "attention_mask")}
        out.update(input_ids=ids, attention_mask=am, completion_mask=cm)
        return out

    torch_call = __call__


class DPOTrainer(Trainer):
    _tag_names = ["trl", "dpo"]
    _name = "DPO"
    _needs_ref = True  # reference-free subclasses (CPO, ORPO, ...) turn the frozen copy off

    def __init__(self, model, ref_model=None, args: DPOConfig | None = None, data_collator=None, train_dataset=None,
                 eval_dataset=None, processing_class=None, compute_metrics=None, callbacks=None,
                 optimizers=(None, None), peft_config=None):
        if args is None:
            name = model if isinstance(model, str) else getattr(model, "name_or_path", "model")
            args = DPOConfig(f"{os.path.basename(str(name).rstrip('/'))}-DPO")
        if isinstance(model, str):
            model_id = model
            model = create_model_from_path(model, **dict(args.model_init_kwargs or {}))
        else:
            model_id = getattr(model, "name_or_path", "")
        if ref_model is model:
            raise ValueError("`model` and `ref_model` cannot be the same object; pass ref_model=None for a frozen copy")
        if isinstance(ref_model, str):
            ref_model = create_model_from_path(ref_model, **dict(args.model_init_kwargs or {}))
        if processing_class is None:
            from transformers import AutoTokenizer

            processing_class = AutoTokenizer.from_pretrained(model_id)
        tok = getattr(processing_class, "tokenizer", processing_class)  # a processor wraps the text tokenizer
        if args.eos_token is not None:
            tok.eos_token = args.eos_token
        if tok.pad_token is None:
            tok.pad_token = args.pad_token or tok.eos_token
        if peft_config is not None:
            from ..models.lora import get_peft_model

            model = get_peft_model(model, peft_config)
        if args.disable_dropout:
            disable_dropout_in_model(model)
            if ref_model is not None:
                disable_dropout_in_model(ref_model)
        self.beta, self.loss_types = args.beta, list(args.loss_type)
        self.loss_weights = list(args.loss_weights) if args.loss_weights else [1.0] * len(self.loss_types)
        self.label_smoothing, self.use_weighting = args.label_smoothing, args.use_weighting
        self.f_divergence_type, self.f_alpha = args.f_divergence_type, args.f_alpha_divergence_coef
        self.ld_alpha = args.ld_alpha
        self.precompute_ref_log_probs = args.precompute_ref_log_probs
        self.aux_loss_enabled = getattr(getattr(model, "config", None), "is_moe", False)
        self.padding_free = args.padding_free
        first = next(iter(train_dataset)) if train_dataset is not None else {}
        self._is_vlm = "images" in first or "image" in first
        if self._is_vlm:
            if not hasattr(processing_class, "tokenizer"):
                raise ValueError("a dataset with images needs a processor (image processor + tokenizer) as "
                                 "processing_class, e.g. models.vision_processing.VisionProcessor")
            if args.precompute_ref_log_probs or args.padding_free:
                raise ValueError("precompute_ref_log_probs / padding_free are not supported for vision-language datasets")
            if data_collator is None:
                data_collator = DataCollatorForVisionPreference(processing_class, args.max_length, args.pad_to_multiple_of)
            args.remove_unused_columns = False
        if data_collator is None:
            data_collator = DataCollatorForPreference(tok.pad_token_id, args.max_length, args.truncation_mode,
                                                      args.pad_to_multiple_of)
        with D.main_process_first():
            if self._is_vlm:
                pass  # the collator reads the raw columns
            elif train_dataset is not None:
                train_dataset = self._prepare_dataset(train_dataset, tok, args, "train")
            if eval_dataset is not None and not self._is_vlm:
                if isinstance(eval_dataset, dict):
                    eval_dataset = {k: self._prepare_dataset(v, tok, args, k) for k, v in eval_dataset.items()}
                else:
                    eval_dataset = self._prepare_dataset(eval_dataset, tok, args, "eval")
        super().__init__(optimizers=optimizers, model=model, args=args, data_collator=data_collator, train_dataset=train_dataset,
                         eval_dataset=eval_dataset, processing_class=processing_class if self._is_vlm else tok,
                         compute_metrics=compute_metrics, callbacks=callbacks)
        self.model_accepts_loss_kwargs = False  # loss is divided by the accumulation steps by the loop
        self._ref_adapter_off = False
        if not self._needs_ref:
            self.ref_model = None
        elif ref_model is not None:
            self.ref_model = ref_model.to(self.args.device, dtype=self.model.dtype).eval().requires_grad_(False)
        elif getattr(self.model, "peft_config", None) is not None:
            self.ref_model, self._ref_adapter_off = None, True
        elif self.precompute_ref_log_probs:
            self.ref_model = None  # the policy's initial weights are the reference; computed before training
        else:
            self.ref_model = copy.deepcopy(self.model).eval().requires_grad_(False)
        if args.sync_ref_model:
            if self.ref_model is None:
                raise ValueError("sync_ref_model needs a separate reference model (not PEFT adapter-off / precomputed)")
            from .callbacks import SyncRefModelCallback

            self.add_callback(SyncRefModelCallback(ref_model=self.ref_model))
        self._precomputed = {"train": False, "eval": False}
        if self.precompute_ref_log_probs:
            self.train_dataset = self._precompute_ref_logps(self.train_dataset, "train")
            if isinstance(self.eval_dataset, dict):
                self.eval_dataset = {k: self._precompute_ref_logps(v, k) for k, v in self.eval_dataset.items()}
            elif self.eval_dataset is not None:
                self.eval_dataset = self._precompute_ref_logps(self.eval_dataset, "eval")

    def evaluate(self, eval_dataset=None, ignore_keys=None, metric_key_prefix: str = "eval"):
        """A dataset handed to ``evaluate`` gets the preparation of ``__init__`` (tokenisation, reference log-probs when
        they are precomputed), dpo_trainer.py:1657-1713."""
        if eval_dataset is not None and not isinstance(eval_dataset, str) and not self._is_vlm:
            if (self.precompute_ref_log_probs and self.ref_model is None and not self._ref_adapter_off
                    and self.state.global_step > 0):
                raise ValueError(
                    "Cannot compute reference log-probs for a dataset passed to `evaluate()` after training has started, "
                    "because `precompute_ref_log_probs=True` and no `ref_model` was provided (full fine-tuning): the "
                    "reference is the policy before training and is not kept in memory. Provide this dataset as "
                    "`eval_dataset` at initialization, pass an explicit `ref_model`, or set "
                    "`precompute_ref_log_probs=False`.")
            tok = getattr(self.processing_class, "tokenizer", self.processing_class)
            parts = eval_dataset if isinstance(eval_dataset, dict) else {"eval": eval_dataset}
            done = {}
            for name, ds in parts.items():
                ds = self._prepare_dataset(ds, tok, self.args, name)
                if self.precompute_ref_log_probs and "ref_chosen_logps" not in next(iter(ds)):
                    ds = self._precompute_ref_logps(ds, name)
                done[name] = ds
            if isinstance(eval_dataset, dict):
                out = {}
                for name, ds in done.items():
                    out.update(super().evaluate(ds, ignore_keys, f"{metric_key_prefix}_{name}"))
                return out
            eval_dataset = done["eval"]
        return super().evaluate(eval_dataset, ignore_keys, metric_key_prefix)

    # ---- dataset ------------------------------------------------------------------------------------
    def _prepare_dataset(self, dataset, tok, args, name):
        first = next(iter(dataset))
        if "prompt_ids" in first:
            return dataset
        ds = _map(dataset, maybe_extract_prompt)
        conv = is_conversational(next(iter(ds)))
        ds = _map(ds, lambda ex: maybe_apply_chat_template(
            {k: ex[k] for k in ("prompt", "chosen", "rejected", "chat_template_kwargs") if k in ex}, tok,
            tools=ex.get("tools")))
        eos = tok.eos_token

        def tokenize(ex):
            chosen, rejected = ex["chosen"], ex["rejected"]
            if not conv:
                if not chosen.endswith(eos):
                    chosen = chosen + eos
                if not rejected.endswith(eos):
                    rejected = rejected + eos
            p = tok(text=ex["prompt"], add_special_tokens=not conv)["input_ids"]
            c = tok(text=chosen, add_special_tokens=False)["input_ids"]
            r = tok(text=rejected, add_special_tokens=False)["input_ids"]
            return {"prompt_ids": p, "chosen_ids": c, "rejected_ids": r}
        ds = _map(ds, tokenize)
        if args.max_length is not None and args.truncation_mode == "keep_start":
            # a prompt that fills max_length alone leaves no completion token after truncation: such rows are dropped
            if hasattr(ds, "filter"):
                ds = ds.filter(lambda ex: len(ex["prompt_ids"]) < args.max_length)
            else:
                ds = [r for r in ds if len(r["prompt_ids"]) < args.max_length]
        keep = {"prompt_ids", "chosen_ids", "rejected_ids", "ref_chosen_logps", "ref_rejected_logps"}
        if hasattr(ds, "remove_columns"):
            ds = ds.remove_columns([c for c in ds.column_names if c not in keep])
        else:
            ds = [{k: v for k, v in r.items() if k in keep} for r in ds]
        return ds

    def _precompute_ref_logps(self, dataset, name):
        """Reference log-probs for the whole dataset, cached on disk under a key made of the data and
        the reference weights (dpo_trainer.py:1107-1176)."""
        a = self.args
        ref = self.ref_model if self.ref_model is not None else self.model
        fp = getattr(dataset, "_fingerprint", None) or str(len(dataset))
        key = [f"{fp}-{hash_module(ref)[:16]}" if D.is_main() else None]
        D.broadcast_object_list(key)
        cache = os.path.join(a.output_dir, f"ref_logps_{name}_{key[0]}.pt")
        if os.path.exists(cache):
            vals = torch.load(cache, weights_only=True)
        else:
            bs = a.precompute_ref_batch_size or a.per_device_train_batch_size
            rows = [dataset[i] for i in range(len(dataset))]
            cs, rs = [], []
            for s in range(0, len(rows), bs):
                batch = self._prepare_inputs(self.data_collator(rows[s:s + bs]))
                with torch.no_grad():
                    lp, _, _ = self._sequence_logps(ref, batch, no_grad=True, adapter_off=self._ref_adapter_off)
                n = len(rows[s:s + bs])
                cs.append(lp[:n].cpu())
                rs.append(lp[n:].cpu())
            vals = {"c": torch.cat(cs), "r": torch.cat(rs)}
            if D.is_main():
                os.makedirs(a.output_dir, exist_ok=True)
                torch.save(vals, cache)
            D.barrier()
        self._precomputed[name] = True
        if hasattr(dataset, "add_column"):
            dataset = dataset.add_column("ref_chosen_logps", vals["c"].tolist())
            return dataset.add_column("ref_rejected_logps", vals["r"].tolist())
        return [{**r, "ref_chosen_logps": float(c), "ref_rejected_logps": float(rr)}
                for r, c, rr in zip(dataset, vals["c"], vals["r"])]

    # ---- log-probabilities -------------------------------------------------------------------------------
    def _sequence_logps(self, model, inputs, no_grad=False, adapter_off=False, need_stats=False):
        """Per-sequence sums of completion-token log-probs.  Returns (seq_logps[2P], aux, extras)."""
        ids, am, cm = inputs["input_ids"], inputs["attention_mask"], inputs["completion_mask"]
        flat, ctx, _ = model.pack_inputs(ids, am)
        mask_flat = am.reshape(-1).bool()
        # position t predicts t+1: target mask/ids shifted left inside every row
        tgt = torch.full_like(ids, 0)
        tgt[:, :-1] = ids[:, 1:]
        pred = torch.zeros_like(cm)
        pred[:, :-1] = cm[:, 1:] * am[:, 1:]
        tgt_f, pred_f = tgt.reshape(-1)[mask_flat], pred.reshape(-1)[mask_flat].bool()
        cmgr = use_adapter(model, None) if adapter_off else _null()
        extra = {"pixel_values": inputs.get("pixel_values")} if getattr(model, "is_vlm", False) else {}
        if extra and inputs.get("image_grid_thw") is not None:
            extra["image_grid_thw"] = inputs["image_grid_thw"]
        with cmgr:
            hidden = model.forward_hidden(flat, ctx, **extra)
        sel = pred_f.nonzero().flatten()
        lp, ent = ops.lm_head_logprobs(hidden[sel], model.lm_head_weight, tgt_f[sel], 1.0,
                                       softcap=model.config.final_logit_softcapping, compute_entropy=need_stats)
        seq_id = torch.repeat_interleave(torch.arange(ctx.cu_seqlens.numel() - 1, device=ids.device),
                                         (ctx.cu_seqlens[1:] - ctx.cu_seqlens[:-1]).long())[sel]
        n_seq = ids.shape[0]
        extras = {"tok_logps": lp, "seq_id": seq_id, "entropy": ent, "n_tok": pred.sum(1).float(), "hidden_sel": hidden[sel],
                  "targets": tgt_f[sel]}
        if self.ld_alpha is not None:
            # LD-DPO: tokens beyond the shorter completion of the pair are down-weighted by alpha
            P = n_seq // 2
            n_tok = extras["n_tok"]
            pub = torch.minimum(n_tok[:P], n_tok[P:]).repeat(2)
            pos_in_comp = _rank_within(seq_id, n_seq)
            w = torch.where(pos_in_comp < pub[seq_id], torch.ones_like(lp), torch.full_like(lp, self.ld_alpha))
            seq_lp = torch.zeros(n_seq, device=ids.device, dtype=lp.dtype).index_add(0, seq_id, lp * w)
        else:
            seq_lp = torch.zeros(n_seq, device=ids.device, dtype=lp.dtype).index_add(0, seq_id, lp)
        aux = model.aux_loss(ctx) if (self.aux_loss_enabled and not no_grad) else None
        return seq_lp, aux, extras

    # ---- loss ------------------------------------------------------------------------------------------------
    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        mode = "train" if model.training else "eval"
        m = self._metrics[mode]
        seq_lp, aux, ex = self._sequence_logps(model, inputs, need_stats=True)
        P = seq_lp.shape[0] // 2
        pc, pr = seq_lp[:P], seq_lp[P:]
        fused_loss = None
        if "ref_chosen_logps" in inputs:
            rc, rr = inputs["ref_chosen_logps"].to(pc), inputs["ref_rejected_logps"].to(pc)
        else:
            if (self.ref_model is not None and getattr(self, "_ref_stream", None) is None
                    and getattr(getattr(self, "engine", None), "mode", "") == "full_shard_stream"):
                # streamed policy => streamed frozen reference (one slice per layer and rank, no optimizer state)
                from ..parallel.streamshard import StreamShardEngine

                if getattr(self.args, "sync_ref_model", False):
                    raise NotImplementedError("sync_ref_model copies whole parameters; it is not available with "
                                              "shard_mode='full_shard_stream'")
                self._ref_stream = StreamShardEngine(self.ref_model, frozen=True, device=self.args.device,
                                                    init_seed=self.args.seed)
            with torch.no_grad():
                ref = self.ref_model if self.ref_model is not None else model
                rlp, _, rex = self._sequence_logps(ref, inputs, no_grad=True, adapter_off=self._ref_adapter_off)
            rc, rr = rlp[:P], rlp[P:]
            if (seq_lp.is_cuda and self.loss_types == ["sigmoid"] and self.f_divergence_type == "reverse_kl"
                    and not self.use_weighting and self.ld_alpha is None):
                # one kernel: masked per-sequence sums, sigmoid loss, its gradient and the reward metrics
                from ..ops import cuda as K

                counts = torch.bincount(ex["seq_id"], minlength=2 * P)
                cu = torch.zeros(2 * P + 1, dtype=torch.int32, device=counts.device)
                cu[1:] = counts.cumsum(0)
                fused_loss, _ = K.dpo_loss(ex["tok_logps"], rex["tok_logps"], torch.ones_like(rex["tok_logps"]), cu,
                                           self.beta, self.label_smoothing)
        c_lr, r_lr = pc - rc, pr - rr
        if self.f_divergence_type == "reverse_kl":
            cs, rs = c_lr, r_lr
        elif self.f_divergence_type == "forward_kl":
            cs, rs = -torch.exp(-c_lr), -torch.exp(-r_lr)
        elif self.f_divergence_type == "js_divergence":
            cs, rs = F.logsigmoid(c_lr), F.logsigmoid(r_lr)
        else:
            a_ = self.f_alpha
            if abs(a_ - 1.0) < 1e-6:
                cs, rs = c_lr, r_lr
            else:
                k = 1.0 / (a_ - 1.0)
                cs = torch.exp(torch.clamp((a_ - 1.0) * c_lr.float(), max=80.0)).to(c_lr.dtype) * k
                rs = torch.exp(torch.clamp((a_ - 1.0) * r_lr.float(), max=80.0)).to(r_lr.dtype) * k
        delta = cs - rs
        beta, ls = self.beta, self.label_smoothing
        n_tok = ex["n_tok"]
        cn, rn = n_tok[:P].clamp(min=1.0), n_tok[P:].clamp(min=1.0)
        loss = 0.0
        for lt, lw in zip(self.loss_types, self.loss_weights):
            if fused_loss is not None:
                loss = fused_loss * lw
                break
            if lt == "sigmoid":
                per = -F.logsigmoid(beta * delta) * (1 - ls) - F.logsigmoid(-beta * delta) * ls
            elif lt == "hinge":
                per = torch.relu(1 - beta * delta)
            elif lt == "ipo":
                per = ((cs / cn - rs / rn) - 1 / (2 * beta)) ** 2
            elif lt == "exo_pair":
                eps = torch.tensor(ls if ls > 0 else 1e-3, device=delta.device)
                qw, ql = torch.sigmoid(beta * delta), torch.sigmoid(-beta * delta)
                per = qw * (F.logsigmoid(beta * delta) - torch.log1p(-eps)) + ql * (F.logsigmoid(-beta * delta) - torch.log(eps))
            elif lt == "nca_pair":
                per = -F.logsigmoid(beta * cs) - 0.5 * F.logsigmoid(-beta * cs) - 0.5 * F.logsigmoid(-beta * rs)
            elif lt == "robust":
                per = (-(1 - ls) * F.logsigmoid(beta * delta) + ls * F.logsigmoid(-beta * delta)) / (1 - 2 * ls)
            elif lt == "bco_pair":
                per = -F.logsigmoid(beta * cs) - F.logsigmoid(-beta * rs)
            elif lt == "sppo_hard":
                per = (cs - 0.5 / beta) ** 2 + (rs + 0.5 / beta) ** 2
            elif lt == "aot":
                d = torch.sort(pc - pr, dim=0).values - torch.sort(rc - rr, dim=0).values
                per = -F.logsigmoid(beta * d) * (1 - ls) - F.logsigmoid(-beta * d) * ls
            elif lt == "aot_unpaired":
                d = torch.sort(c_lr, dim=0).values - torch.sort(r_lr, dim=0).values
                per = -F.logsigmoid(beta * d) * (1 - ls) - F.logsigmoid(-beta * d) * ls
            elif lt == "apo_zero":
                per = (1 - torch.sigmoid(beta * c_lr)) + torch.sigmoid(beta * r_lr)
            elif lt == "apo_down":
                per = torch.sigmoid(beta * c_lr) + (1 - torch.sigmoid(beta * delta))
            elif lt == "discopop":
                z = delta * beta
                mod = torch.sigmoid(z / self.args.discopop_tau)
                per = -F.logsigmoid(z) * (1 - mod) + torch.exp(-z) * mod
            elif lt == "sft":
                chosen_tok = ex["seq_id"] < P
                nll = -(ex["tok_logps"] * chosen_tok).sum() / chosen_tok.sum().clamp(min=1)
                per = nll.expand(P)
            elif lt == "sigmoid_norm":
                per = -F.logsigmoid(beta * (cs / cn - rs / rn))
            else:
                raise ValueError(f"Unknown loss type: {lt}")
            if self.use_weighting:
                per = per * self._wpo_weights(model, ex, P)
            loss = loss + per.mean() * lw
        if aux is not None:
            loss = loss + self.args.router_aux_loss_coef * aux
            m["aux_loss"].append(aux.detach())
        # ---- metrics: local partial results only; one reduction per logging step resolves them ---------------------
        with torch.no_grad():
            cr, rrw = beta * c_lr.detach(), beta * r_lr.detach()
            ent = ex["entropy"]
            vals = [cr.mean(), rrw.mean(), (cr > rrw).float().mean(), (cr - rrw).mean(), pc.detach().mean(),
                    pr.detach().mean()]
            names = ["rewards/chosen", "rewards/rejected", "rewards/accuracies", "rewards/margins", "logps/chosen",
                     "logps/rejected"]
            for n, v in zip(names, vals):
                m[n].append(defer_mean(v))
            m["entropy"].append(defer_ratio(ent.sum(), torch.tensor(float(ent.numel()), device=ent.device)))
            if mode == "train":
                seen = inputs["attention_mask"].sum().float()
                prev = getattr(self, "_num_tokens_local", None)
                self._num_tokens_local = seen if prev is None else prev + seen
            if getattr(self, "_num_tokens_local", None) is not None:
                # running local count; summed over the ranks when the log call resolves it
                m["num_tokens"].append(DeferredMetric(self._num_tokens_local.reshape(1).clone(), "sum"))
        return (loss, None) if return_outputs else loss

    def _wpo_weights(self, model, ex, P):
        """WPO: exp(mean over completion tokens of (log p - log sum p^2)) for chosen x rejected."""
        with torch.no_grad():
            h, W, y = ex["hidden_sel"].detach(), model.lm_head_weight, ex["targets"]
            if h.is_cuda and h.dtype == torch.bfloat16:
                from ..ops import cuda as K

                _, _, lse1, _ = K.lmhead_forward(h.contiguous(), W, y, 1.0, False, False)
                _, _, lse2, _ = K.lmhead_forward(h.contiguous(), W, y, 2.0, False, False)
            else:
                z = h.float() @ W.float().t()
                lse1, lse2 = torch.logsumexp(z, -1), torch.logsumexp(2 * z, -1)
            aligned = ex["tok_logps"].detach() - (lse2 - 2 * lse1)
            n_seq = 2 * P
            s = torch.zeros(n_seq, device=h.device).index_add(0, ex["seq_id"], aligned.float())
            w = torch.exp(s / ex["n_tok"].clamp(min=1))
        return w[:P] * w[P:]

    def prediction_step(self, model, inputs, prediction_loss_only=True, ignore_keys=None):
        inputs = self._prepare_inputs(inputs)
        with torch.no_grad():
            loss = self.compute_loss(model, inputs)
        return loss.detach(), None, None

    def log(self, logs, start_time=None):
        mode = "train" if self.model.training else "eval"
        resolve_deferred_metrics(self._metrics[mode])
        for k in list(self._metrics[mode].keys()):
            self._metrics[mode][k] = [float(v) for v in self._metrics[mode][k]]
        super().log(logs, start_time)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _rank_within(seq_id: torch.Tensor, n_seq: int) -> torch.Tensor:
    """Index of every element inside its (sorted, contiguous) segment."""
    counts = torch.bincount(seq_id, minlength=n_seq)
    starts = torch.cumsum(counts, 0) - counts
    return (torch.arange(seq_id.numel(), device=seq_id.device) - starts[seq_id]).float()
