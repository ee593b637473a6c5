"""Helpers shared by the experimental trainers (counterpart of trl/experimental/utils.py:59-1101): preference and
ChatML collators, byte-offset utilities for cross-tokenizer alignment, truncation / padding helpers, reward scoring
with a sequence-classification head, reference-model creation."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Optional

import torch

from ..trainer.utils import pad


# ---- collators -----------------------------------------------------------------------------------------------------
@dataclass
class DPODataCollatorWithPadding:
    """Pads every ``*_input_ids / *_attention_mask / *_labels`` key; ``prompt*`` keys are padded on the left."""

    pad_token_id: int = 0
    label_pad_token_id: int = -100
    is_encoder_decoder: Optional[bool] = False

    def __call__(self, features: list[dict[str, Any]]) -> dict[str, Any]:
        out = {}
        for k in features[0]:
            if k.endswith(("_input_ids", "_attention_mask", "_labels", "_pixel_values")):
                if k.endswith("_input_ids"):
                    val = self.pad_token_id
                elif k.endswith("_labels"):
                    val = self.label_pad_token_id
                else:
                    val = 0
                side = "left" if k.startswith("prompt") else "right"
                dt = torch.float32 if k.endswith("_pixel_values") else torch.int64
                out[k] = pad([torch.tensor(f[k], dtype=dt) for f in features], val, side)
            elif k.endswith("_logps"):
                out[k] = torch.tensor([f[k] for f in features])
            else:
                out[k] = [f[k] for f in features]
        return out


@dataclass
class DataCollatorForChatML:
    """Renders ``messages`` with the chat template; the last assistant message becomes the labelled completion, the
    rest the prompt (also returned separately as ``prompts`` / ``prompt_attention_mask``, left padded, for generation)."""

    tokenizer: Any
    ignore_index: int = -100
    max_length: Optional[int] = None
    prompt_key: str = "prompt"
    messages_key: str = "messages"

    def __post_init__(self):
        if self.tokenizer.pad_token_id is None:
            raise ValueError("The tokenizer does not have a pad token. Please set `pad_token_id` in the tokenizer.")
        if self.max_length is None:
            self.max_length = min(getattr(self.tokenizer, "model_max_length", 1024) or 1024, 1024)

    def __call__(self, examples: list[dict[str, Any]]) -> dict[str, torch.Tensor]:
        tok = self.tokenizer
        ids, labels, prompts = [], [], []
        for ex in examples:
            msgs = ex[self.messages_key]
            p = tok.apply_chat_template(msgs[:-1], tokenize=True, add_generation_prompt=True)
            full = tok.apply_chat_template(msgs, tokenize=True)
            p = p["input_ids"] if isinstance(p, dict) else p
            full = full["input_ids"] if isinstance(full, dict) else full
            p, full = list(p)[: self.max_length], list(full)[: self.max_length]
            n = len(p) if full[: len(p)] == p else 0
            ids.append(torch.tensor(full))
            labels.append(torch.tensor([self.ignore_index] * n + full[n:]))
            prompts.append(torch.tensor(p))
        return {"input_ids": pad(ids, tok.pad_token_id, "left"),
                "attention_mask": pad([torch.ones_like(x) for x in ids], 0, "left"),
                "labels": pad(labels, self.ignore_index, "left"),
                "prompts": pad(prompts, tok.pad_token_id, "left"),
                "prompt_attention_mask": pad([torch.ones_like(x) for x in prompts], 0, "left")}


class DataCollatorForVisionLanguageChatML:
    def __init__(self, *a, **kw):
        raise NotImplementedError("vision-language ChatML collation needs an image processor and a vision tower; the "
                                  "native decoder is text-only")


# ---- byte offsets (cross-tokenizer alignment) ------------------------------------------------------------------------
def pad_byte_offsets(offsets: list[tuple[int, int]], target_length: int, padding_side: str) -> torch.Tensor:
    t = torch.tensor(offsets, dtype=torch.long).reshape(-1, 2)
    fill = torch.full((max(0, target_length - t.shape[0]), 2), -1, dtype=torch.long)
    return torch.cat([fill, t] if padding_side == "left" else [t, fill])[:target_length]


def _bytes_to_unicode() -> dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs, n = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, map(chr, cs)))


_U2B = {v: k for k, v in _bytes_to_unicode().items()}


def is_byte_level_tokenizer(backend) -> bool:
    try:
        vocab = backend.get_vocab()
    except Exception:
        return False
    return "Ġ" in "".join(list(vocab)[:2000]) or any(k.startswith("Ġ") for k in list(vocab)[:5000])


def piece_byte_len(piece: str) -> int:
    """Byte length of a token piece: byte-level pieces map one character to one byte, others are UTF-8."""
    if piece and all(ch in _U2B for ch in piece):
        return len(piece)
    return len(piece.replace("▁", " ").encode("utf-8"))


def encode_with_byte_offsets(backend, texts: list[str], add_special_tokens: bool = False):
    """Token ids plus (start, end) byte offsets into the UTF-8 text for every token."""
    all_ids, all_offs = [], []
    for text in texts:
        enc = backend(text, add_special_tokens=add_special_tokens, return_offsets_mapping=True)
        ids, offs = enc["input_ids"], enc.get("offset_mapping")
        if offs is None:
            pos, offs = 0, []
            for t in backend.convert_ids_to_tokens(ids):
                n = piece_byte_len(t)
                offs.append((pos, pos + n))
                pos += n
        else:  # character offsets -> byte offsets
            prefix = [0]
            for ch in text:
                prefix.append(prefix[-1] + len(ch.encode("utf-8")))
            offs = [(prefix[s], prefix[e]) for s, e in offs]
        all_ids.append(ids)
        all_offs.append(offs)
    return all_ids, all_offs


# ---- tensor helpers ------------------------------------------------------------------------------------------------------
def first_true_indices(bools: torch.Tensor, dtype=torch.long) -> torch.Tensor:
    """Index of the first True along the last dim; the row length when there is none."""
    n = bools.size(-1)
    idx = n * (~bools).type(dtype) + torch.arange(n, dtype=dtype, device=bools.device)
    return torch.min(idx, dim=-1).values


def truncate_right(input_ids: torch.Tensor, stop_token_id: int, pad_token_id: int):
    """Everything after the first stop token becomes padding; returns (ids, mask)."""
    trunc = first_true_indices(input_ids == stop_token_id).unsqueeze(-1)
    shape = [1] * (input_ids.dim() - 1) + [input_ids.shape[-1]]
    idxs = torch.arange(input_ids.shape[-1], device=input_ids.device).view(*shape)
    out = torch.masked_fill(input_ids, idxs > trunc, pad_token_id)
    return out, torch.masked_fill(torch.ones_like(input_ids), idxs > trunc, 0)


def pad_to_length(tensor: torch.Tensor, length: int, pad_value, dim: int = -1) -> torch.Tensor:
    if tensor.size(dim) >= length:
        return tensor
    shape = list(tensor.shape)
    shape[dim] = length - tensor.size(dim)
    return torch.cat([tensor, pad_value * torch.ones(*shape, dtype=tensor.dtype, device=tensor.device)], dim=dim)


def add_bos_token_if_needed(bos_token_id, prompt_len_input_ids, prompt_tokens, chosen_prompt_len_input_ids, chosen_tokens,
                            rejected_prompt_len_input_ids, rejected_tokens):
    if bos_token_id is not None:
        for n, t in ((prompt_len_input_ids, prompt_tokens), (chosen_prompt_len_input_ids, chosen_tokens),
                     (rejected_prompt_len_input_ids, rejected_tokens)):
            if n == 0 or bos_token_id != t["prompt_input_ids"][0]:
                t["prompt_input_ids"] = [bos_token_id] + t["prompt_input_ids"]
                t["prompt_attention_mask"] = [1] + t["prompt_attention_mask"]
    return prompt_tokens, chosen_tokens, rejected_tokens


def add_eos_token_if_needed(eos_token_id: int, chosen_tokens: dict, rejected_tokens: dict):
    for t in (chosen_tokens, rejected_tokens):
        if len(t["input_ids"]) == 0 or eos_token_id != t["input_ids"][-1]:
            t["input_ids"].append(eos_token_id)
            t["attention_mask"].append(1)
    return chosen_tokens, rejected_tokens


def get_reward(model, query_responses: torch.Tensor, pad_token_id: int, context_length: int):
    """Scores of a scalar-head model: (per-token scores, score at the last non-pad token, sequence lengths)."""
    am = (query_responses != pad_token_id).long()
    flat, ctx, _ = model.pack_inputs(query_responses, am)
    hidden = model.forward_hidden(flat, ctx)
    per_tok = (hidden.float() @ model.score.float().t()).squeeze(-1)
    B, T = query_responses.shape
    full = per_tok.new_zeros(B * T)
    full[am.reshape(-1).bool()] = per_tok
    full = full.view(B, T)
    lengths = first_true_indices(query_responses[:, context_length:] == pad_token_id) - 1 + context_length
    return full, full[torch.arange(B, device=full.device), lengths.clamp(min=0)], lengths


def empty_cache() -> None:
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def create_reference_model(model, num_shared_layers: int | None = None, pattern: str | None = None):
    """Frozen copy of ``model``; with ``num_shared_layers`` the first layers are shared (not copied) and frozen in both."""
    ref = copy.deepcopy(model).eval()
    for p in ref.parameters():
        p.requires_grad_(False)
    if num_shared_layers:
        for i in range(num_shared_layers):
            ref.layers[i] = model.layers[i]
            for p in model.layers[i].parameters():
                p.requires_grad_(False)
    return ref


def truncate_dataset(dataset, max_length: int, map_kwargs: dict | None = None):
    from ..data_utils import truncate_dataset as _t

    return _t(dataset, max_length, map_kwargs)


def prepare_peft_model(model, peft_config, args=None):
    if peft_config is None:
        return model
    from ..models.lora import get_peft_model

    return get_peft_model(model, peft_config)


def peft_module_casting_to_bf16(model):
    for n, p in model.named_parameters():
        if "lora_" not in n and p.dtype == torch.float32 and ("norm" in n or "embed" in n or "lm_head" in n):
            p.data = p.data.to(torch.bfloat16)


def enable_gradient_checkpointing(model, gradient_checkpointing_kwargs=None):
    model.gradient_checkpointing_enable(gradient_checkpointing_kwargs)
    return model


def prepare_model_for_kbit_training(model, use_gradient_checkpointing=True, gradient_checkpointing_kwargs=None):
    raise NotImplementedError("4/8-bit base weights (bitsandbytes) have no kernels here; train bf16 or LoRA on bf16")
