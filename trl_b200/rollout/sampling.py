"""Sampling parameters and the PyTorch reference sampler.

The reference hands these to vLLM's ``SamplingParams`` (trl/generation/vllm_generation.py:503-704);
the returned log-probabilities are those of the *processed* distribution
(``logprobs_mode="processed_logprobs"``), i.e. after temperature and filtering.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class SamplingParams:
    n: int = 1
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 16
    eos_token_id: Optional[int] = None
    eos_prob_floor: float = 0.0  # synthetic-benchmark knob: p(eos) is raised to at least this value
    seed: int = 0
    greedy: bool = False
    stop_token_ids: list = field(default_factory=list)

    @property
    def needs_filter_pass(self) -> bool:
        return (self.top_k and self.top_k > 0) or (self.top_p is not None and self.top_p < 1.0)


def apply_repetition_penalty(logits: torch.Tensor, seen: torch.Tensor, penalty: float) -> torch.Tensor:
    if penalty == 1.0:
        return logits
    pen = torch.where(logits > 0, logits / penalty, logits * penalty)
    return torch.where(seen.bool(), pen, logits)


def filter_top_k_top_p(logits: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    """Mask logits outside top-k / nucleus with -inf (static shapes: usable under graph capture)."""
    if top_k and top_k > 0:
        k = min(top_k, logits.shape[-1])
        kth = torch.topk(logits, k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and top_p < 1.0:
        srt, idx = torch.sort(logits, dim=-1, descending=True)
        probs = torch.softmax(srt.float(), dim=-1)
        cum = probs.cumsum(-1)
        remove = (cum - probs) > top_p  # keep the first token that crosses the threshold
        srt = srt.masked_fill(remove, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, srt)
    return logits


def process_logits(logits: torch.Tensor, sp: SamplingParams, seen: torch.Tensor | None = None) -> torch.Tensor:
    """Reference of the whole logit pipeline; returns fp32 processed logits (log-softmax = reported logprobs)."""
    z = logits.float()
    if seen is not None:
        z = apply_repetition_penalty(z, seen, sp.repetition_penalty)
    z = z / max(sp.temperature, 1e-6)
    z = filter_top_k_top_p(z, sp.top_k, sp.top_p)
    if sp.min_p and sp.min_p > 0:
        p = torch.softmax(z, -1)
        z = z.masked_fill(p < sp.min_p * p.max(-1, keepdim=True).values, float("-inf"))
    if sp.eos_prob_floor and sp.eos_token_id is not None:
        e = sp.eos_token_id
        others = z.clone()
        others[..., e] = float("-inf")
        lse_o = torch.logsumexp(others, -1)
        need = lse_o + torch.log(torch.tensor(sp.eos_prob_floor / (1 - sp.eos_prob_floor), device=z.device))
        z[..., e] = torch.maximum(z[..., e], need)
    return z


def sample_reference(logits: torch.Tensor, sp: SamplingParams, generator: torch.Generator | None = None,
                     seen: torch.Tensor | None = None):
    z = process_logits(logits, sp, seen)
    logp = torch.log_softmax(z, -1)
    if sp.greedy or sp.temperature == 0:
        tok = z.argmax(-1)
    else:
        tok = torch.multinomial(logp.exp(), 1, generator=generator).squeeze(-1)
    return tok, logp.gather(-1, tok[:, None]).squeeze(-1)
