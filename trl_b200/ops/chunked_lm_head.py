"""``patch_chunked_lm_head``: replace a model's forward by one that returns per-token log-probs and
entropies of the completion tokens instead of logits (role of trl/trainer/utils.py:1427-1517).

On the native decoder this is a thin wrapper around the fused lm_head op: hidden states are filtered
to the ``completion_mask`` positions before the head, so neither full logits nor prompt positions are
ever computed.  Returns ``{"log_probs", "entropy", "aux_loss"}`` with [B, S-1] tensors.
"""
from __future__ import annotations

import types

import torch

from . import functional as ops


def patch_chunked_lm_head(model, chunk_size: int = 8192, temperature: float = 1.0):
    def forward(self, input_ids, attention_mask=None, completion_mask=None, position_ids=None, **kw):
        flat, ctx, scatter = self.pack_inputs(input_ids, attention_mask, position_ids)
        hidden = scatter(self.forward_hidden(flat, ctx))  # [B, S, H]
        B, S = input_ids.shape
        tgt = input_ids[:, 1:]
        mask = torch.ones_like(tgt, dtype=torch.bool) if completion_mask is None else completion_mask[:, 1:].bool()
        if attention_mask is not None:
            mask = mask & attention_mask[:, 1:].bool()
        h = hidden[:, :-1][mask]
        lp, ent = ops.lm_head_logprobs(h, self.lm_head_weight, tgt[mask], temperature,
                                       softcap=self.config.final_logit_softcapping, compute_entropy=True,
                                       chunk_tokens=chunk_size)
        log_probs = torch.zeros(B, S - 1, dtype=lp.dtype, device=lp.device).masked_scatter(mask, lp)
        entropy = torch.zeros(B, S - 1, dtype=lp.dtype, device=lp.device).masked_scatter(mask, ent)
        return {"log_probs": log_probs, "entropy": entropy, "aux_loss": self.aux_loss(ctx)}

    model.forward = types.MethodType(forward, model)
    return model
