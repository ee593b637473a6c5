"""Value head on a causal LM (trl/experimental/ppo/modeling_value_head.py: ValueHead :36-80,
AutoModelForCausalLMWithValueHead :83-300).

The head is a (dropout, linear -> 1) on the final hidden states of the native decoder; ``forward`` returns
(lm_logits, loss, values) like the reference.  ``state_dict`` carries the head under ``v_head.`` so checkpoints are
the base model's tensors plus the head."""
from __future__ import annotations

import torch
import torch.nn as nn

from ...models.decoder import CausalLM


class ValueHead(nn.Module):
    def __init__(self, hidden_size: int, summary_dropout_prob: float = 0.0, dtype=None, device=None):
        super().__init__()
        self.dropout = nn.Dropout(summary_dropout_prob) if summary_dropout_prob else nn.Identity()
        self.summary = nn.Linear(hidden_size, 1, dtype=dtype, device=device)

    def forward(self, hidden_states):
        out = self.dropout(hidden_states)
        if out.dtype != self.summary.weight.dtype:
            out = out.to(self.summary.weight.dtype)
        return self.summary(out)


class AutoModelForCausalLMWithValueHead(nn.Module):
    supported_args = ("summary_dropout_prob", "v_head_initializer_range", "v_head_init_strategy")

    def __init__(self, pretrained_model: CausalLM, summary_dropout_prob: float = 0.0, v_head_initializer_range: float = 0.2,
                 v_head_init_strategy: str | None = None):
        super().__init__()
        self.pretrained_model = pretrained_model
        cfg = pretrained_model.config
        p = next(pretrained_model.parameters())
        self.v_head = ValueHead(cfg.hidden_size, summary_dropout_prob, dtype=p.dtype, device=p.device)
        if v_head_init_strategy == "normal":
            self.v_head.summary.weight.data.normal_(mean=0.0, std=v_head_initializer_range)
            self.v_head.summary.bias.data.zero_()
        self.config = cfg

    @classmethod
    def from_pretrained(cls, model_or_path, **kw):
        head_kw = {k: kw.pop(k) for k in list(kw) if k in cls.supported_args}
        if isinstance(model_or_path, str):
            from ...trainer.utils import create_model_from_path

            model_or_path = create_model_from_path(model_or_path, **kw)
        return cls(model_or_path, **head_kw)

    def forward(self, input_ids=None, attention_mask=None, **kw):
        flat, ctx, _ = self.pretrained_model.pack_inputs(input_ids, attention_mask)
        hidden = self.pretrained_model.forward_hidden(flat, ctx)
        logits = hidden.float() @ self.pretrained_model.lm_head_weight.float().t()
        values = self.v_head(hidden).squeeze(-1)
        if attention_mask is not None and not bool(attention_mask.all()):
            B, T = input_ids.shape
            full_l = logits.new_zeros(B * T, logits.shape[-1])
            full_v = values.new_zeros(B * T)
            idx = attention_mask.reshape(-1).bool().nonzero().flatten()
            full_l[idx], full_v[idx] = logits, values
            return full_l.view(B, T, -1), None, full_v.view(B, T)
        return logits.view(*input_ids.shape, -1), None, values.view(*input_ids.shape)

    def generate(self, *a, **kw):
        return self.pretrained_model.generate(*a, **kw)

    def state_dict(self, *a, **kw):
        sd = self.pretrained_model.state_dict(*a, **kw)
        for k, v in self.v_head.state_dict(*a, **kw).items():
            sd[f"v_head.{k}"] = v
        return sd

    def post_init(self, state_dict):
        head = {k[len("v_head."):]: v for k, v in state_dict.items() if k.startswith("v_head.")}
        if head:
            self.v_head.load_state_dict(head, strict=False)

    def save_pretrained(self, path, **kw):
        self.pretrained_model.save_pretrained(path, **kw)
        import os

        torch.save(self.v_head.state_dict(), os.path.join(path, "v_head.pt"))
