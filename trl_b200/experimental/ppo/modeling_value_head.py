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


class PreTrainedModelWrapper(nn.Module):
    """A model plus extra heads behind one ``nn.Module``: keeps the wrapped model's configuration and its
    gradient-checkpointing switches reachable, filters the head arguments out of ``from_pretrained`` and saves the
    heads next to the base checkpoint (trl/experimental/ppo/modeling_value_head.py:52-330)."""

    transformers_parent_class = None
    supported_args: tuple = ()
    supported_modules = ("v_head",)
    supported_rm_modules = ("score",)

    def __init__(self, pretrained_model=None, score_module=None, supports_rm_adapter=False, rm_adapter_name=None, **kw):
        super().__init__()
        self.pretrained_model = pretrained_model
        self.config = pretrained_model.config
        self.is_loaded_in_8bit = self.is_loaded_in_4bit = False
        self.is_sequential_parallel = False
        for name in ("gradient_checkpointing_disable", "gradient_checkpointing_enable", "enable_input_require_grads"):
            if hasattr(pretrained_model, name):
                setattr(self, name, getattr(pretrained_model, name))
        self.supports_rm_adapter, self.rm_adapter_name, self.policy_adapter_name = supports_rm_adapter, rm_adapter_name, "default"
        if score_module is not None:
            self.score = score_module

    @classmethod
    def _split_kwargs(cls, kwargs):
        head = {k: v for k, v in kwargs.items() if k in (cls.supported_args or ())}
        rest = {k: v for k, v in kwargs.items() if k not in head}
        return head, rest

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, *model_args, **kwargs):
        head_kw, kw = cls._split_kwargs(kwargs)
        model = pretrained_model_name_or_path
        path = None
        if isinstance(model, str):
            from ...trainer.utils import create_model_from_path

            path = model
            model = create_model_from_path(model, **kw)
        wrapped = cls(model, **head_kw)
        if path is not None:
            import os

            f = os.path.join(path, "v_head.pt")
            if os.path.exists(f):
                wrapped.post_init({f"v_head.{k}": v for k, v in torch.load(f, map_location="cpu", weights_only=True).items()})
        return wrapped

    def post_init(self, *a, **kw):
        raise NotImplementedError

    def compute_reward_score(self, input_ids, attention_mask=None, **kw):
        """Score of the last real token from the ``score`` module (reward-adapter use of the wrapper)."""
        if not hasattr(self, "score"):
            raise ValueError("this wrapper was built without a score module")
        flat, ctx, _ = self.pretrained_model.pack_inputs(input_ids, attention_mask)
        hidden = self.pretrained_model.forward_hidden(flat, ctx)
        return self.score(hidden[(ctx.cu_seqlens[1:] - 1).long()])


class AutoModelForSeq2SeqLMWithValueHead(PreTrainedModelWrapper):
    """Encoder-decoder counterpart of the value-head wrapper.  The native model families are decoder-only, so there is
    nothing to wrap: construction fails with that message instead of an import error at the call site."""

    lm_head_namings = ["lm_head", "embed_out", "output_projection"]
    supported_args = ("summary_dropout_prob", "v_head_initializer_range", "v_head_init_strategy")

    def __init__(self, pretrained_model=None, **kw):
        raise NotImplementedError("encoder-decoder models have no native implementation in this framework; "
                                  "use AutoModelForCausalLMWithValueHead with a decoder-only model")


class AutoModelForCausalLMWithValueHead(PreTrainedModelWrapper):
    supported_args = ("summary_dropout_prob", "v_head_initializer_range", "v_head_init_strategy")

    def __init__(self, pretrained_model: CausalLM, summary_dropout_prob: float = 0.0, v_head_initializer_range: float = 0.2,
                 v_head_init_strategy: str | None = None, **kw):
        super().__init__(pretrained_model, **kw)
        cfg = pretrained_model.config
        p = next(pretrained_model.parameters())
        self.v_head = ValueHead(cfg.hidden_size, summary_dropout_prob, dtype=p.dtype, device=p.device)
        if v_head_init_strategy == "normal":
            self.v_head.summary.weight.data.normal_(mean=0.0, std=v_head_initializer_range)
            self.v_head.summary.bias.data.zero_()

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
