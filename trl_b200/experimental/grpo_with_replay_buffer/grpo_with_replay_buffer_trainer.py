"""GRPO with a replay buffer (trl/experimental/grpo_with_replay_buffer/grpo_with_replay_buffer_trainer.py:
ReplayBuffer :29-58, update/sample :516-760).

Groups whose rewards all coincide carry no gradient.  Groups with reward variance are kept in a bounded min-heap
scored by sum(|advantage| * std); a zero-variance group of the current batch is replaced by a group sampled from the
heap (probability proportional to its score) together with that group's stored behaviour/reference log-probs."""
from __future__ import annotations

import heapq
import itertools

import torch

from ...trainer.grpo_trainer import GRPOTrainer
from .grpo_with_replay_buffer_config import GRPOWithReplayBufferConfig


class ReplayBuffer:
    def __init__(self, max_size: int):
        self.max_size, self.heap = max_size, []
        self._tie = itertools.count()  # heap entries never compare their payloads

    def add(self, scores, data):
        for s, d in zip(scores, data, strict=True):
            item = (float(s), next(self._tie), d)
            if len(self.heap) < self.max_size:
                heapq.heappush(self.heap, item)
            elif s > self.heap[0][0]:
                heapq.heapreplace(self.heap, item)

    def sample(self, num_samples: int):
        if not self.heap:
            return None
        scores = torch.tensor([h[0] for h in self.heap], dtype=torch.float32).clamp(min=1e-12)
        idx = torch.multinomial(scores / scores.sum(), num_samples, replacement=num_samples > len(self.heap)).tolist()
        return [self.heap[i][2] for i in idx]

    def __len__(self):
        return len(self.heap)


def _fit_cols(t: torch.Tensor, width: int) -> torch.Tensor:
    return t[:, :width] if t.shape[1] >= width else torch.nn.functional.pad(t, (0, width - t.shape[1]))


class GRPOWithReplayBufferTrainer(GRPOTrainer):
    _tag_names = ["trl", "grpo-replay-buffer"]

    def __init__(self, model, reward_funcs, args: GRPOWithReplayBufferConfig | None = None, **kw):
        args = args or GRPOWithReplayBufferConfig("model-GRPO-replay")
        super().__init__(model, reward_funcs, args, **kw)
        self.replay_buffer = ReplayBuffer(args.replay_buffer_size) if args.replay_buffer_size > 0 else None

    _ROW_KEYS = ("completion_mask", "old_per_token_logps", "ref_per_token_logps", "importance_sampling_ratio",
                 "sampling_per_token_logps", "tool_mask")

    def _generate_and_score_completions(self, inputs):
        out = super()._generate_and_score_completions(inputs)
        if self.replay_buffer is None or not self.model.training:
            return out
        ng = self.num_generations
        adv = out["advantages"]
        B = adv.shape[0]
        if adv.ndim != 1 or B % ng:
            return out
        std = getattr(self, "_last_group_std", None)
        std = torch.ones_like(adv) if std is None else std.to(adv)
        groups = adv.view(-1, ng)
        has_var = groups.abs().sum(1) > 0
        width = out["completion_mask"].shape[1]
        scores, payloads = [], []
        for g in has_var.nonzero().flatten().tolist():
            rows = slice(g * ng, (g + 1) * ng)
            d = {"prompt_ids": out["prompt_ids"][rows], "completion_ids_list": out["completion_ids_list"][rows],
                 "advantages": adv[rows].clone()}
            for k in self._ROW_KEYS:
                if k in out and torch.is_tensor(out[k]) and out[k].ndim == 2 and out[k].shape[0] == B:
                    d[k] = out[k][rows].clone()
            scores.append(float((adv[rows].abs() * std[rows]).sum()))
            payloads.append(d)
        flat = [g for g in (~has_var).nonzero().flatten().tolist()]
        if flat and len(self.replay_buffer):
            sampled = self.replay_buffer.sample(len(flat))
            for g, d in zip(flat, sampled):
                rows = slice(g * ng, (g + 1) * ng)
                out["prompt_ids"][rows] = d["prompt_ids"]
                out["completion_ids_list"][rows] = d["completion_ids_list"]
                out["advantages"][rows] = d["advantages"].to(adv)
                for k in self._ROW_KEYS:
                    if k in d and k in out:
                        w = max(width, d[k].shape[1])
                        if w > out[k].shape[1]:
                            out[k] = _fit_cols(out[k], w)
                        out[k][rows] = _fit_cols(d[k].to(out[k]), out[k].shape[1])
            self._metrics["train"]["replay_buffer/replaced_groups"].append(float(len(flat)))
        if payloads:
            self.replay_buffer.add(scores, payloads)
        self._metrics["train"]["replay_buffer/size"].append(float(len(self.replay_buffer)))
        return out
