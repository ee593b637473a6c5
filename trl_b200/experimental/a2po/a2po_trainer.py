"""A*-PO: optimal-advantage regression (trl/experimental/a2po/a2po_trainer.py: stage 1 :213-277, inputs :279-333,
loss :335-349).

Stage 1 (once, before training): for every prompt draw ``num_value_samples`` completions from the reference policy and
estimate  V*(x) = beta1 * log mean exp(r / beta1).  Stage 2: one on-policy completion per prompt,
loss = (beta2 * log(pi/pi_ref)(y|x) - (r(x, y) - V*(x)))^2."""
from __future__ import annotations

import math
from typing import Any

import torch

from ...data_utils import is_conversational
from ...parallel import dist as D
from ...trainer.online_base import OnlineTrainer
from .._distill import sample_completions
from .a2po_config import A2POConfig


class A2POTrainer(OnlineTrainer):
    _tag_names = ["trl", "a2po"]
    _name = "A2PO"

    def __init__(self, model, reward_funcs, args: A2POConfig | None = None, **kw):
        args = args or A2POConfig("model-A2PO")
        super().__init__(model, reward_funcs, args, **kw)
        self._optimal_values: dict = {}
        self._gen_cache: dict = {}

    @staticmethod
    def _key(prompt) -> str:
        return prompt if isinstance(prompt, str) else repr(prompt)

    def _score(self, examples, prompts, completion_ids):
        tok = self.processing_class
        texts = tok.batch_decode(completion_ids, skip_special_tokens=True)
        comps = [[{"role": "assistant", "content": t}] for t in texts] if is_conversational(examples[0]) else texts
        rw = self._calculate_rewards([dict(e) for e in examples], prompts, comps, completion_ids)
        n = len(prompts)
        return (rw[D.rank() * n:(D.rank() + 1) * n] * self.reward_weights.to(rw.device)[None]).nansum(1)

    def _estimate_optimal_values(self):
        a = self.args
        n = a.num_value_samples
        ref = self.ref_model if self.ref_model is not None else self.model
        rows = list(self.train_dataset) + (list(self.eval_dataset) if self.eval_dataset is not None else [])
        rows = rows[D.rank()::D.world_size()]
        values, all_incorrect = {}, set()
        bs = max(1, a.per_device_train_batch_size)
        for s in range(0, len(rows), bs):
            batch = rows[s:s + bs]
            prompts = [ex["prompt"] for ex in batch]
            p_ids = self._tokenize_prompts(prompts)
            rep_ids = [p for p in p_ids for _ in range(n)]
            comps = sample_completions(ref, rep_ids, self.max_completion_length, temperature=a.temperature,
                                       top_p=a.top_p, top_k=a.top_k, eos_token_id=self.eos_token_id, seed=a.seed + s,
                                       engine_cache=self._gen_cache)
            r = self._score([ex for ex in batch for _ in range(n)], [p for p in prompts for _ in range(n)], comps)
            r = r.view(len(batch), n)
            v = a.beta1 * (torch.logsumexp(r / a.beta1, dim=1) - math.log(n))
            for j, pr in enumerate(prompts):
                values[self._key(pr)] = float(v[j])
                if float(r[j].sum()) == 0:
                    all_incorrect.add(self._key(pr))
        merged = {}
        for part in D.gather_object([values]) if D.world_size() > 1 else [values]:
            merged.update(part)
        bad = set().union(*D.gather_object([all_incorrect])) if D.world_size() > 1 else all_incorrect
        self._optimal_values = merged
        if a.filter_all_incorrect and bad:
            kept = [ex for ex in self.train_dataset if self._key(ex["prompt"]) not in bad]
            if kept:
                self.train_dataset = kept

    def train(self, *args, **kw):
        if not self._optimal_values:
            self._estimate_optimal_values()
        return super().train(*args, **kw)

    def _generate_and_score_completions(self, inputs: list[dict]) -> dict[str, Any]:
        dev = self.args.device
        prompts = [x["prompt"] for x in inputs]
        prompt_ids, completion_ids, _, _ = self._generate(prompts)
        rewards = self._score(inputs, prompts, completion_ids)
        v_star = torch.tensor([self._optimal_values.get(self._key(p), 0.0) for p in prompts], device=dev)
        with torch.no_grad():
            ref_lp = self._ref_logps(prompt_ids, completion_ids, len(prompt_ids))
        lens = torch.tensor([len(c) for c in completion_ids], device=dev)
        mask = (torch.arange(ref_lp.shape[1], device=dev)[None] < lens[:, None]).float()
        m = self._metrics["train" if self.model.training else "eval"]
        m["reward"].append(D.gather(rewards.mean().reshape(1)).mean())
        m["v_star"].append(D.gather(v_star.mean().reshape(1)).mean())
        return {"prompt_ids": prompt_ids, "completion_ids_list": completion_ids, "rewards": rewards, "v_star": v_star,
                "ref_logps": (ref_lp * mask).sum(1), "completion_mask": mask}

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        lp, _ = self._get_per_token_logps_and_entropies(model, inputs["prompt_ids"], inputs["completion_ids_list"])
        Tc = lp.shape[1]
        mask = inputs["completion_mask"]
        mask = mask[:, :Tc] if mask.shape[1] >= Tc else torch.nn.functional.pad(mask, (0, Tc - mask.shape[1]))
        policy = (lp * mask).sum(1)
        implicit = self.args.beta2 * (policy - inputs["ref_logps"])
        target = inputs["rewards"] - inputs["v_star"]
        loss = ((implicit - target) ** 2).mean() / self.current_gradient_accumulation_steps
        m = self._metrics["train" if model.training else "eval"]
        m["implicit_reward"].append(implicit.detach().mean())
        m["advantage"].append(target.mean())
        return (loss, None) if return_outputs else loss
