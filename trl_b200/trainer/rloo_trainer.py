"""REINFORCE Leave-One-Out.

Behaviour of trl/trainer/rloo_trainer.py: same rollout/buffering skeleton as GRPO; the KL penalty is
folded into the reward, ``r~ = r - beta * sum_t(logp_old - logp_ref)`` (:1526-1535); the baseline of a
sample is the mean reward of the other scorable samples of its group (:1544-1554); optional advantage
normalisation; sequence-level PPO clip on ``sum_t logp`` (:1683-1694).
"""
from __future__ import annotations

import os
from typing import Any

import torch

from ..data_utils import is_conversational
from ..parallel import dist as D
from .grpo_config import RLOOConfig
from .online_base import OnlineTrainer
from .utils import defer_mean, defer_ratio, nanstd


class RLOOTrainer(OnlineTrainer):
    _tag_names = ["trl", "rloo"]
    _name = "RLOO"

    def __init__(self, model, reward_funcs, args: RLOOConfig | None = None, train_dataset=None, eval_dataset=None,
                 processing_class=None, reward_processing_classes=None, callbacks=None, optimizers=(None, None),
                 peft_config=None):
        if args is None:
            name = model if isinstance(model, str) else getattr(model, "name_or_path", "model")
            args = RLOOConfig(f"{os.path.basename(str(name).rstrip('/'))}-RLOO")
        super().__init__(model, reward_funcs, args, train_dataset, eval_dataset, processing_class,
                         reward_processing_classes, callbacks, optimizers, peft_config)
        self.normalize_advantages = args.normalize_advantages
        self.reward_clip_range = args.reward_clip_range

    def _generate_and_score_completions(self, inputs: list[dict]) -> dict[str, Any]:
        a = self.args
        dev = a.device
        mode = "train" if self.model.training else "eval"
        prompts = [x["prompt"] for x in inputs]
        images = [x.get("images") if "images" in x else ([x["image"]] if x.get("image") is not None else None)
                  for x in inputs]
        prompt_ids, completion_ids, _, extras = self._generate(prompts, images if any(i for i in images) else None)
        pixel_list = extras.pop("pixel_values_list", None)  # vision-language prompts
        B = len(prompts)
        comp_lens = torch.tensor([len(c) for c in completion_ids], device=dev)
        Tc = max(1, int(comp_lens.max()))
        completion_mask = (torch.arange(Tc, device=dev)[None] < comp_lens[:, None]).int()
        eos_or_pad = {self.eos_token_id, self.pad_token_id}
        is_trunc = torch.tensor([len(c) == 0 or c[-1] not in eos_or_pad for c in completion_ids], device=dev)
        if self.mask_truncated_completions:
            completion_mask = completion_mask * (~is_trunc)[:, None].int()
        bs = a.per_device_train_batch_size if mode == "train" else a.per_device_eval_batch_size
        maskf = completion_mask.float()
        with torch.no_grad():
            old_logps, _ = self._get_per_token_logps_and_entropies(self.model, prompt_ids, completion_ids, bs,
                                                                   pixel_values_list=pixel_list)
            old_sum = (old_logps * maskf).sum(1)
            if self.beta != 0.0:
                ref_logps = self._ref_logps(prompt_ids, completion_ids, bs, pixel_list)
                kl = ((old_logps - ref_logps) * maskf).sum(1)
            else:
                kl = None
        tok = self.processing_class
        texts = tok.batch_decode(completion_ids, skip_special_tokens=True)
        completions = [[{"role": "assistant", "content": c}] for c in texts] if is_conversational(inputs[0]) else texts
        rewards_per_func = self._calculate_rewards(inputs, prompts, completions, completion_ids)
        w = self.reward_weights.to(dev)
        unscorable = torch.isnan(rewards_per_func).all(dim=1)
        rewards = (rewards_per_func * w[None]).nansum(dim=1)
        if self.reward_clip_range is not None:
            rewards = rewards.clamp(min=self.reward_clip_range[0], max=self.reward_clip_range[1])
        if kl is not None:
            rewards = rewards - self.beta * D.gather(kl)
        rewards[unscorable] = float("nan")
        ng = self.num_generations if mode == "train" else self.num_generations_eval
        g = rewards.view(-1, ng)
        valid = ~torch.isnan(g)
        cnt = valid.sum(1, keepdim=True)
        tot = torch.nansum(g, dim=1, keepdim=True)
        # leave-one-out mean over the *other* scorable samples of the group
        baseline = (tot - torch.nan_to_num(g, nan=0.0)) / (cnt - 1).clamp(min=1)
        adv = (g - baseline).view(-1)
        std = nanstd(g, dim=1).repeat_interleave(ng) if ng > 1 else torch.zeros_like(rewards)
        if self.normalize_advantages:
            adv = (adv - torch.nanmean(adv)) / (nanstd(adv) + 1e-4)
        adv = torch.nan_to_num(adv, nan=0.0)
        sl = slice(D.rank() * B, (D.rank() + 1) * B)
        m = self._metrics[mode]
        if mode == "train":
            self._total_train_tokens += int(D.gather((torch.tensor([len(p) for p in prompt_ids], device=dev).sum()
                                                      + comp_lens.sum()).reshape(1)).sum())
        m["num_tokens"].append(float(self._total_train_tokens))
        agg_len = D.gather(comp_lens.float())
        m["completions/mean_length"].append(agg_len.mean())
        m["completions/min_length"].append(agg_len.min())
        m["completions/max_length"].append(agg_len.max())
        m["completions/clipped_ratio"].append(D.gather(is_trunc.float()).mean())
        for i, name in enumerate(self.reward_func_names):
            m[f"rewards/{name}/mean"].append(torch.nanmean(rewards_per_func[:, i]))
            m[f"rewards/{name}/std"].append(nanstd(rewards_per_func[:, i]))
        m["reward"].append(torch.nanmean(rewards))
        m["reward_std"].append(torch.nanmean(std))
        m["frac_reward_zero_std"].append(torch.isclose(std, torch.zeros_like(std)).float().mean())
        if kl is not None:
            m["kl"].append(D.gather(kl / maskf.sum(1).clamp(min=1)).mean())
        out = {"prompt_ids": prompt_ids, "completion_ids_list": completion_ids, "completion_mask": completion_mask,
               "advantages": adv[sl], "old_logps": old_sum}
        if pixel_list is not None:
            out["pixel_values_list"] = pixel_list
        return out

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        mode = "train" if model.training else "eval"
        m = self._metrics[mode]
        logps, ents = self._get_per_token_logps_and_entropies(model, inputs["prompt_ids"], inputs["completion_ids_list"],
                                                              compute_entropy=True,
                                                              pixel_values_list=inputs.get("pixel_values_list"))
        Tc = logps.shape[1]
        maskf = inputs["completion_mask"].float()
        maskf = maskf[:, :Tc] if maskf.shape[1] >= Tc else torch.nn.functional.pad(maskf, (0, Tc - maskf.shape[1]))
        seq_lp = (logps * maskf).sum(1)
        adv = inputs["advantages"]
        ratio = torch.exp(seq_lp - inputs["old_logps"])
        clipped = torch.clamp(ratio, 1 - self.epsilon_low, 1 + self.epsilon_high)
        per_seq = -torch.min(ratio * adv, clipped * adv)
        ga = self.current_gradient_accumulation_steps if mode == "train" else 1.0
        loss = per_seq.mean() / ga
        aux = getattr(self, "_last_aux_loss", None)
        if aux is not None:
            loss = loss + self.args.router_aux_loss_coef * aux / ga
        with torch.no_grad():  # local partial results; reduced once per logging step
            m["entropy"].append(defer_ratio((ents * maskf).sum(), maskf.sum()))
            low = ((ratio < 1 - self.epsilon_low) & (adv < 0)).float()
            high = ((ratio > 1 + self.epsilon_high) & (adv > 0)).float()
            m["clip_ratio/low_mean"].append(defer_mean(low.mean()))
            m["clip_ratio/high_mean"].append(defer_mean(high.mean()))
            m["clip_ratio/region_mean"].append(defer_mean(((low + high) > 0).float().mean()))
        return loss

    def prediction_step(self, model, inputs, prediction_loss_only=True, ignore_keys=None):
        inputs = self._prepare_inputs(inputs)
        with torch.no_grad():
            loss = self.compute_loss(model, inputs)
        return loss.detach(), None, None
