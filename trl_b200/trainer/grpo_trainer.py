"""Group Relative Policy Optimization.

Algorithm and option surface of trl/trainer/grpo_trainer.py: generation + scoring
(:2260-2853), advantages (:2679-2738), loss variants grpo/bnpo/dr_grpo/dapo/cispo/
sapo/luspo/vespo (:3054-3150), token- or sequence-level importance sampling, k3 KL,
two-sided clip, off-policy sequence mask, top-entropy-quantile mask, entropy bonus
(static / adaptive with a checkpointed controller), rollout importance-sampling
correction.  On GPUs the default loss family (token-level ratio, clip, KL, masked
normalisation and all metric sums) is one fused kernel (`ops.cuda.grpo_loss`).
"""
from __future__ import annotations

import json
import os
from typing import Any

import torch

from ..data_utils import is_conversational
from ..parallel import dist as D
from .grpo_config import GRPOConfig
from .online_base import OnlineTrainer
from .utils import balanced_partition, defer_mean, defer_ratio, nanmax, nanmin, nanstd, pad


class GRPOTrainer(OnlineTrainer):
    _tag_names = ["trl", "grpo"]
    _name = "GRPO"

    def __init__(self, model, reward_funcs, args: GRPOConfig | None = None, train_dataset=None, eval_dataset=None,
                 processing_class=None, reward_processing_classes=None, callbacks=None, optimizers=(None, None),
                 quantization_config=None, peft_config=None, tools=None, rollout_func=None, environment_factory=None):
        if args is None:
            name = model if isinstance(model, str) else getattr(model, "name_or_path", "model")
            args = GRPOConfig(f"{os.path.basename(str(name).rstrip('/'))}-GRPO")
        if quantization_config is not None:
            raise NotImplementedError("quantised policies: no 4/8-bit weight kernels in this build")
        super().__init__(model, reward_funcs, args, train_dataset, eval_dataset, processing_class,
                         reward_processing_classes, callbacks, optimizers, peft_config, tools, rollout_func,
                         environment_factory)
        a = args
        self.loss_type, self.scale_rewards = a.loss_type, a.scale_rewards
        self.importance_sampling_level = a.importance_sampling_level
        self.multi_objective_aggregation = a.multi_objective_aggregation
        self.top_entropy_quantile = a.top_entropy_quantile
        self.off_policy_mask_threshold = a.off_policy_mask_threshold
        self.vllm_importance_sampling_correction = a.vllm_importance_sampling_correction
        self.entropy_coef = a.entropy_coef
        self._entropy_bonus_enabled = a.entropy_coef != 0.0 or a.use_adaptive_entropy
        # entropy measured over the previous optimizer step; with the adaptive controller the bonus stays off until one was measured
        self._last_world_entropy = float("inf")
        self._entropy_window_stats = None
        if self.tools and not self.rollout_func:
            from .tool_loop import ToolLoop

            self._tool_loop = ToolLoop(self, self.tools, a.max_tool_calling_iterations)
        else:
            self._tool_loop = None

    # ---- generation + scoring ------------------------------------------------------------------------------
    def _generate_and_score_completions(self, inputs: list[dict]) -> dict[str, Any]:
        a = self.args
        dev = a.device
        mode = "train" if self.model.training else "eval"
        prompts = [x["prompt"] for x in inputs]
        images = [x.get("images") if "images" in x else ([x["image"]] if x.get("image") is not None else None)
                  for x in inputs]
        images = images if any(i for i in images) else None
        if self._tool_loop is not None:
            if images is not None:
                raise ValueError("tool calling and image prompts cannot be combined")
            prompt_ids, completion_ids, sampling_logps, extras = self._tool_loop.generate(prompts)
        else:
            prompt_ids, completion_ids, sampling_logps, extras = self._generate(prompts, images)
        pixel_list = extras.pop("pixel_values_list", None)
        tool_mask = extras.pop("env_mask", extras.pop("tool_mask", None))
        B = len(prompts)
        comp_lens = torch.tensor([len(c) for c in completion_ids], device=dev)
        eos_or_pad = {self.eos_token_id, self.pad_token_id}
        is_trunc = torch.tensor([len(c) == 0 or c[-1] not in eos_or_pad for c in completion_ids], device=dev)
        # ---- rewards and advantages (on the completions this rank generated) -----------------------------------------
        tok = self.processing_class
        completions_text = tok.batch_decode(completion_ids, skip_special_tokens=True)
        if prompts and is_conversational(inputs[0]):
            completions = [[{"role": "assistant", "content": c}] for c in completions_text]
        else:
            completions = completions_text
        for k, v in extras.items():
            if isinstance(v, list) and len(v) == B:
                for ex, val in zip(inputs, v):
                    ex[k] = val
        rewards_per_func = self._calculate_rewards(inputs, prompts, completions, completion_ids)
        ng = self.num_generations if mode == "train" else self.num_generations_eval
        advantages, rewards, std_rewards, is_std_zero = self._advantages(rewards_per_func, ng)
        sl = slice(D.rank() * B, (D.rank() + 1) * B)
        all_adv = advantages.clone()
        advantages = advantages[sl]
        self._last_group_std = std_rewards[sl] if std_rewards.ndim and std_rewards.shape[0] == all_adv.shape[0] else None
        gen_comp_lens, gen_is_trunc, gen_prompt_ids = comp_lens, is_trunc, prompt_ids  # for the metrics below
        # ---- even out the training work: completions change ranks, token ids travel, activations never do ------------
        if (mode == "train" and D.world_size() > 1 and getattr(a, "balance_completions", True) and pixel_list is None):
            (prompt_ids, completion_ids, sampling_logps, tool_mask, advantages, self._last_group_std) = \
                self._rebalance_across_ranks(prompt_ids, completion_ids, sampling_logps, tool_mask, advantages,
                                             self._last_group_std)
            comp_lens = torch.tensor([len(c) for c in completion_ids], device=dev)
            is_trunc = torch.tensor([len(c) == 0 or c[-1] not in eos_or_pad for c in completion_ids], device=dev)
        Tc = max(1, int(comp_lens.max()))
        completion_mask = (torch.arange(Tc, device=dev)[None] < comp_lens[:, None]).int()
        if self.mask_truncated_completions:
            completion_mask = completion_mask * (~is_trunc)[:, None].int()
        if tool_mask is not None:
            tm = pad([torch.tensor(t, device=dev) for t in tool_mask], 0, "right")
            tm = torch.nn.functional.pad(tm, (0, Tc - tm.shape[1]))
        else:
            tm = None
        loss_mask = completion_mask if tm is None else completion_mask * tm
        num_items_in_batch = D.gather(loss_mask.sum().reshape(1)).sum().float()
        bs = a.per_device_train_batch_size if mode == "train" else a.per_device_eval_batch_size
        out: dict[str, Any] = {}
        with torch.no_grad():
            generate_every = a.steps_per_generation * self.num_iterations
            need_old = a.gradient_accumulation_steps % generate_every != 0 or (
                self.use_vllm and self.vllm_importance_sampling_correction and sampling_logps is not None)
            old_logps = None
            if need_old:
                with self._profile("old_logps"):
                    old_logps, _ = self._get_per_token_logps_and_entropies(self.model, prompt_ids, completion_ids, bs,
                                                                           pixel_values_list=pixel_list)
            if self.use_vllm and self.vllm_importance_sampling_correction and sampling_logps is not None:
                slp = pad([torch.tensor(l, dtype=torch.float32, device=dev) for l in sampling_logps], 0.0, "right")
                slp = torch.nn.functional.pad(slp, (0, Tc - slp.shape[1]))
                out["sampling_per_token_logps"] = slp
                out["importance_sampling_ratio"] = self._rollout_is_ratio(old_logps, slp, loss_mask)
            if self.beta != 0.0:
                with self._profile("ref_logps"):
                    out["ref_per_token_logps"] = self._ref_logps(prompt_ids, completion_ids, bs, pixel_list)
            if old_logps is not None:
                out["old_per_token_logps"] = old_logps
        # ---- metrics ----------------------------------------------------------------------------------------------
        m = self._metrics[mode]
        if mode == "train":
            self._total_train_tokens += int(D.gather((torch.tensor([len(p) for p in gen_prompt_ids], device=dev).sum()
                                                      + gen_comp_lens.sum()).reshape(1)).sum())
        m["num_tokens"].append(float(self._total_train_tokens))
        agg_len = D.gather(gen_comp_lens.float())
        if mode == "train":  # completion tokens produced by the whole job (each completion counted once)
            self._total_generated_tokens = getattr(self, "_total_generated_tokens", 0) + int(agg_len.sum())
        m["completions/mean_length"].append(agg_len.mean())
        m["completions/min_length"].append(agg_len.min())
        m["completions/max_length"].append(agg_len.max())
        agg_trunc = D.gather(gen_is_trunc.float())
        term = agg_len[agg_trunc == 0]
        m["completions/clipped_ratio"].append(agg_trunc.mean())
        if term.numel() == 0:
            term = torch.zeros(1, device=dev)
        m["completions/mean_terminated_length"].append(term.mean())
        m["completions/min_terminated_length"].append(term.min())
        m["completions/max_terminated_length"].append(term.max())
        for i, name in enumerate(self.reward_func_names):
            col = rewards_per_func[:, i]
            m[f"rewards/{name}/mean"].append(torch.nanmean(col))
            m[f"rewards/{name}/std"].append(nanstd(col))
        m["reward"].append(torch.nanmean(rewards))
        m["reward_std"].append(torch.nanmean(std_rewards))
        m["frac_reward_zero_std"].append(is_std_zero.float().mean())
        for k, v in getattr(self, "_extra_metrics", {}).items():
            m[k].append(sum(v) / max(1, len(v)))
        if "importance_sampling_ratio" in out:
            r = out["importance_sampling_ratio"]
            flat = r[loss_mask.bool()] if r.shape == loss_mask.shape else r.flatten()
            if flat.numel():
                m["sampling/importance_sampling_ratio/min"].append(flat.min())
                m["sampling/importance_sampling_ratio/mean"].append(flat.mean())
                m["sampling/importance_sampling_ratio/max"].append(flat.max())
            d = (out["old_per_token_logps"] - out["sampling_per_token_logps"]).abs()[loss_mask.bool()]
            if d.numel():
                m["sampling/sampling_logp_difference/mean"].append(d.mean())
                m["sampling/sampling_logp_difference/max"].append(d.max())
        if self.log_completions:
            pt = D.gather_object([p if isinstance(p, str) else p for p in prompts])
            ct = D.gather_object(completions_text)
            self._logs["prompt"].extend(pt)
            self._logs["completion"].extend(ct)
            for i, name in enumerate(self.reward_func_names):
                self._logs["rewards"][name].extend(rewards_per_func[:, i].tolist())
            self._logs["advantages"].extend(all_adv.tolist())
            for k, v in getattr(self, "_extra_cols", {}).items():
                self._logs["extra"][k].extend(D.gather_object(v))
        if pixel_list is not None:
            out["pixel_values_list"] = pixel_list
        out.update({
            "prompt_ids": prompt_ids, "completion_ids_list": completion_ids,
            "completion_mask": completion_mask, "advantages": advantages,
            "num_items_in_batch": num_items_in_batch,
        })
        if tm is not None:
            out["tool_mask"] = tm
        return out

    def _rebalance_across_ranks(self, prompt_ids, completion_ids, sampling_logps, tool_mask, advantages, group_std):
        """Deals the job's completions to the ranks so that every rank trains on the same amount of work.

        Completion lengths differ a lot (an EOS can come at any step), and every rank trains on what it generated, so
        the rank with the longest completions sets the step time of all.  After scoring (advantages are final: a
        completion no longer needs its group), all ranks exchange the token ids and per-sample scalars, run the same
        deterministic partition and keep their share: equal counts per rank, costs ``L + L^2 / s`` (linear layers +
        attention) balanced by longest-first assignment to the least loaded rank.  Only token ids travel; log-probs
        and activations are computed after the exchange, on the owner.  The reference balances ``sum L^2`` the same
        way for its asynchronous trainer (trl/experimental/async_grpo/async_grpo_trainer.py:303-406).
        """
        B, W, r = len(prompt_ids), D.world_size(), D.rank()
        adv = advantages.tolist()
        std = group_std.tolist() if group_std is not None else [None] * B
        recs = D.gather_object([(prompt_ids[i], completion_ids[i], None if sampling_logps is None else sampling_logps[i],
                                 None if tool_mask is None else tool_mask[i], adv[i], std[i]) for i in range(B)])
        cfg = getattr(self.model, "config", None)
        try:  # sequence length at which attention costs as much as the linear layers
            s = float(cfg.num_parameters()) / (2.0 * cfg.hidden_size * cfg.num_hidden_layers)
        except Exception:
            s = 32768.0
        lens = [len(x[0]) + len(x[1]) for x in recs]
        mine = balanced_partition([l + l * l / s for l in lens], W, B)[r]
        pick = [recs[i] for i in mine]
        dev = advantages.device
        new_adv = torch.tensor([x[4] for x in pick], dtype=advantages.dtype, device=dev)
        new_std = None if group_std is None else torch.tensor([x[5] for x in pick], dtype=group_std.dtype, device=dev)
        return ([x[0] for x in pick], [x[1] for x in pick], None if sampling_logps is None else [x[2] for x in pick],
                None if tool_mask is None else [x[3] for x in pick], new_adv, new_std)

    def _advantages(self, rewards_per_func, ng):
        dev = rewards_per_func.device
        w = self.reward_weights.to(dev)
        unscorable = torch.isnan(rewards_per_func).all(dim=1)
        if self.multi_objective_aggregation == "sum_then_normalize":
            rewards = (rewards_per_func * w[None]).nansum(dim=1)
            rewards[unscorable] = float("nan")
            mean_g = torch.nanmean(rewards.view(-1, ng), dim=1).repeat_interleave(ng)
            if self.scale_rewards in ("group", "none"):
                std = nanstd(rewards.view(-1, ng), dim=1).repeat_interleave(ng) if ng > 1 else torch.zeros_like(rewards)
            else:
                std = nanstd(rewards).expand_as(rewards) if rewards.numel() > 1 else torch.zeros_like(rewards)
            adv = rewards - mean_g
            if self.scale_rewards != "none":
                adv = adv / (std + 1e-4)
        elif self.multi_objective_aggregation == "normalize_then_sum":
            g = rewards_per_func.view(-1, ng, rewards_per_func.shape[1])
            mean_k = torch.nanmean(g, dim=1, keepdim=True)
            std_k = nanstd(g, dim=1, keepdim=True) if ng > 1 else torch.zeros_like(mean_k)
            rk = ((g - mean_k) / (std_k + 1e-4)).view(-1, rewards_per_func.shape[1])
            rewards = (rk * w[None]).nansum(dim=1)
            rewards[unscorable] = float("nan")
            std = nanstd(rewards).expand_as(rewards) if rewards.numel() > 1 else torch.zeros_like(rewards)
            adv = (rewards - torch.nanmean(rewards)) / (std + 1e-4)
        else:
            raise ValueError(f"Invalid multi_objective_aggregation: {self.multi_objective_aggregation}")
        is_std_zero = torch.isclose(std, torch.zeros_like(std))
        return torch.nan_to_num(adv, nan=0.0), rewards, std, is_std_zero

    def _rollout_is_ratio(self, train_logps, sampling_logps, mask):
        """Correction for the mismatch between the rollout engine's and the trainer's log-probs
        (modes of grpo_trainer.py:2579-2623)."""
        a = self.args
        mode = a.vllm_importance_sampling_mode
        diff = (train_logps - sampling_logps) * mask
        if mode.startswith("sequence"):
            lr = diff.sum(-1, keepdim=True)
        else:
            lr = diff
        ratio = torch.exp(lr)
        # a missing bound does not clip on that side (grpo_trainer.py:2596-2616)
        cmax = float("inf") if a.vllm_importance_sampling_clip_max is None else a.vllm_importance_sampling_clip_max
        cmin = float("-inf") if a.vllm_importance_sampling_clip_min is None else a.vllm_importance_sampling_clip_min
        if mode.endswith("truncate"):
            ratio = torch.clamp(ratio, min=cmin, max=cmax)
        else:
            ratio = ratio.masked_fill((ratio > cmax) | (ratio < cmin), 0.0)
        return ratio.expand_as(mask) if ratio.shape != mask.shape else ratio

    # ---- loss ----------------------------------------------------------------------------------------------------------
    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        if return_outputs:
            raise ValueError("The GRPOTrainer does not support returning outputs")
        return self._compute_loss(model, inputs)

    @staticmethod
    def get_off_policy_mask(advantages, per_token_logps, sampling_per_token_logps, mask, off_policy_threshold):
        kl = ((sampling_per_token_logps - per_token_logps.detach()) * mask).sum(-1, keepdim=True) / mask.sum(
            -1, keepdim=True).clamp(min=1.0)
        keep = (advantages >= 0) | (kl <= off_policy_threshold)
        return keep.to(per_token_logps.dtype)

    @staticmethod
    def get_gamma_weights(advantages, log_ratio_per_token, mask, importance_sampling_ratio, k_pos, lambda_pos, k_neg,
                          lambda_neg):
        """VESPO sequence weights: phi(w) = w^k exp(lambda (1 - w)) on the detached sequence ratio."""
        # numeric guards of grpo_trainer.py:2943-2990: token log-ratios are clamped to [-20, 20] before the sequence
        # sum, the rollout correction enters unmasked, log w is clamped again, lambda has a floor, NaN/inf -> finite
        lr = torch.clamp(log_ratio_per_token.detach(), -20.0, 20.0)
        seq = (lr * mask).sum(-1, keepdim=True)
        if importance_sampling_ratio is not None:
            isr = torch.log(importance_sampling_ratio.clamp_min(1e-8))
            seq = seq + (isr.sum(-1, keepdim=True) if isr.shape[-1] == mask.shape[-1] else isr)
        seq = torch.clamp(seq, -20.0, 20.0)
        k = torch.where(advantages >= 0, torch.full_like(advantages, k_pos), torch.full_like(advantages, k_neg))
        lam = torch.where(advantages >= 0, torch.full_like(advantages, lambda_pos),
                          torch.full_like(advantages, lambda_neg)).clamp(min=1e-4)
        logphi = k * seq + lam * (1 - torch.exp(seq))
        return torch.nan_to_num(torch.exp(logphi), nan=0.0, posinf=0.0, neginf=0.0).detach()

    def _compute_loss(self, model, inputs):
        a = self.args
        mode = "train" if self.model.training else "eval"
        m = self._metrics[mode]
        prompt_ids, completion_ids = inputs["prompt_ids"], inputs["completion_ids_list"]
        completion_mask = inputs["completion_mask"]
        mask = completion_mask if "tool_mask" not in inputs else completion_mask * inputs["tool_mask"]
        maskf = mask.float()
        logps, entropies = self._get_per_token_logps_and_entropies(model, prompt_ids, completion_ids,
                                                                   compute_entropy=True,
                                                                   pixel_values_list=inputs.get("pixel_values_list"),
                                                                   entropy_grad=self._entropy_bonus_enabled
                                                                   and torch.is_grad_enabled())
        ent_stat = entropies.detach()
        Tc = logps.shape[1]
        if maskf.shape[1] != Tc:  # the buffered mask is padded to the generation batch's longest completion
            maskf = maskf[:, :Tc] if maskf.shape[1] > Tc else torch.nn.functional.pad(maskf, (0, Tc - maskf.shape[1]))

        def fit(t):
            if t is None or t.ndim < 2 or t.shape[1] == Tc or t.shape[1] == 1:
                return t
            return t[:, :Tc] if t.shape[1] > Tc else torch.nn.functional.pad(t, (0, Tc - t.shape[1]))
        entropy_mask = None
        if self.top_entropy_quantile < 1.0:
            entropy_mask = self.get_high_entropy_mask(ent_stat, maskf, 1 - self.top_entropy_quantile)
        advantages = inputs["advantages"]
        adv2 = advantages[:, None] if advantages.ndim == 1 else advantages
        old = fit(inputs.get("old_per_token_logps"))
        ref = fit(inputs.get("ref_per_token_logps"))
        isr = fit(inputs.get("importance_sampling_ratio"))
        B = logps.shape[0]
        ga = self.current_gradient_accumulation_steps if mode == "train" else 1.0
        simple = (self.loss_type in ("grpo", "bnpo", "dr_grpo", "dapo") and self.importance_sampling_level == "token"
                  and entropy_mask is None and self.off_policy_mask_threshold is None and isr is None
                  and not a.use_bias_correction_kl and not self._entropy_bonus_enabled and advantages.ndim == 1)
        if simple and logps.is_cuda:
            from ..ops import cuda as K

            if self.loss_type == "grpo":
                row_scale = 1.0 / (maskf.sum(-1).clamp(min=1.0) * B * ga)
            elif self.loss_type == "bnpo":
                row_scale = (1.0 / (maskf.sum().clamp(min=1.0) * ga)).expand(B)
            elif self.loss_type == "dr_grpo":
                row_scale = torch.full((B,), 1.0 / (B * self.max_completion_length * ga), device=logps.device)
            else:
                row_scale = (D.world_size() / inputs["num_items_in_batch"].clamp(min=1.0)).expand(B)
            loss, stats = K.grpo_loss(logps, old, ref if self.beta != 0.0 else None, advantages, maskf, row_scale.float(),
                                      entropies, self.epsilon_low, self.epsilon_high, self.beta, a.delta)
            # local partial sums only: the cross-rank reduction happens once per logging step
            st = stats.detach().clone()
            if self.beta != 0.0:
                m["kl"].append(defer_ratio(st[1], st[4]))
            m["clip_ratio/low_mean"].append(defer_ratio(st[2], st[4]))
            m["clip_ratio/high_mean"].append(defer_ratio(st[3], st[4]))
            m["clip_ratio/region_mean"].append(defer_ratio(st[6], st[4]))
            m["entropy"].append(defer_ratio(st[7], st[4]))
            return self._add_aux(loss, m)
        # ---- general path (autograd over PyTorch ops) -----------------------------------------------------------------
        old = logps.detach() if old is None else old
        off_mask = None
        if self.off_policy_mask_threshold is not None:
            samp = fit(inputs.get("sampling_per_token_logps"))
            off_mask = self.get_off_policy_mask(adv2, logps, samp if samp is not None else old, maskf,
                                                self.off_policy_mask_threshold)
        log_ratio = logps - old
        if self.importance_sampling_level == "token":
            liw = log_ratio
        elif self.importance_sampling_level == "sequence_token":
            # GSPO-token: the sequence-level weight as value, the token's own log-prob as gradient path
            seq = ((log_ratio * maskf).sum(-1) / maskf.sum(-1).clamp(min=1.0))[:, None]
            liw = logps - logps.detach() + seq.detach()
        else:
            liw = ((log_ratio * maskf).sum(-1) / maskf.sum(-1).clamp(min=1.0))[:, None]
        coef_1 = torch.exp(liw)
        kl = None
        if self.beta != 0.0:
            kl = torch.exp(ref - logps) - (ref - logps) - 1
            if a.use_bias_correction_kl:
                kl = kl * coef_1
        if self.loss_type == "cispo":
            per_tok = -torch.clamp(coef_1, max=self.epsilon_high).detach() * adv2 * logps
        elif self.loss_type in ("grpo", "bnpo", "dr_grpo", "dapo", "luspo"):
            coef_2 = torch.clamp(coef_1, 1 - self.epsilon_low, 1 + self.epsilon_high)
            c1 = torch.clamp(coef_1, max=a.delta) if a.delta is not None else coef_1
            per_tok = -torch.min(c1 * adv2, coef_2 * adv2)
        elif self.loss_type == "gmpo":
            # geometric mean of the token ratios: clip in log space on the side the advantage pushes towards,
            # average over the sequence, exponentiate once (one weight per sequence)
            sgn = torch.where(adv2 > 0, torch.ones_like(adv2), -torch.ones_like(adv2))
            lo, hi = -float(getattr(a, "gmpo_log_clip", 0.4)), float(getattr(a, "gmpo_log_clip", 0.4))
            clipped = sgn * torch.minimum(sgn * log_ratio, sgn * torch.clamp(log_ratio, lo, hi))
            seq_w = torch.exp((clipped * maskf).sum(-1, keepdim=True) / maskf.sum(-1, keepdim=True).clamp(min=1.0))
            per_tok = (-seq_w * adv2).expand_as(logps)
        elif self.loss_type == "sapo":
            temps = torch.where(adv2 > 0, torch.full_like(adv2, a.sapo_temperature_pos),
                                torch.full_like(adv2, a.sapo_temperature_neg))
            per_tok = -(torch.sigmoid(temps * (coef_1 - 1)) * 4 / temps) * adv2
        elif self.loss_type == "vespo":
            phi = self.get_gamma_weights(adv2, log_ratio, maskf, isr, a.vespo_k_pos, a.vespo_lambda_pos, a.vespo_k_neg,
                                         a.vespo_lambda_neg)
            m["vespo/phi_seq_mean"].append(phi.mean().detach())
            per_tok = -phi * adv2 * logps
        else:
            raise ValueError(f"Unknown loss type: {self.loss_type}")
        if off_mask is not None:
            per_tok = per_tok * off_mask
        if entropy_mask is not None:
            per_tok = per_tok * entropy_mask
        if isr is not None and self.loss_type != "vespo":
            per_tok = per_tok * isr
        if kl is not None:
            per_tok = per_tok + self.beta * kl
        if self.loss_type in ("grpo", "sapo", "gmpo"):
            loss, normalizer = ((per_tok * maskf).sum(-1) / maskf.sum(-1).clamp(min=1.0)).mean(), ga
        elif self.loss_type == "bnpo":
            loss, normalizer = (per_tok * maskf).sum() / maskf.sum().clamp(min=1.0), ga
        elif self.loss_type == "dr_grpo":
            loss, normalizer = (per_tok * maskf).sum() / (B * self.max_completion_length), ga
        elif self.loss_type in ("cispo", "dapo", "vespo"):
            normalizer = inputs["num_items_in_batch"].clamp(min=1.0) / D.world_size()
            loss = (per_tok * maskf).sum()
        else:  # luspo
            loss, normalizer = (per_tok * maskf.sum(1, keepdim=True)).mean(), ga
        loss = loss / normalizer
        if self._entropy_bonus_enabled:
            # L = L_policy - coef * H with H the mean per-token entropy of the active tokens, differentiable through
            # the lm_head (grpo_trainer.py:3155-3215).  The term is scaled so that it accumulates to H over the
            # optimizer step whatever the loss type's own normaliser is.
            eff = maskf if entropy_mask is None else maskf * entropy_mask
            if self.loss_type in ("cispo", "dapo", "vespo"):
                entropy_loss = (entropies * eff).sum() / normalizer
            else:
                entropy_loss = (entropies * eff).sum() / eff.sum().clamp(min=1.0) / normalizer
            # coefficient and gate are those fixed at the end of the previous optimizer step, so that every
            # micro-batch of the window applies the same bonus
            apply_coef = self.entropy_coef
            if a.use_adaptive_entropy and not (self._last_world_entropy <= a.entropy_target):
                apply_coef = 0.0
            m["policy_loss"].append(defer_mean(loss.detach() * (1.0 if self.loss_type in ("cispo", "dapo", "vespo")
                                                                else normalizer)))
            loss = loss - apply_coef * entropy_loss
            if a.use_adaptive_entropy and mode == "train":
                # running [entropy sum, token count] of the accumulation window, kept on the device
                stats_w = torch.stack([(ent_stat * eff).sum(), eff.sum()])
                self._entropy_window_stats = stats_w if self._entropy_window_stats is None \
                    else self._entropy_window_stats + stats_w
                if getattr(self, "sync_gradients", True):
                    self._update_entropy_controller()
            if mode == "train" and getattr(self, "sync_gradients", True):
                m["entropy_coef"].append(self.entropy_coef)

        def mmean(x):
            if x.shape[1] == 1 and maskf.shape[1] != 1:  # one value per sequence (sequence-level importance sampling)
                return defer_ratio(x.sum(), torch.tensor(float(x.shape[0]), device=x.device))
            return defer_ratio((x * maskf).sum(), maskf.sum())
        m["entropy"].append(mmean(ent_stat))
        if kl is not None:
            m["kl"].append(mmean(kl.detach()))
        if self.loss_type in ("grpo", "bnpo", "dr_grpo", "dapo", "luspo"):
            low = ((coef_1 < 1 - self.epsilon_low) & (adv2 < 0)).float()
            high = ((coef_1 > 1 + self.epsilon_high) & (adv2 > 0)).float()
            m["clip_ratio/low_mean"].append(mmean(low))
            m["clip_ratio/high_mean"].append(mmean(high))
            m["clip_ratio/region_mean"].append(mmean(((low + high) > 0).float()))
        elif self.loss_type == "cispo":
            m["cispo_clip_ratio"].append(mmean(((coef_1 > self.epsilon_high) & (adv2 > 0)).float()))
        return self._add_aux(loss, m)

    def _add_aux(self, loss, m):
        aux = getattr(self, "_last_aux_loss", None)
        if aux is not None:
            loss = loss + self.args.router_aux_loss_coef * aux / self.current_gradient_accumulation_steps
            m["aux_loss"].append(aux.detach())
        return loss

    def get_high_entropy_mask(self, entropies, mask, threshold: float):
        """Keep tokens whose entropy is at or above the global ``threshold`` quantile (:1396-1432)."""
        local = entropies[mask.bool()].float()
        if D.world_size() > 1:
            n = torch.tensor([local.numel()], device=local.device)
            mx = int(D.all_reduce(n.clone(), "max"))
            padded = torch.cat([local, local.new_full((mx - local.numel(),), float("nan"))])
            allv = D.gather(padded)
            allv = allv[~torch.isnan(allv)]
        else:
            allv = local
        if allv.numel() == 0:
            return torch.zeros_like(entropies)
        thr = torch.quantile(allv, threshold)
        return ((entropies >= thr) & mask.bool()).float()

    # ---- adaptive entropy controller --------------------------------------------------------------------------------
    def _update_entropy_controller(self):
        """At the optimizer-step boundary: reduce the window's [entropy sum, token count] over the ranks (one small
        collective and one host read per optimizer step), move the coefficient by one delta towards the target and
        remember the measured entropy, which gates the bonus of the next window (grpo_trainer.py:3189-3210)."""
        a = self.args
        w = self._entropy_window_stats
        self._entropy_window_stats = None
        if w is None:
            return
        if D.world_size() > 1:
            w = D.all_reduce(w.clone(), "sum")
        tot = w.tolist()
        world_entropy = tot[0] / max(tot[1], 1.0)
        if world_entropy <= a.entropy_target:
            self.entropy_coef = min(self.entropy_coef + a.entropy_coef_delta, a.entropy_coef_max)
        else:
            self.entropy_coef = max(self.entropy_coef - a.entropy_coef_delta, a.entropy_coef_min)
        self._last_world_entropy = world_entropy

    def prediction_step(self, model, inputs, prediction_loss_only=True, ignore_keys=None):
        inputs = self._prepare_inputs(inputs)
        with torch.no_grad():
            loss = self._compute_loss(model, inputs)
        return loss.detach(), None, None

    def _save_checkpoint(self, model, trial=None, metrics=None):
        super()._save_checkpoint(model, trial, metrics)
        if self.args.use_adaptive_entropy and self.args.should_save:
            folder = os.path.join(self.args.output_dir, f"checkpoint-{self.state.global_step}")
            with open(os.path.join(folder, "entropy_ctrl_state.json"), "w") as f:
                json.dump({"entropy_coef": self.entropy_coef, "last_world_entropy": self._last_world_entropy}, f)

    def _on_checkpoint_loaded(self, folder: str):
        p = os.path.join(folder, "entropy_ctrl_state.json")
        if os.path.exists(p):
            with open(p) as f:
                st = json.load(f)
            self.entropy_coef = st["entropy_coef"]
            self._last_world_entropy = st.get("last_world_entropy", float("inf"))
        self._buffered_inputs = None  # a resumed run regenerates (grpo_trainer.py:1572-1574)
