"""PPO with a learned value function (trl/experimental/ppo/ppo_trainer.py: rollout + rewards + GAE :700-800,
clipped policy / value losses :820-900).

One rollout batch -> ``num_ppo_epochs`` passes of ``num_mini_batches`` optimizer steps, scheduled by the online
trainer's generation buffer.  Rewards: -kl_coef * KL(pi || pi_ref) per token (k1 or k3 estimator) plus the sequence
score on the last token; advantages by GAE(gamma, lam), whitened; the value function is either a separate model with
a scalar head or a ``ValueHead`` on the policy's trunk.  Policy and value parameters share one optimizer."""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ...parallel import dist as D
from ...trainer.online_base import OnlineTrainer
from .modeling_value_head import ValueHead
from .ppo_config import PPOConfig


def masked_mean(x, mask):
    return (x * mask).sum() / mask.sum().clamp(min=1)


def masked_whiten(x, mask, shift_mean: bool = True):
    mean = masked_mean(x, mask)
    var = masked_mean((x - mean) ** 2, mask)
    n = mask.sum()
    var = var * n / (n - 1).clamp(min=1)  # unbiased
    out = (x - mean) * torch.rsqrt(var + 1e-8)
    return out if shift_mean else out + mean


class PPOTrainer(OnlineTrainer):
    _tag_names = ["trl", "ppo"]
    _name = "PPO"

    def __init__(self, args: PPOConfig, processing_class, model, ref_model=None, reward_model=None, train_dataset=None,
                 value_model=None, reward_funcs=None, eval_dataset=None, callbacks=None, peft_config=None, **kw):
        if reward_model is None and reward_funcs is None:
            raise ValueError("PPOTrainer needs a reward_model or reward_funcs")
        if value_model is not None:
            if not getattr(value_model.config, "num_labels", 0):
                raise ValueError("value_model must carry a scalar head (num_labels=1)")
            model.value_model = value_model  # registered submodule: trained by the same optimizer
        else:
            p = next(model.parameters())
            model.v_head = ValueHead(model.config.hidden_size, dtype=p.dtype, device=p.device)
        beta0, args.beta = args.beta, 0.0
        super().__init__(model, reward_model if reward_model is not None else reward_funcs, args,
                         train_dataset=train_dataset, eval_dataset=eval_dataset, processing_class=processing_class,
                         callbacks=callbacks, peft_config=peft_config)
        args.beta = beta0
        if ref_model is not None:
            self.ref_model = ref_model.to(self.args.device, dtype=self.model.dtype).eval().requires_grad_(False)
        if self.ref_model is not None:  # the frozen copy does not need the value parts
            for name in ("value_model", "v_head"):
                if name in self.ref_model._modules:
                    del self.ref_model._modules[name]
        self.temperature = args.temperature

    # ---- values -----------------------------------------------------------------------------------------------------
    def _values_from_selected(self, model, shape):
        hidden_sel, r, c_, flat, ctx, sel_t = self._selected_hidden
        if "value_model" in model._modules:
            vm = model.value_model
            v = (vm.forward_hidden(flat, ctx)[sel_t].float() @ vm.score.float().t()).squeeze(-1)
        else:
            v = model.v_head(hidden_sel).squeeze(-1).float()
        return torch.zeros(shape, dtype=torch.float32, device=v.device).index_put((r, c_), v)

    def _logps_values(self, model, prompt_ids, completion_ids, entropy=False):
        self._keep_selected_hidden = True
        try:
            lp, ent = self._get_per_token_logps_and_entropies(model, prompt_ids, completion_ids, compute_entropy=entropy)
            values = self._values_from_selected(model, lp.shape)
        finally:
            self._keep_selected_hidden = False
            self._selected_hidden = None
        return lp, values, ent

    # ---- rollout ------------------------------------------------------------------------------------------------------
    def _generate_and_score_completions(self, inputs: list[dict]) -> dict[str, Any]:
        a, dev = self.args, self.args.device
        prompts = [x["prompt"] for x in inputs]
        prompt_ids, completion_ids, _, _ = self._generate(prompts)
        B = len(prompt_ids)
        tok = self.processing_class
        stop = a.stop_token_id if a.stop_token_id is not None else (tok.eos_token_id if a.stop_token == "eos" else None)
        if stop is not None:  # truncate after the first stop token
            completion_ids = [c[: c.index(stop) + 1] if stop in c else c for c in completion_ids]
        lens = torch.tensor([len(c) for c in completion_ids], device=dev)
        with torch.no_grad():
            logps, values, _ = self._logps_values(self.model, prompt_ids, completion_ids)
            ref_logps = self._ref_logps(prompt_ids, completion_ids, B)
        Tc = logps.shape[1]
        mask = (torch.arange(Tc, device=dev)[None] < lens[:, None]).float()
        texts = tok.batch_decode(completion_ids, skip_special_tokens=True)
        rw = self._calculate_rewards([dict(x) for x in inputs], prompts, texts, completion_ids)
        scores = (rw[D.rank() * B:(D.rank() + 1) * B] * self.reward_weights.to(dev)[None]).nansum(1)
        has_eos = torch.tensor([tok.eos_token_id in c for c in completion_ids], device=dev)
        if a.missing_eos_penalty is not None:
            scores = scores - a.missing_eos_penalty * (~has_eos).float()
        logr = (ref_logps - logps) * mask
        kl = -logr if a.kl_estimator == "k1" else (torch.exp(logr) - 1) - logr
        non_score = -a.kl_coef * kl * mask
        rewards = non_score.clone()
        rewards[torch.arange(B, device=dev), (lens - 1).clamp(min=0)] += scores
        if a.whiten_rewards:
            rewards = masked_whiten(rewards, mask, shift_mean=False) * mask
        values = values * mask
        adv_rev, last = [], torch.zeros(B, device=dev)
        for t in reversed(range(Tc)):
            nxt = values[:, t + 1] if t < Tc - 1 else torch.zeros(B, device=dev)
            delta = rewards[:, t] + a.gamma * nxt - values[:, t]
            last = delta + a.gamma * a.lam * last
            adv_rev.append(last)
        advantages = torch.stack(adv_rev[::-1], 1) * mask
        returns = advantages + values
        advantages = masked_whiten(advantages, mask) * mask
        m = self._metrics["train" if self.model.training else "eval"]
        stats = torch.stack([kl.sum(1).mean(), non_score.sum(1).mean(), (non_score.sum(1) + scores).mean(), scores.mean(),
                             has_eos.float().mean(), lens.float().mean()])
        if D.world_size() > 1:
            D.all_reduce(stats, "mean")
        for k, v in zip(["objective/kl", "objective/non_score_reward", "objective/rlhf_reward", "objective/scores",
                         "val/num_eos_tokens", "completions/mean_length"], stats):
            m[k].append(v)
        self._total_train_tokens += int(D.gather((torch.tensor([len(p) for p in prompt_ids], device=dev).sum()
                                                  + lens.sum()).reshape(1)).sum())
        return {"prompt_ids": prompt_ids, "completion_ids_list": completion_ids, "old_logps": logps, "values": values,
                "advantages": advantages, "returns": returns, "mask": mask}

    # ---- loss -------------------------------------------------------------------------------------------------------------
    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        a = self.args
        mode = "train" if model.training else "eval"
        m = self._metrics[mode]
        new_lp, vpred, ent = self._logps_values(model, inputs["prompt_ids"], inputs["completion_ids_list"], entropy=True)
        Tc = new_lp.shape[1]

        def fit(t):
            return t[:, :Tc] if t.shape[1] >= Tc else torch.nn.functional.pad(t, (0, Tc - t.shape[1]))
        mask, old, adv = fit(inputs["mask"]), fit(inputs["old_logps"]), fit(inputs["advantages"])
        ret, val = fit(inputs["returns"]), fit(inputs["values"])
        vclip = torch.clamp(vpred, val - a.cliprange_value, val + a.cliprange_value)
        vf1, vf2 = (vpred - ret) ** 2, (vclip - ret) ** 2
        vf_loss = 0.5 * masked_mean(torch.max(vf1, vf2), mask)
        diff = (new_lp - old) * mask
        ratio = torch.exp(diff)
        pg1, pg2 = -adv * ratio, -adv * torch.clamp(ratio, 1 - a.cliprange, 1 + a.cliprange)
        pg_loss = masked_mean(torch.max(pg1, pg2), mask)
        loss = (pg_loss + a.vf_coef * vf_loss) / self.current_gradient_accumulation_steps
        with torch.no_grad():
            vals = torch.stack([pg_loss, vf_loss, masked_mean((pg2 > pg1).float(), mask), masked_mean((vf2 > vf1).float(), mask),
                                0.5 * masked_mean(diff ** 2, mask), masked_mean(ent, mask), masked_mean(ratio, mask)])
            if D.world_size() > 1:
                D.all_reduce(vals, "mean")
            for k, v in zip(["loss/policy_avg", "loss/value_avg", "policy/clipfrac_avg", "val/clipfrac_avg",
                             "policy/approxkl_avg", "policy/entropy_avg", "val/ratio"], vals):
                m[k].append(v)
        return (loss, None) if return_outputs else loss

    # ---- sample generations ------------------------------------------------------------------------------------------
    def generate_completions(self, sampling: bool = False, max_prompts: int = 8) -> dict:
        """Near-greedy completions for a few evaluation prompts with their scores, printed as a table and kept in
        ``self.sample_generations`` (trl/experimental/ppo/ppo_trainer.py:951-1029).  ``sampling=True``: one batch only."""
        ds = self.eval_dataset if self.eval_dataset is not None else self.train_dataset
        rows = [dict(ds[i]) for i in range(min(len(ds), max_prompts))]
        prompts = [r["prompt"] for r in rows]
        was_t, was_training = self.temperature, self.model.training
        self.temperature = 0.01 + 1e-7
        self.model.eval()
        try:
            with torch.no_grad():
                _, completion_ids, _, _ = self._generate(prompts)
                texts = self.processing_class.batch_decode(completion_ids, skip_special_tokens=True)
                rw = self._calculate_rewards(rows, prompts, texts, completion_ids)
        finally:
            self.temperature = was_t
            self.model.train(was_training)
        B, r = len(prompts), D.rank()
        scores = (rw[r * B:(r + 1) * B] * self.reward_weights.to(rw.device)[None]).nansum(1).tolist()
        table = {"query": [p if isinstance(p, str) else str(p) for p in prompts], "model response": texts, "score": scores}
        self.sample_generations = table
        if D.is_main():
            from ...trainer.utils import print_prompt_completions_sample

            print_prompt_completions_sample(table["query"], texts, {"score": scores}, [0.0] * B, self.state.global_step, B)
        return table

    def _maybe_log_save_evaluate(self, tr_loss, grad_norm, lr, t_start):
        out = super()._maybe_log_save_evaluate(tr_loss, grad_norm, lr, t_start)
        n, st = self.args.num_sample_generations, self.state
        if n and n > 0 and st.max_steps and st.global_step > getattr(self, "_sampled_at", -1):
            every = max(1, st.max_steps // n)
            if st.global_step % every == 0:
                self._sampled_at = st.global_step
                self.generate_completions(sampling=True)
        return out

    def _save(self, output_dir: str, state_dict=None):
        """The checkpoint is the policy; the value parts are stored next to it."""
        import os

        held = {n: self.model._modules.pop(n) for n in ("value_model", "v_head") if n in self.model._modules}
        try:
            super()._save(output_dir, state_dict)
        finally:
            self.model._modules.update(held)
        for n, mod in held.items():
            torch.save(mod.state_dict(), os.path.join(output_dir, f"{n}.pt"))
