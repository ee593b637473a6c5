"""Online DPO (trl/experimental/online_dpo/online_dpo_trainer.py: training_step :1097-1297).

Per prompt two completions are sampled from the current policy, scored by the reward functions (or ranked by a
pairwise judge), the better one becomes "chosen", and the DPO loss (sigmoid or IPO) against the frozen reference
is applied.  XPO and Nash-MD reuse the skeleton with a different second candidate and loss."""
from __future__ import annotations

from typing import Any

import torch
import torch.nn.functional as F

from ...data_utils import is_conversational
from ...parallel import dist as D
from ...trainer.online_base import OnlineTrainer
from .online_dpo_config import OnlineDPOConfig


class OnlineDPOTrainer(OnlineTrainer):
    _tag_names = ["trl", "online-dpo"]
    _name = "OnlineDPO"

    def __init__(self, model, ref_model=None, reward_funcs=None, judge=None, args: OnlineDPOConfig | None = None,
                 train_dataset=None, eval_dataset=None, processing_class=None, reward_processing_classes=None,
                 callbacks=None, peft_config=None, **kw):
        args = args or OnlineDPOConfig("model-OnlineDPO")
        if reward_funcs is None and args.reward_model_path is not None:
            reward_funcs = args.reward_model_path
        if (reward_funcs is None) == (judge is None):
            raise ValueError("Exactly one of `reward_funcs` and `judge` must be provided")
        self.judge = judge
        beta_schedule = args.beta
        args.beta = beta_schedule[0] if isinstance(beta_schedule, (list, tuple)) else beta_schedule
        super().__init__(model, reward_funcs if reward_funcs is not None else [], args, train_dataset=train_dataset,
                         eval_dataset=eval_dataset, processing_class=processing_class,
                         reward_processing_classes=reward_processing_classes, callbacks=callbacks, peft_config=peft_config)
        args.beta = beta_schedule
        self._beta_schedule = beta_schedule
        if ref_model is not None:
            self.ref_model = ref_model.to(self.args.device, dtype=self.model.dtype).eval().requires_grad_(False)
        self._gen_cache: dict = {}

    # ---- schedule values that may be given per epoch -------------------------------------------------------------------
    def _per_epoch(self, v):
        if isinstance(v, (list, tuple)):
            e = int(self.state.epoch or 0)
            return v[e] if e < len(v) else v[-1]
        return v

    @property
    def beta(self):
        return self._per_epoch(self._beta_schedule) if hasattr(self, "_beta_schedule") else self.__dict__.get("_beta0", 0.1)

    @beta.setter
    def beta(self, v):
        self.__dict__["_beta0"] = v

    # ---- candidates ---------------------------------------------------------------------------------------------------
    def _second_candidates(self, prompt_ids, first):
        """Completions the policy's samples are compared with; here: a second sample from the policy."""
        return None

    def _generate_and_score_completions(self, inputs: list[dict]) -> dict[str, Any]:
        dev = self.args.device
        prompts = [x["prompt"] for x in inputs]
        second = self._second_candidates  # bound method; subclasses override
        # two policy samples per prompt unless the subclass provides the opponent itself
        own_pair = type(self)._second_candidates is OnlineDPOTrainer._second_candidates
        if own_pair:
            doubled = [p for p in prompts for _ in range(2)]
            self.num_generations, keep = 2, self.num_generations
            try:
                p_ids, c_ids, _, _ = self._generate(doubled)
            finally:
                self.num_generations = keep
            prompt_ids = p_ids[0::2]
            cand_a, cand_b = c_ids[0::2], c_ids[1::2]
        else:
            prompt_ids, cand_a, _, _ = self._generate(prompts)
            cand_b = second(prompt_ids, cand_a)
        tok = self.processing_class
        n = len(prompts)
        eos = tok.eos_token_id
        has_eos = torch.tensor([[eos in a, eos in b] for a, b in zip(cand_a, cand_b)], device=dev)
        texts_a = tok.batch_decode(cand_a, skip_special_tokens=True)
        texts_b = tok.batch_decode(cand_b, skip_special_tokens=True)
        if self.judge is not None:
            plain = [p if isinstance(p, str) else tok.apply_chat_template(p, tokenize=False, add_generation_prompt=True)
                     for p in prompts]
            ranks = self.judge.judge(plain, list(zip(texts_a, texts_b)))
            a_wins = torch.tensor([r == 0 for r in ranks], device=dev)
            scores = torch.stack([a_wins.float(), 1 - a_wins.float()], 1)
        else:
            conv = is_conversational(inputs[0])
            wrap = (lambda t: [{"role": "assistant", "content": t}]) if conv else (lambda t: t)
            both_inputs = [dict(x) for x in inputs] * 2
            rw = self._calculate_rewards(both_inputs, prompts * 2, [wrap(t) for t in texts_a + texts_b], cand_a + cand_b)
            sl = slice(D.rank() * 2 * n, (D.rank() + 1) * 2 * n)
            local = (rw[sl] * self.reward_weights.to(dev)[None]).nansum(1)
            scores = torch.stack([local[:n], local[n:]], 1)
            if self.args.missing_eos_penalty is not None:
                scores = scores - self.args.missing_eos_penalty * (~has_eos).float()
            a_wins = scores[:, 0] >= scores[:, 1]
        m = self._metrics["train" if self.model.training else "eval"]
        m["objective/scores"].append(D.gather(scores.mean().reshape(1)).mean())
        m["objective/scores_margin"].append(D.gather((scores[:, 0] - scores[:, 1]).abs().mean().reshape(1)).mean())
        m["val/contain_eos_token"].append(D.gather(has_eos.float().mean().reshape(1)).mean())
        return {"prompt_ids": prompt_ids, "cand_a": cand_a, "cand_b": cand_b, "a_wins": a_wins, "scores": scores}

    # ---- loss -----------------------------------------------------------------------------------------------------------
    def _seq_logps(self, model, prompt_ids, completion_ids, no_grad=False):
        ctx = torch.no_grad() if no_grad else torch.enable_grad()
        with ctx:
            lp, ent = self._get_per_token_logps_and_entropies(model, prompt_ids, completion_ids, compute_entropy=not no_grad)
        lens = torch.tensor([len(c) for c in completion_ids], device=lp.device)
        mask = (torch.arange(lp.shape[1], device=lp.device)[None] < lens[:, None]).float()
        return lp * mask, mask, ent

    def _ref_seq_logps(self, prompt_ids, completion_ids):
        lp = self._ref_logps(prompt_ids, completion_ids, len(prompt_ids))
        lens = torch.tensor([len(c) for c in completion_ids], device=lp.device)
        mask = (torch.arange(lp.shape[1], device=lp.device)[None] < lens[:, None]).float()
        return lp * mask

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        return self._compute_loss(model, inputs)

    def _compute_loss(self, model, inputs):
        mode = "train" if model.training else "eval"
        m = self._metrics[mode]
        p, a, b, a_wins = inputs["prompt_ids"], inputs["cand_a"], inputs["cand_b"], inputs["a_wins"]
        n = len(p)
        lp, mask, ent = self._seq_logps(model, p + p, a + b)
        with torch.no_grad():
            ref = self._ref_seq_logps(p + p, a + b)
        pol_sum, ref_sum = lp.sum(1), ref.sum(1)
        lr_a, lr_b = pol_sum[:n] - ref_sum[:n], pol_sum[n:] - ref_sum[n:]
        chosen_lr, rejected_lr = torch.where(a_wins, lr_a, lr_b), torch.where(a_wins, lr_b, lr_a)
        logits = chosen_lr - rejected_lr
        beta = self.beta
        if self.args.loss_type == "sigmoid":
            losses = -F.logsigmoid(beta * logits)
        else:
            losses = (logits - 1 / (2 * beta)) ** 2
        loss = losses.mean() / self.current_gradient_accumulation_steps
        with torch.no_grad():
            kl = (lp.detach() - ref).sum(1).mean()
            entropy = (ent * mask).sum() / mask.sum().clamp(min=1) if ent is not None else torch.zeros(())
            cr, rr = beta * chosen_lr.detach(), beta * rejected_lr.detach()
            vals = torch.stack([kl, entropy.to(kl), cr.mean(), rr.mean(), (cr > rr).float().mean(), (cr - rr).mean(),
                                torch.where(a_wins, pol_sum[:n], pol_sum[n:]).detach().mean(),
                                torch.where(a_wins, pol_sum[n:], pol_sum[:n]).detach().mean()])
            if D.world_size() > 1:
                D.all_reduce(vals, "mean")
            for k, v in zip(["objective/kl", "objective/entropy", "rewards/chosen", "rewards/rejected",
                             "rewards/accuracies", "rewards/margins", "logps/chosen", "logps/rejected"], vals):
                m[k].append(v)
            m["objective/non_score_reward"].append(-beta * vals[0])
            m["beta"].append(float(beta))
        return loss
