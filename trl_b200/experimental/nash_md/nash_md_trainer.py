"""Nash-MD (trl/experimental/nash_md/nash_md_trainer.py: GeometricMixtureWrapper :49-100, rewards/probabilities
:324-400, losses :402-425).

The opponent is sampled from the geometric mixture  softmax(c * z_ref + (1 - c) * z_policy).  With P = the
probability that the policy's sample is preferred (sigmoid of the score difference, or a pairwise judge model's probability),
loss = beta * sum_t (log pi - log pi_ref)_sg * log pi  -  (P - 1/2) * sum_t log pi   on the policy's own sample."""
from __future__ import annotations

import torch

from ...models.decoder import SeqCtx
from ...parallel import dist as D
from ..online_dpo.online_dpo_trainer import OnlineDPOTrainer
from .nash_md_config import NashMDConfig


class GeometricMixtureGenerator:
    """Samples from the mixture of two models' next-token logits (full recompute per step: no KV cache is shared
    between two models; meant for the short completions of preference optimisation)."""

    def __init__(self, model, ref_model, mixture_coef: float = 0.5):
        self.model, self.ref_model, self.mixture_coef = model, ref_model, mixture_coef

    @torch.no_grad()
    def generate(self, prompts, max_new_tokens, temperature=1.0, eos_token_id=None, seed=0):
        dev = self.model.device
        g = torch.Generator(device="cpu").manual_seed(seed)
        seqs = [list(p) for p in prompts]
        outs = [[] for _ in prompts]
        alive = list(range(len(prompts)))
        was = self.model.training
        self.model.eval()
        for _ in range(max_new_tokens):
            if not alive:
                break
            flat = torch.tensor([t for i in alive for t in seqs[i]], dtype=torch.long, device=dev)
            ctx = SeqCtx.from_lengths([len(seqs[i]) for i in alive], dev)
            last = (ctx.cu_seqlens[1:] - 1).long()
            z = self.model.forward_hidden(flat, ctx)[last].float() @ self.model.lm_head_weight.float().t()
            zr = self.ref_model.forward_hidden(flat, ctx)[last].float() @ self.ref_model.lm_head_weight.float().t()
            mix = self.mixture_coef * zr + (1 - self.mixture_coef) * z
            probs = torch.softmax(mix / max(temperature, 1e-6), -1).cpu()
            tok = torch.multinomial(probs, 1, generator=g).flatten().tolist()
            nxt = []
            for i, t in zip(alive, tok):
                seqs[i].append(t)
                outs[i].append(t)
                if eos_token_id is None or t != eos_token_id:
                    nxt.append(i)
            alive = nxt
        self.model.train(was)
        return outs


class NashMDTrainer(OnlineDPOTrainer):
    _tag_names = ["trl", "nash-md"]
    _name = "NashMD"

    def __init__(self, model, ref_model=None, reward_funcs=None, judge=None, args: NashMDConfig | None = None, **kw):
        args = args or NashMDConfig("model-NashMD")
        super().__init__(model, ref_model, reward_funcs, judge, args, **kw)
        self._mixture_schedule = args.mixture_coef

    @property
    def mixture_coef(self):
        return self._per_epoch(self._mixture_schedule)

    def _second_candidates(self, prompt_ids, first):
        ref = self.ref_model if self.ref_model is not None else self.model
        gen = GeometricMixtureGenerator(self.model, ref, self.mixture_coef)
        return gen.generate(prompt_ids, self.max_completion_length, self.args.temperature, self.eos_token_id,
                            seed=self.args.seed + self.state.global_step)

    def _compute_loss(self, model, inputs):
        mode = "train" if model.training else "eval"
        m = self._metrics[mode]
        p, a, scores = inputs["prompt_ids"], inputs["cand_a"], inputs["scores"]
        if self.judge is not None:
            prob = scores[:, 0]  # judge: 1 when the policy's sample wins
        else:
            prob = torch.sigmoid(scores[:, 0] - scores[:, 1])
        lp, mask, ent = self._seq_logps(model, p, a)
        with torch.no_grad():
            ref = self._ref_seq_logps(p, a)
            log_ratio = lp.detach() - ref
        score = (prob - 0.5) * lp.sum(1)
        kl_loss = (log_ratio * lp).sum(1)
        beta = self.beta
        loss = (beta * kl_loss - score).mean() / self.current_gradient_accumulation_steps
        with torch.no_grad():
            vals = torch.stack([score.mean(), log_ratio.sum(1).mean(), (ent * mask).sum() / mask.sum().clamp(min=1),
                                prob.mean(), (prob > 0.5).float().mean()])
            if D.world_size() > 1:
                D.all_reduce(vals, "mean")
            for k, v in zip(["loss/score", "objective/kl", "objective/entropy", "rewards/probabilities",
                             "rewards/accuracies"], vals):
                m[k].append(v)
            m["loss/kl"].append((beta * kl_loss.detach()).mean())
            m["mixture_coef"].append(float(self.mixture_coef))
            m["beta"].append(float(beta))
        return loss
