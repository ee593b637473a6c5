"""Reference-free pairwise preference trainers share this base: DPO's data pipeline (tokenisation of
prompt/chosen/rejected, ``[chosen..., rejected...]`` batches, padding-free forward, log-probs fused into the lm_head
GEMM) without a reference model; subclasses supply ``pair_loss``."""
from __future__ import annotations

import torch

from ..parallel import dist as D
from ..trainer.dpo_trainer import DPOTrainer


class _Shim:
    """Gives a reference-free config the DPO fields the shared pipeline reads."""

    _DEFAULTS = dict(loss_type=["sigmoid"], loss_weights=None, use_weighting=False, f_divergence_type="reverse_kl",
                     f_alpha_divergence_coef=0.5, ld_alpha=None, precompute_ref_log_probs=False, sync_ref_model=False,
                     padding_free=False, eos_token=None, pad_token=None, truncation_mode="keep_start",
                     pad_to_multiple_of=None, label_smoothing=0.0, router_aux_loss_coef=0.001, discopop_tau=0.05)


class PairwiseTrainer(DPOTrainer):
    _needs_ref = False
    _average_logps = False  # True: losses work on length-normalised log-probs

    def __init__(self, model, args=None, **kw):
        kw.pop("ref_model", None)
        own_loss_type = getattr(args, "loss_type", None)
        for k, v in _Shim._DEFAULTS.items():
            if not hasattr(args, k):
                setattr(args, k, v)
        args.loss_type = ["sigmoid"]  # what the shared constructor validates; the subclass keeps its own below
        try:
            super().__init__(model, None, args, **kw)
        finally:
            args.loss_type = own_loss_type
        self.loss_type = own_loss_type

    def pair_loss(self, chosen_logps, rejected_logps, nll_chosen, ex, P):
        """Returns (per-pair losses [P], extra scalar loss, dict of extra metrics)."""
        raise NotImplementedError

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        mode = "train" if model.training else "eval"
        m = self._metrics[mode]
        seq_lp, aux, ex = self._sequence_logps(model, inputs, need_stats=True)
        P = inputs["completion_mask"].shape[0] // self._branches
        n_tok = ex["n_tok"].clamp(min=1.0)
        logps = seq_lp / n_tok if self._average_logps else seq_lp
        pc, pr = logps[:P], logps[P:2 * P]
        chosen_tok = ex["seq_id"] < P
        nll = -(ex["tok_logps"] * chosen_tok).sum() / chosen_tok.sum().clamp(min=1)
        per, extra, extra_metrics = self.pair_loss(pc, pr, nll, ex, P)
        loss = per.mean() + extra
        if aux is not None:
            loss = loss + self.args.router_aux_loss_coef * aux
            m["aux_loss"].append(aux.detach())
        with torch.no_grad():
            cr, rr = self._rewards(pc.detach()), self._rewards(pr.detach())
            vals = torch.stack([cr.mean(), rr.mean(), (cr > rr).float().mean(), (cr - rr).mean(), pc.detach().mean(),
                                pr.detach().mean(), nll.detach()] + [v.detach().float() for v in extra_metrics.values()])
            if D.world_size() > 1:
                D.all_reduce(vals, "mean")
            names = ["rewards/chosen", "rewards/rejected", "rewards/accuracies", "rewards/margins", "logps/chosen",
                     "logps/rejected", "nll_loss"] + list(extra_metrics)
            for n, v in zip(names, vals):
                m[n].append(v)
            ent = ex["entropy"]
            sums = torch.stack([ent.sum(), torch.tensor(float(ent.numel()), device=ent.device),
                                inputs["attention_mask"].sum().float()])
            if D.world_size() > 1:
                D.all_reduce(sums, "sum")
            m["entropy"].append(sums[0] / sums[1].clamp(min=1))
            if mode == "train":
                self._num_tokens = getattr(self, "_num_tokens", 0.0) + float(sums[2])
            m["num_tokens"].append(getattr(self, "_num_tokens", 0.0))
        return (loss, None) if return_outputs else loss

    _branches = 2

    def _rewards(self, logps):
        return self.args.beta * logps
