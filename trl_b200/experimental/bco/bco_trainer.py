"""Binary classifier optimisation (trl/experimental/bco/bco_trainer.py: RunningMoments :119-175, bco_loss :1178-1236).

Unpaired data as in KTO.  reward = beta * log(pi/pi_ref); delta = running mean of all rewards seen so far;
loss = -log sigmoid(r - delta) for desirable and -log sigmoid(-(r - delta)) for undesirable completions.  With
``embedding_func`` the undesirable losses are re-weighted by a density ratio p(desirable prompt)/p(undesirable prompt)
from a logistic classifier on prompt embeddings (underlying-distribution matching)."""
from __future__ import annotations

import json

import torch
import torch.nn.functional as F

from ...parallel import dist as D
from ...trainer.kto_trainer import KTOTrainer
from .bco_config import BCOConfig


class RunningMoments:
    """Running mean / variance of a stream, merged across ranks per update (parallel-variance formula)."""

    def __init__(self):
        self.mean, self.std, self.var, self.count = 0.0, 1.0, 1.0, 1e-24

    @torch.no_grad()
    def update(self, xs: torch.Tensor):
        xs = xs.float().flatten()
        stats = torch.stack([xs.sum(), (xs * xs).sum(), torch.tensor(float(xs.numel()), device=xs.device)])
        if D.world_size() > 1:
            D.all_reduce(stats, "sum")
        n = float(stats[2])
        if n == 0:
            return self.mean, self.std
        xs_mean = float(stats[0]) / n
        xs_var = max(float(stats[1]) / n - xs_mean * xs_mean, 0.0)
        delta = xs_mean - self.mean
        tot = self.count + n
        old_sum = self.var * self.count + delta * delta * self.count * n / tot
        tot_sum = old_sum + xs_var * n
        self.mean += delta * n / tot
        self.var = tot_sum / tot
        self.std = (self.var * tot / max(tot - 1, 1e-24)) ** 0.5
        self.count = tot
        return xs_mean, (xs_var * n / max(n - 1, 1e-24)) ** 0.5

    def save_to_json(self, path: str):
        with open(path, "w") as f:
            json.dump({"mean": self.mean, "std": self.std, "var": self.var, "count": self.count}, f, indent=2)

    @classmethod
    def load_from_json(cls, path: str):
        r = cls()
        with open(path) as f:
            for k, v in json.load(f).items():
                setattr(r, k, v)
        return r


class BCOTrainer(KTOTrainer):
    _tag_names = ["trl", "bco"]
    _name = "BCO"

    def __init__(self, model, ref_model=None, args: BCOConfig | None = None, embedding_func=None,
                 embedding_tokenizer=None, **kw):
        args = args or BCOConfig("model-BCO")
        super().__init__(model, ref_model, args, **kw)
        self.running = RunningMoments()
        self.embedding_func, self.embedding_tokenizer = embedding_func, embedding_tokenizer
        self.match_underlying_distribution = embedding_func is not None
        self.clf = None
        if self.match_underlying_distribution:
            self._fit_density_ratio_classifier()

    # ---- underlying-distribution matching ------------------------------------------------------------------------
    def _prompt_embeddings(self, rows):
        ids = [torch.tensor(r["prompt_ids"] if "prompt_ids" in r else r["input_ids"]) for r in rows]
        from ...trainer.utils import pad

        batch = pad(ids, self.processing_class.pad_token_id, "right").to(self.args.device)
        with torch.no_grad():
            return self.embedding_func(input_ids=batch, attention_mask=(batch != self.processing_class.pad_token_id).long()).float()

    def _fit_density_ratio_classifier(self):
        from sklearn.linear_model import LogisticRegression

        rows = [self.train_dataset[i] for i in range(min(len(self.train_dataset), self.args.prompt_sample_size))]
        emb = self._prompt_embeddings(rows).cpu().numpy()
        y = [int(bool(r["label"])) for r in rows]
        if len(set(y)) < 2:
            return
        self.clf = LogisticRegression(class_weight="balanced", max_iter=200).fit(emb, y)

    def _udm_weight(self, inputs, label):
        if self.clf is None:
            return None
        emb = self.embedding_func(input_ids=inputs["input_ids"], attention_mask=inputs["attention_mask"]).float()
        prob = torch.as_tensor(self.clf.predict_proba(emb[~label].detach().cpu().numpy())[:, 1], device=emb.device)
        w = prob / (1 - prob + 1e-8)
        return w.clamp(self.args.min_density_ratio, self.args.max_density_ratio).float()

    # ---- loss ------------------------------------------------------------------------------------------------------
    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        self._udm_w = self._udm_weight(inputs, inputs["label"].bool()) if self.match_underlying_distribution else None
        return super().compute_loss(model, inputs, return_outputs, num_items_in_batch)

    def _unpaired_losses(self, c_lr, r_lr, kl, mode):
        c_rew, r_rew = self.beta * c_lr, self.beta * r_lr
        if mode == "train":
            self.running.update(torch.cat([c_rew, r_rew]).detach())
        delta = self.running.mean
        self._metrics[mode]["delta"].append(delta)
        c_loss = -F.logsigmoid(c_rew - delta)
        r_loss = -F.logsigmoid(-(r_rew - delta))
        if getattr(self, "_udm_w", None) is not None and self._udm_w.numel() == r_loss.numel():
            r_loss = r_loss * self._udm_w
        return c_loss, r_loss

    def _save_checkpoint(self, model, trial=None, metrics=None):
        super()._save_checkpoint(model, trial, metrics)
        import os

        folder = os.path.join(self.args.output_dir, f"checkpoint-{self.state.global_step}")
        if self.args.should_save and os.path.isdir(folder):
            self.running.save_to_json(os.path.join(folder, "running.json"))
