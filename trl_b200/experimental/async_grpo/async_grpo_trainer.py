"""Asynchronous GRPO (trl/experimental/async_grpo/async_grpo_trainer.py: batching :300-520, loss :911-960).

Training never waits for a full synchronous generation phase: a worker keeps a queue of scored rollouts filled; every
micro-batch takes what it needs from the queue (rank 0 pops, objects are broadcast), drops samples older than
``max_staleness`` weight versions, spreads the rest over the data-parallel ranks so that the sum of squared lengths is
balanced (attention cost) within ``token_budget`` real tokens per rank, and trains padding-free with the clipped
token-level objective against the *sampling* log-probs.  Every ``weight_sync_steps`` optimizer steps the worker is told
the new weight version (and a generation server receives the weights)."""
from __future__ import annotations

import queue
import warnings
from typing import Any, Callable, Optional

import torch

from ...loop.trainer import Trainer
from ...models.decoder import SeqCtx
from ...ops import functional as ops
from ...parallel import dist as D
from ...trainer.utils import create_model_from_path
from .async_grpo_config import AsyncGRPOConfig
from .async_rollout_worker import AsyncRolloutWorker, ProcessRolloutWorker, RolloutSample


class _ServerSideReward:
    """Picklable reward call for the spawned rollout process: decodes completions with the tokenizer it carries and
    sums the (picklable) reward functions, exactly like ``AsyncGRPOTrainer._reward``."""

    def __init__(self, reward_funcs, tokenizer):
        self.reward_funcs, self.tok = list(reward_funcs), tokenizer

    def __call__(self, examples, prompt_ids, completion_ids):
        texts = self.tok.batch_decode(completion_ids, skip_special_tokens=True)
        total = [0.0] * len(texts)
        keys = [k for k in examples[0] if k not in ("prompt", "prompt_text", "completion")]
        kw = {k: [ex[k] for ex in examples] for k in keys}
        for rf in self.reward_funcs:
            vals = rf(prompts=[ex.get("prompt_text", ex["prompt"]) for ex in examples], completions=texts,
                      completion_ids=completion_ids, **kw)
            total = [t + (float(v) if v is not None else 0.0) for t, v in zip(total, vals)]
        return total


class TokenBudgetBatcher:
    """Longest-first assignment of samples to ``world`` rows minimising the largest sum of squared lengths, each row
    holding at most ``token_budget`` tokens (``<= 0``: exactly ``per_rank`` samples per row)."""

    def __init__(self, world: int, token_budget: int, per_rank: int):
        self.world, self.budget, self.per_rank = world, token_budget, per_rank

    def assign(self, samples: list) -> tuple[list[list], list]:
        rows, load, toks = [[] for _ in range(self.world)], [0] * self.world, [0] * self.world
        left = []
        for s in sorted(samples, key=len, reverse=True):
            L = len(s)
            if self.budget > 0 and L > self.budget:
                warnings.warn(f"dropping a rollout of {L} tokens: longer than token_budget={self.budget}")
                continue
            cands = [r for r in range(self.world)
                     if (self.budget > 0 and toks[r] + L <= self.budget) or (self.budget <= 0 and len(rows[r]) < self.per_rank)]
            if not cands:
                left.append(s)
                continue
            r = min(cands, key=lambda i: load[i])
            rows[r].append(s)
            load[r] += L * L
            toks[r] += L
        return rows, left


class AsyncGRPOTrainer(Trainer):
    _tag_names = ["trl", "async-grpo"]
    _name = "AsyncGRPO"

    def __init__(self, model, reward_funcs, args: AsyncGRPOConfig | None = None, train_dataset=None, processing_class=None,
                 callbacks=None, generate_fn: Optional[Callable] = None, **kw):
        args = args or AsyncGRPOConfig("model-AsyncGRPO")
        if isinstance(model, str):
            model = create_model_from_path(model, **dict(args.model_init_kwargs or {}))
        self.reward_funcs = reward_funcs if isinstance(reward_funcs, list) else [reward_funcs]
        self._prompt_rows = train_dataset
        super().__init__(model=model, args=args, data_collator=lambda x: x, train_dataset=train_dataset,
                         processing_class=processing_class, callbacks=callbacks)
        self.model_accepts_loss_kwargs = False
        self.compute_loss_func = "non-None: the loss is already divided by the accumulation steps"
        self._leftover: list[RolloutSample] = []
        self._dropped_stale = 0
        self._version = 0
        self.worker: Optional[AsyncRolloutWorker] = None
        self._generate_fn = generate_fn
        self._client = None
        budget = args.token_budget if args.token_budget is not None else 0
        self.batcher = TokenBudgetBatcher(D.world_size(), budget, args.per_device_train_batch_size)

    # ---- rollout side -------------------------------------------------------------------------------------------------
    def _default_generate_fn(self):
        a, tok = self.args, self.processing_class
        from ...rollout.sampling import SamplingParams

        if a.vllm_server_base_url and self._generate_fn is None and self.args.device.type == "cuda":
            from .vllm_client import VLLMClient

            self._client = VLLMClient(base_url=a.vllm_server_base_url, connection_timeout=a.vllm_server_timeout)
            self._client.check_server(a.vllm_server_timeout)

            def via_server(prompts, n):
                ids = self._tokenize(prompts)
                res = self._client.generate(ids, n=n, temperature=a.temperature, max_tokens=a.max_completion_length)
                rep = [p for p in ids for _ in range(n)]
                return list(zip(rep, res["completion_ids"], res["logprobs"]))
            return via_server
        from ...rollout.engine import EagerGenerator

        gen = EagerGenerator(self.model)
        lock = self._model_lock

        def in_process(prompts, n):
            ids = self._tokenize(prompts)
            sp = SamplingParams(n=n, max_tokens=a.max_completion_length, temperature=a.temperature,
                                eos_token_id=tok.eos_token_id, seed=int(torch.randint(0, 1 << 30, (1,))))
            with lock:  # the eager generator flips train/eval mode on the shared module
                outs = gen.generate(ids, sp)
            rep = [p for p in ids for _ in range(n)]
            return [(p, o.token_ids, o.logprobs) for p, o in zip(rep, outs)]
        return in_process

    def _tokenize(self, prompts):
        tok = self.processing_class
        if prompts and not isinstance(prompts[0], str):
            return [tok.apply_chat_template(p, add_generation_prompt=True, tokenize=True,
                                            **(self.args.chat_template_kwargs or {})) for p in prompts]
        return tok(text=list(prompts), add_special_tokens=False)["input_ids"]

    def _reward(self, examples, prompt_ids, completion_ids):
        tok = self.processing_class
        texts = tok.batch_decode(completion_ids, skip_special_tokens=True)
        total = [0.0] * len(texts)
        keys = [k for k in examples[0] if k not in ("prompt", "completion")]
        kw = {k: [ex[k] for ex in examples] for k in keys}
        for rf in self.reward_funcs:
            vals = rf(prompts=[ex["prompt"] for ex in examples], completions=texts, completion_ids=completion_ids, **kw)
            total = [t + (float(v) if v is not None else 0.0) for t, v in zip(total, vals)]
        return total

    def _start_worker(self):
        import threading

        self._model_lock = threading.RLock()
        a = self.args
        mode = getattr(a, "rollout_worker", "auto")
        use_process = mode == "process" or (mode == "auto" and a.vllm_server_base_url and self._generate_fn is None
                                            and a.device.type == "cuda")
        if D.rank() == 0 and use_process:
            # a spawned child keeps the generation server busy and scores its answers; the trainer only pushes weights
            from .vllm_client import VLLMClient

            if not a.vllm_server_base_url:
                raise ValueError("rollout_worker='process' needs vllm_server_base_url (the child talks to a generation server)")
            self._client = VLLMClient(base_url=a.vllm_server_base_url, connection_timeout=a.vllm_server_timeout)
            rows = []
            for i in range(len(self._prompt_rows)):
                row = dict(self._prompt_rows[i])
                row["prompt_text"] = row["prompt"]
                row["prompt"] = self._tokenize([row["prompt"]])[0]
                rows.append(row)
            inflight = a.max_inflight_tasks if a.max_inflight_tasks and a.max_inflight_tasks > 0 else 4
            self.worker = ProcessRolloutWorker(rows, a.vllm_server_base_url, _ServerSideReward(self.reward_funcs, self.processing_class),
                                               a.num_generations, max_tokens=a.max_completion_length,
                                               queue_maxsize=a.queue_maxsize, scale_rewards=a.scale_rewards, seed=a.seed,
                                               temperature=a.temperature, max_inflight=inflight,
                                               server_timeout=a.vllm_server_timeout)
            self.worker.start()
        elif D.rank() == 0:
            fn = self._generate_fn or self._default_generate_fn()
            self.worker = AsyncRolloutWorker(self._prompt_rows, fn, self._reward, self.args.num_generations,
                                             self.args.queue_maxsize, self.args.scale_rewards, self.args.seed)
            self.worker.start()

    def train(self, *a, **kw):
        self._start_worker()
        try:
            return super().train(*a, **kw)
        finally:
            if self.worker is not None:
                self.worker.stop()

    # ---- batches come from the queue, not from the dataset ----------------------------------------------------------
    def get_train_dataloader(self):
        trainer = self

        class _QueueLoader:
            def __len__(self):
                return 1 << 30

            def set_epoch(self, e):
                pass

            def __iter__(self):
                while True:
                    yield trainer._next_rows()
        return _QueueLoader()

    def _next_rows(self):
        a = self.args
        world = D.world_size()
        need = a.per_device_train_batch_size * world
        rows = None
        if D.rank() == 0:
            have = self._leftover
            self._leftover = []
            while len(have) < need:
                self.worker.check_health(a.heartbeat_stale_after_s)
                try:
                    s = self.worker.get(timeout=1.0)
                except queue.Empty:
                    continue
                if self._version - s.model_version > a.max_staleness:
                    self._dropped_stale += 1
                    continue
                have.append(s)
            rows, self._leftover = self.batcher.assign(have)
        if world > 1:
            rows = D.broadcast_object_list([rows], src=0)[0]
        return rows[D.rank()]

    def _count_items(self, batches):
        return None

    def _prepare_inputs(self, inputs):
        return inputs

    # ---- loss -----------------------------------------------------------------------------------------------------------
    def compute_loss(self, model, inputs: list[RolloutSample], return_outputs=False, num_items_in_batch=None):
        a, dev = self.args, self.args.device
        m = self._metrics["train" if model.training else "eval"]
        if not inputs:
            return next(model.parameters()).sum() * 0.0
        seqs = [s.prompt_ids + s.completion_ids for s in inputs]
        flat = torch.tensor([t for x in seqs for t in x], dtype=torch.long, device=dev)
        with self._model_lock:
            hidden = model.forward_hidden(flat, SeqCtx.from_lengths([len(x) for x in seqs], dev))
        sel, old, adv, msk, off = [], [], [], [], 0
        for s in inputs:
            n, p = len(s.completion_ids), len(s.prompt_ids)
            sel.extend(range(off + p - 1, off + p - 1 + n))
            old.extend(s.logprobs)
            adv.extend([s.advantage] * n)
            msk.extend(s.completion_mask if s.completion_mask is not None else [1] * n)
            off += p + n
        sel_t = torch.tensor(sel, device=dev)
        lp, ent = ops.lm_head_logprobs(hidden[sel_t], model.lm_head_weight, flat[sel_t + 1], a.temperature,
                                       compute_entropy=True)
        old_t = torch.tensor(old, dtype=torch.float32, device=dev)
        adv_t = torch.tensor(adv, dtype=torch.float32, device=dev)
        mask = torch.tensor(msk, dtype=torch.float32, device=dev)
        ratio = torch.exp(lp - old_t)
        clipped = torch.clamp(ratio, 1 - a.epsilon, 1 + a.epsilon_high)
        per_tok = -torch.min(ratio * adv_t, clipped * adv_t)
        n_tok = mask.sum()
        tot = n_tok.clone()
        if D.world_size() > 1:
            D.all_reduce(tot, "sum")
        loss = (per_tok * mask).sum() / (tot / D.world_size()).clamp(min=1.0) / self.current_gradient_accumulation_steps
        with torch.no_grad():
            low = ((ratio < 1 - a.epsilon) & (adv_t < 0)).float()
            high = ((ratio > 1 + a.epsilon_high) & (adv_t > 0)).float()
            st = torch.stack([(low * mask).sum(), (high * mask).sum(), (ent * mask).sum(), n_tok,
                              torch.tensor(float(sum(self._version - s.model_version for s in inputs)), device=dev),
                              torch.tensor(float(len(inputs)), device=dev),
                              torch.tensor(sum(s.reward for s in inputs), device=dev)])
            if D.world_size() > 1:
                D.all_reduce(st, "sum")
            m["clip_ratio/low_mean"].append(st[0] / st[3].clamp(min=1))
            m["clip_ratio/high_mean"].append(st[1] / st[3].clamp(min=1))
            m["entropy"].append(st[2] / st[3].clamp(min=1))
            m["async/staleness_mean"].append(st[4] / st[5].clamp(min=1))
            m["reward"].append(st[6] / st[5].clamp(min=1))
            m["async/dropped_stale"].append(float(self._dropped_stale))
        return (loss, None) if return_outputs else loss

    def log(self, logs, start_time=None):
        with self._model_lock:  # the in-process generator flips train/eval on the shared module
            for k, v in self._metrics["train"].items():
                self._metrics["train"][k] = [float(x) for x in v]
            super().log(logs, start_time)

    def optimizer_step(self, batches: list):
        with self._model_lock:  # the worker must not read half-updated weights through the eager generator
            out = super().optimizer_step(batches)
        self._version += 1
        if self._version % max(1, self.args.weight_sync_steps) == 0:
            if self._client is not None and D.rank() == 0:
                from .weight_transfer import push_weights

                push_weights(self._client, self.model, getattr(self.engine, "gather_full_params", None))
            if self.worker is not None:
                self.worker.update_model_version(self._version)
        return out
