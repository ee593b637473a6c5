"""Asynchronous rollout worker (trl/experimental/async_grpo/async_rollout_worker.py: RolloutSample :188-230,
_AsyncRolloutLoop :276-760, AsyncRolloutWorker :914-1053).

A background thread keeps sampling groups of completions (through a generation server, or in-process on its own CUDA
stream next to training), scores them, turns group rewards into advantages and pushes ``RolloutSample`` objects,
tagged with the weight version they were sampled under, into a bounded queue.  The trainer drops samples that are
more than ``max_staleness`` versions old.  A heartbeat lets the trainer notice a dead worker."""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch


@dataclass
class RolloutSample:
    prompt_ids: list
    completion_ids: list
    logprobs: list            # sampling log-probs of the completion tokens (the behaviour policy)
    reward: float
    advantage: float
    model_version: int
    group_id: int
    completion_mask: Optional[list] = None  # 0 for tokens not produced by the policy (tool output)
    extras: dict = field(default_factory=dict)

    def __len__(self):
        return len(self.prompt_ids) + len(self.completion_ids)


class AsyncRolloutWorker:
    def __init__(self, dataset, generate_fn: Callable, reward_fn: Callable, num_generations: int, queue_maxsize: int = 1024,
                 scale_rewards: bool = True, seed: int = 0):
        """generate_fn(prompts, n) -> list (len(prompts) * n) of (prompt_ids, completion_ids, logprobs);
        reward_fn(examples, prompt_ids, completion_ids) -> list of floats (one per completion)."""
        self.dataset, self.generate_fn, self.reward_fn = dataset, generate_fn, reward_fn
        self.ng, self.scale_rewards, self.seed = num_generations, scale_rewards, seed
        self.queue: "queue.Queue[RolloutSample]" = queue.Queue(maxsize=queue_maxsize)
        self._version = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._heartbeat = time.monotonic()
        self._error: Optional[BaseException] = None
        self.groups_done = 0
        self.prompts_per_call = 4

    @property
    def model_version(self) -> int:
        return self._version

    def update_model_version(self, v: int) -> None:
        self._version = int(v)

    def start(self) -> None:
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="trl-b200-rollout", daemon=True)
            self._thread.start()

    def _run(self):
        g = torch.Generator().manual_seed(self.seed)
        n = len(self.dataset)
        try:
            while not self._stop.is_set():
                idx = torch.randint(0, n, (self.prompts_per_call,), generator=g).tolist()
                examples = [self.dataset[i] for i in idx]
                version = self._version
                outs = self.generate_fn([ex["prompt"] for ex in examples], self.ng)
                rep = [ex for ex in examples for _ in range(self.ng)]
                rewards = torch.tensor(self.reward_fn(rep, [o[0] for o in outs], [o[1] for o in outs]), dtype=torch.float32)
                groups = rewards.view(-1, self.ng)
                adv = groups - groups.mean(1, keepdim=True)
                if self.scale_rewards:
                    adv = adv / (groups.std(1, keepdim=True) + 1e-4)
                adv = adv.flatten()
                for j, (p, c, lp) in enumerate(outs):
                    s = RolloutSample(list(p), list(c), list(lp), float(rewards[j]), float(adv[j]), version,
                                      self.groups_done + j // self.ng)
                    while not self._stop.is_set():
                        try:
                            self.queue.put(s, timeout=0.2)
                            break
                        except queue.Full:
                            self._heartbeat = time.monotonic()
                self.groups_done += len(examples)
                self._heartbeat = time.monotonic()
        except BaseException as e:  # surfaced by check_health on the trainer's thread
            self._error = e

    def check_health(self, stale_after_s: float) -> None:
        if self._error is not None:
            raise RuntimeError("rollout worker failed") from self._error
        if self._thread is not None and not self._thread.is_alive() and not self._stop.is_set():
            raise RuntimeError("rollout worker exited")
        if time.monotonic() - self._heartbeat > stale_after_s:
            raise RuntimeError(f"rollout worker produced nothing for {stale_after_s:.0f} s")

    def get(self, timeout: float) -> RolloutSample:
        return self.queue.get(timeout=timeout)

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
