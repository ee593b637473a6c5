"""Asynchronous rollout worker (trl/experimental/async_grpo/async_rollout_worker.py: RolloutSample :188-230,
_AsyncRolloutLoop :276-760, AsyncRolloutWorker :914-1053).

Two workers with one interface (``start / get / update_model_version / check_health / stop``):

* :class:`AsyncRolloutWorker`: a background thread next to training (in-process engine on its own CUDA stream, or any
  ``generate_fn``);
* :class:`ProcessRolloutWorker`: a spawned child process, like the reference's: an asyncio loop keeps several
  ``/generate`` requests to the generation server in flight, a second task scores finished groups (reward functions
  must be picklable), turns group rewards into advantages and puts ``RolloutSample`` objects on a
  ``multiprocessing.Queue``.  The weight version travels through a shared integer, the heartbeat through a shared
  double, a failure through an error queue; the parent notices a dead, silent or failed child in ``check_health``.

Samples are tagged with the weight version they were sampled under; the trainer drops samples that are more than
``max_staleness`` versions old."""
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


# ---- child-process worker ---------------------------------------------------------------------------------------------
def _advantages(rewards: list, ng: int, scale: bool) -> list:
    r = torch.tensor(rewards, dtype=torch.float32).view(-1, ng)
    a = r - r.mean(1, keepdim=True)
    if scale:
        a = a / (r.std(1, keepdim=True) + 1e-4)
    return a.flatten().tolist()


def _process_main(cfg: dict, rows: list, reward_fn, out_q, version, heartbeat, stop, err_q):
    """Entry point of the spawned rollout process."""
    import asyncio
    import traceback

    async def run():
        from .vllm_client import AsyncGenerationClient

        client = AsyncGenerationClient(cfg["server_url"], request_timeout=cfg.get("request_timeout", 600.0))
        await client.wait_healthy(cfg.get("server_timeout", 60.0))
        g = torch.Generator().manual_seed(cfg.get("seed", 0))
        ng, ppc = cfg["num_generations"], cfg.get("prompts_per_call", 4)
        done_groups = asyncio.Queue(maxsize=cfg.get("max_inflight", 4) * 2)
        state = {"groups": 0}

        async def generate_loop():
            sem = asyncio.Semaphore(cfg.get("max_inflight", 4))

            async def one(examples, v):
                try:
                    res = await client.generate([ex["prompt"] for ex in examples], n=ng, max_tokens=cfg["max_tokens"],
                                                temperature=cfg.get("temperature", 1.0),
                                                generation_kwargs=cfg.get("generation_kwargs") or {})
                    await done_groups.put((examples, v, res))
                finally:
                    sem.release()

            tasks = set()
            while not stop.is_set():
                await sem.acquire()
                idx = torch.randint(0, len(rows), (ppc,), generator=g).tolist()
                t = asyncio.ensure_future(one([rows[i] for i in idx], version.value))
                tasks.add(t)
                t.add_done_callback(lambda f: (tasks.discard(f), f.exception() and err_q.put(repr(f.exception()))))
                heartbeat.value = time.monotonic()
            for t in tasks:
                t.cancel()

        async def score_loop():
            loop = asyncio.get_running_loop()
            while not stop.is_set():
                try:
                    examples, v, res = await asyncio.wait_for(done_groups.get(), timeout=0.2)
                except asyncio.TimeoutError:
                    continue
                prompts = [p for p in res["prompt_ids"] for _ in range(ng)]
                comps = res["completion_ids"]
                lps = [[x[0] for x in seq] for seq in res["logprobs"]]
                rep = [ex for ex in examples for _ in range(ng)]
                rewards = await loop.run_in_executor(None, reward_fn, rep, prompts, comps)
                adv = _advantages(list(rewards), ng, cfg.get("scale_rewards", True))
                for j, (p, c, lp) in enumerate(zip(prompts, comps, lps)):
                    smp = RolloutSample(list(p), list(c), list(lp), float(rewards[j]), float(adv[j]), int(v),
                                        state["groups"] + j // ng)
                    while not stop.is_set():
                        try:
                            out_q.put(smp, timeout=0.2)
                            break
                        except queue.Full:
                            heartbeat.value = time.monotonic()
                state["groups"] += len(examples)
                heartbeat.value = time.monotonic()

        try:
            await asyncio.gather(generate_loop(), score_loop())
        finally:
            await client.close()

    try:
        asyncio.run(run())
    except BaseException as e:  # noqa: BLE001  (reported to the parent)
        err_q.put("".join(traceback.format_exception_only(type(e), e)).strip())


class ProcessRolloutWorker:
    """Rollout generation and scoring in a spawned child process that talks to a generation server
    (trl/experimental/async_grpo/async_rollout_worker.py:914-1053).  ``reward_fn(examples, prompt_ids, completion_ids)``
    and the dataset rows must be picklable."""

    def __init__(self, dataset, server_url: str, reward_fn: Callable, num_generations: int, max_tokens: int = 64,
                 queue_maxsize: int = 1024, scale_rewards: bool = True, seed: int = 0, temperature: float = 1.0,
                 prompts_per_call: int = 4, max_inflight: int = 4, server_timeout: float = 60.0, generation_kwargs=None):
        import multiprocessing as mp

        self._ctx = mp.get_context("spawn")
        self.rows = [dict(dataset[i]) for i in range(len(dataset))]
        self.reward_fn = reward_fn
        self.cfg = dict(server_url=server_url, num_generations=num_generations, max_tokens=max_tokens,
                        scale_rewards=scale_rewards, seed=seed, temperature=temperature, prompts_per_call=prompts_per_call,
                        max_inflight=max_inflight, server_timeout=server_timeout, generation_kwargs=generation_kwargs or {})
        self.queue = self._ctx.Queue(maxsize=queue_maxsize)
        self._version = self._ctx.Value("i", 0)
        self._heartbeat = self._ctx.Value("d", time.monotonic())
        self._stop = self._ctx.Event()
        self._errors = self._ctx.Queue()
        self._proc = None
        self._failure: Optional[str] = None

    @property
    def model_version(self) -> int:
        return self._version.value

    def update_model_version(self, v: int) -> None:
        self._version.value = int(v)

    def start(self) -> None:
        if self._proc is None:
            self._heartbeat.value = time.monotonic()
            self._proc = self._ctx.Process(target=_process_main, name="trl-b200-rollout", daemon=True,
                                           args=(self.cfg, self.rows, self.reward_fn, self.queue, self._version,
                                                 self._heartbeat, self._stop, self._errors))
            self._proc.start()

    def check_health(self, stale_after_s: float) -> None:
        try:
            while True:
                self._failure = self._errors.get_nowait()
        except queue.Empty:
            pass
        if self._failure is not None:
            raise RuntimeError(f"rollout worker failed: {self._failure}")
        if self._proc is not None and not self._proc.is_alive() and not self._stop.is_set():
            raise RuntimeError(f"rollout worker exited (exit code {self._proc.exitcode})")
        if time.monotonic() - self._heartbeat.value > stale_after_s:
            raise RuntimeError(f"rollout worker produced nothing for {stale_after_s:.0f} s")

    def get(self, timeout: float) -> RolloutSample:
        return self.queue.get(timeout=timeout)

    def stop(self) -> None:
        self._stop.set()
        if self._proc is not None:
            self._proc.join(timeout=10)
            if self._proc.is_alive():
                self._proc.terminate()  # this exact child
                self._proc.join(timeout=5)
