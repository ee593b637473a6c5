"""Asynchronous client of the generation server for the rollout worker (role of
trl/experimental/async_grpo/vllm_client.py:44-100): many ``/generate`` requests in flight on one event loop, health
polling with a deadline, and the synchronous client's weight routes for the trainer side."""
from __future__ import annotations

import asyncio
import time

from ...generation.client import VLLMClient

__all__ = ["VLLMClient", "AsyncGenerationClient"]


class AsyncGenerationClient:
    def __init__(self, base_url: str, request_timeout: float = 600.0):
        self.base_url = base_url.rstrip("/")
        self.request_timeout = request_timeout
        self._session = None

    async def _sess(self):
        import aiohttp

        if self._session is None or self._session.closed:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.request_timeout))
        return self._session

    async def wait_healthy(self, total_timeout: float = 60.0, interval: float = 0.5) -> None:
        """Polls ``/health/`` until it answers 200; ConnectionError after ``total_timeout`` seconds."""
        import aiohttp

        t0 = time.monotonic()
        last = None
        while time.monotonic() - t0 < total_timeout:
            try:
                s = await self._sess()
                async with s.get(f"{self.base_url}/health/") as r:
                    if r.status == 200:
                        return
                    last = f"status {r.status}"
            except (aiohttp.ClientError, asyncio.TimeoutError, OSError) as e:
                last = repr(e)
            await asyncio.sleep(interval)
        raise ConnectionError(f"generation server at {self.base_url} not healthy after {total_timeout:.0f} s ({last})")

    async def generate(self, prompts, n=1, max_tokens=16, temperature=1.0, top_p=1.0, top_k=0, min_p=0.0,
                       repetition_penalty=1.0, generation_kwargs=None, retries: int = 3) -> dict:
        payload = dict(prompts=prompts, n=n, max_tokens=max_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                       min_p=min_p, repetition_penalty=repetition_penalty, logprobs=0, generation_kwargs=generation_kwargs or {})
        import aiohttp

        delay = 0.5
        for attempt in range(retries + 1):
            try:
                s = await self._sess()
                async with s.post(f"{self.base_url}/generate/", json=payload) as r:
                    if r.status == 200:
                        return await r.json()
                    if r.status not in (500, 502, 503) or attempt == retries:
                        raise RuntimeError(f"/generate/ failed: {r.status} {await r.text()}")
            except (aiohttp.ClientConnectionError, asyncio.TimeoutError):
                if attempt == retries:
                    raise
            await asyncio.sleep(delay)
            delay *= 2
        raise RuntimeError("unreachable")

    async def close(self):
        if self._session is not None and not self._session.closed:
            await self._session.close()
