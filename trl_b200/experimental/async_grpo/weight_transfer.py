"""Trainer -> generation server weight push (trl/experimental/async_grpo/weight_transfer.py:32-108).

The reference packs parameters into large NCCL broadcasts.  Here the trainer and the server share a box, so the packed
buffer goes device to device through a CUDA IPC handle when both sides are on GPUs, and as one binary HTTP body per
256 MB otherwise; a server that only knows the per-tensor route still works."""
from __future__ import annotations

import time


def push_weights(client, model, gather=None, transport: str | None = None) -> int:
    """Sends every parameter of ``model`` to the server behind ``client``; ``gather`` completes sharded parameters first
    (full-shard engines).  Returns the number of tensors sent."""
    if gather is not None:
        gather()
    if hasattr(client, "update_model_params"):
        n = client.update_model_params(model, transport=transport) if transport is not None else client.update_model_params(model)
        n = n if isinstance(n, int) else sum(1 for _ in model.named_parameters())
    else:
        n = 0
        for name, p in model.named_parameters():
            client.update_named_param(name, p.detach())
            n += 1
    client.reset_prefix_cache()
    return n


class WeightPusher:
    """Keeps the push statistics the trainer logs (``weight_sync/seconds``, ``weight_sync/tensors``)."""

    def __init__(self, client, gather=None, transport: str | None = None):
        self.client, self.gather, self.transport = client, gather, transport
        self.last_seconds, self.last_tensors, self.pushes = 0.0, 0, 0

    def __call__(self, model) -> int:
        t0 = time.perf_counter()
        self.last_tensors = push_weights(self.client, model, self.gather, self.transport)
        self.last_seconds = time.perf_counter() - t0
        self.pushes += 1
        return self.last_tensors
