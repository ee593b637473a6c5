"""Trainer -> generation server weight push (trl/experimental/async_grpo/weight_transfer.py:20-108)."""
from __future__ import annotations


def push_weights(client, model, gather=None) -> int:
    """Sends every parameter of ``model`` to the server behind ``client``; ``gather`` completes sharded parameters first
    (full-shard engines).  Returns the number of tensors sent."""
    if gather is not None:
        gather()
    n = 0
    for name, p in model.named_parameters():
        client.update_named_param(name, p.detach())
        n += 1
    client.reset_prefix_cache()
    return n
