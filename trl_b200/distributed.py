"""Backend abstraction seen by trainers (counterpart of trl/distributed.py:20-91).

The reference asks the accelerator whether parameters are partitioned (ZeRO-3 / FSDP) and, if so, gathers them around
code that reads weights directly.  Here the question goes to the training engine: a full-shard engine completes its
buckets with ``gather_full_params``; every other mode keeps full parameters resident."""
from __future__ import annotations

from contextlib import contextmanager


class DistributedBackend:
    def __init__(self, engine=None):
        self.engine = engine

    @property
    def is_zero3(self) -> bool:
        return getattr(self.engine, "mode", None) == "full_shard" and getattr(self.engine, "sharded", False)

    is_fsdp = is_zero3

    @contextmanager
    def gather_params(self, params=None):
        """Parameters are complete inside the block (a no-op unless the engine shards them)."""
        if self.is_zero3 and hasattr(self.engine, "gather_full_params"):
            self.engine.gather_full_params()
        yield

    @contextmanager
    def summon_full_params(self, module=None):
        with self.gather_params():
            yield
