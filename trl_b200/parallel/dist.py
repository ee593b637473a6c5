"""Process-group plumbing: one process per GPU, NCCL on GPUs, gloo on CPU.

Every helper degrades to the identity when no process group exists, so trainer
code is written once.  The reference gets the same services from accelerate
(``gather``, ``reduce``, ``gather_object``, ``broadcast_object_list``,
``main_process_first``; call sites listed in trl/trainer/grpo_trainer.py:1702,
2427, 3199 and trl/trainer/sft_trainer.py:1758-1830).
"""
from __future__ import annotations

import contextlib
import datetime
import os
import socket

import torch
import torch.distributed as td


def is_initialized() -> bool:
    return td.is_available() and td.is_initialized()


def world_size() -> int:
    return td.get_world_size() if is_initialized() else 1


def rank() -> int:
    return td.get_rank() if is_initialized() else 0


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", 0))


def is_main() -> bool:
    return rank() == 0


def ensure_master_addr_port(addr: str | None = None, port: int | None = None) -> None:
    """Respect the environment; default to 127.0.0.1 and a free port
    (behaviour of trl/trainer/utils.py:75-113, loopback instead of ``localhost``)."""
    os.environ.setdefault("MASTER_ADDR", addr or "127.0.0.1")
    cur = os.environ.get("MASTER_PORT")
    if port is not None:
        os.environ["MASTER_PORT"] = str(port)
    elif cur in (None, "", "0", "auto"):
        for cand in (29500, 23456, 12355, 12345):
            with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
                try:
                    s.bind(("127.0.0.1", cand))
                    os.environ["MASTER_PORT"] = str(cand)
                    return
                except OSError:
                    continue
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            s.bind(("127.0.0.1", 0))
            os.environ["MASTER_PORT"] = str(s.getsockname()[1])


def init_process_group(use_cpu: bool = False, timeout_s: int = 1800) -> None:
    """Join the job described by RANK/WORLD_SIZE/MASTER_*; no-op for a single process."""
    if is_initialized():
        return
    ws = int(os.environ.get("WORLD_SIZE", 1))
    if ws <= 1:
        return
    ensure_master_addr_port()
    cuda = torch.cuda.is_available() and not use_cpu
    if cuda:
        torch.cuda.set_device(local_rank())
    kw = {}
    if cuda:
        kw["device_id"] = torch.device("cuda", local_rank())
    td.init_process_group(backend="nccl" if cuda else "gloo", timeout=datetime.timedelta(seconds=timeout_s), **kw)


def barrier():
    if is_initialized():
        td.barrier()


def all_reduce(t: torch.Tensor, op: str = "sum", group=None) -> torch.Tensor:
    if not is_initialized() or world_size() == 1:
        return t
    ops = {"sum": td.ReduceOp.SUM, "max": td.ReduceOp.MAX, "min": td.ReduceOp.MIN}
    if op == "mean":
        td.all_reduce(t, td.ReduceOp.SUM, group=group)
        t /= td.get_world_size(group)
    else:
        td.all_reduce(t, ops[op], group=group)
    return t


def gather(t: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenate equally-shaped tensors from every rank along dim 0."""
    if not is_initialized() or world_size() == 1:
        return t
    t = t.contiguous()
    if t.ndim == 0:
        t = t[None]
    out = torch.empty((td.get_world_size(group) * t.shape[0],) + t.shape[1:], dtype=t.dtype, device=t.device)
    td.all_gather_into_tensor(out, t, group=group)
    return out


def gather_object(obj_list: list, group=None) -> list:
    if not is_initialized() or world_size() == 1:
        return list(obj_list)
    outs = [None] * td.get_world_size(group)
    td.all_gather_object(outs, list(obj_list), group=group)
    return [x for o in outs for x in o]


def broadcast_object_list(objs: list, src: int = 0, group=None) -> list:
    if is_initialized() and world_size() > 1:
        td.broadcast_object_list(objs, src=src, group=group)
    return objs


def broadcast(t: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
    if is_initialized() and world_size() > 1:
        td.broadcast(t, src=src, group=group)
    return t


def pad_across_processes(t: torch.Tensor, dim: int = 0, pad_value=0) -> torch.Tensor:
    if not is_initialized() or world_size() == 1:
        return t
    n = torch.tensor([t.shape[dim]], device=t.device)
    all_reduce(n, "max")
    if int(n) == t.shape[dim]:
        return t
    shape = list(t.shape)
    shape[dim] = int(n) - t.shape[dim]
    return torch.cat([t, t.new_full(shape, pad_value)], dim=dim)


@contextlib.contextmanager
def main_process_first():
    """Rank 0 runs the block first (dataset caches), the others afterwards."""
    if rank() != 0:
        barrier()
    yield
    if rank() == 0:
        barrier()


def new_subgroups_by_enumeration(groups: list[list[int]]):
    """Return the group this rank belongs to (all ranks must call)."""
    mine = None
    for g in groups:
        pg = td.new_group(g)
        if rank() in g:
            mine = pg
    return mine
