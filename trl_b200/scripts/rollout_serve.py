"""``trl vllm-serve`` / ``trl rollout-serve``: the rollout engine behind an HTTP API.

Endpoints and payloads follow trl/scripts/vllm_serve.py (:533-660 ``/generate``, ``/chat``, :857-871
``/get_sequence_logprobs``, :1124-1177 communicator / ``/update_named_param``, ``/reset_prefix_cache``,
``/health``, ``/get_world_size``; DP worker processes commanded over pipes :332-385,451-460; the 5 ms log-prob
batching window with a token budget :462-485).  Differences: the engine is this framework's own (paged KV,
CUDA-graph decode on GPUs, tensor-parallel engine groups, the eager generator on CPU); weights arrive device to
device through a CUDA IPC handle of the trainer's packed buffer (``/update_ipc/``, same box), or as one packed
binary body (``/update_packed/``), instead of a side NCCL broadcast per parameter; ``/update_named_param/`` stays
for single tensors.
"""
from __future__ import annotations

import argparse
import base64
import io
import itertools
from dataclasses import dataclass, field
from typing import Optional

import numpy as np


def chunk_list(lst: list, n: int) -> list[list]:
    """Split into n nearly equal contiguous chunks (the first ``len % n`` chunks get one extra)."""
    k, r = divmod(len(lst), n)
    out, i = [], 0
    for j in range(n):
        size = k + (1 if j < r else 0)
        out.append(lst[i:i + size])
        i += size
    return out


@dataclass
class ServeArguments:
    model: str = field(default="preset:tiny-qwen2", metadata={"help": "Checkpoint directory or preset name."})
    host: str = "127.0.0.1"
    port: int = 8000
    dtype: str = "auto"
    max_model_len: Optional[int] = 2048
    max_num_seqs: int = 64
    tensor_parallel_size: int = 1
    data_parallel_size: int = 1
    gpu_memory_utilization: float = 0.9
    enable_prefix_caching: Optional[bool] = None
    log_level: str = "info"


_DTYPES = {"torch.bfloat16": "bfloat16", "torch.float16": "float16", "torch.float32": "float32"}


def pack_tensors(named: list) -> tuple[dict, list]:
    """``[(name, tensor)]`` -> (metadata, [byte views]) of the packed wire format: one flat byte blob, every tensor
    at a 256-byte aligned offset.  The views alias the (host or device) tensors; nothing is copied here."""
    import torch

    meta, parts, off = [], [], 0
    for name, t in named:
        t = t.detach().contiguous()
        nbytes = t.numel() * t.element_size()
        pad = (-off) % 256
        off += pad
        meta.append({"name": name, "dtype": str(t.dtype), "shape": list(t.shape), "offset": off, "nbytes": nbytes, "pad": pad})
        parts.append(t.view(-1).view(torch.uint8))
        off += nbytes
    return {"tensors": meta, "total": off}, parts


class EngineHolder:
    def __init__(self, a: ServeArguments, device_index: int = 0, tp_group=None):
        import torch

        from ..models.hf_io import load_model
        from ..rollout.engine import EagerGenerator, RolloutEngine

        cuda = torch.cuda.is_available()
        if cuda:
            torch.cuda.set_device(device_index)
        dt = (torch.bfloat16 if cuda else torch.float32) if a.dtype == "auto" else a.dtype
        self.model = load_model(a.model, dtype=dt, device=f"cuda:{device_index}" if cuda else None).eval()
        self.tok = None
        import os

        if os.path.isdir(a.model):
            from transformers import AutoTokenizer

            self.tok = AutoTokenizer.from_pretrained(a.model)
        if cuda and tp_group is not None:
            from ..rollout.tp_engine import TPRolloutEngine

            self.engine = TPRolloutEngine(self.model, tp_group, max_num_seqs=a.max_num_seqs, max_model_len=a.max_model_len or 2048)
        elif cuda:
            self.engine = RolloutEngine(self.model, a.max_num_seqs, a.max_model_len or 2048)
        else:
            self.engine = EagerGenerator(self.model)
        self.world_size = a.tensor_parallel_size * a.data_parallel_size
        self.max_model_len = a.max_model_len or 2048
        self._named = None  # HF name -> view of the live (fused) parameter storage, built once

    def generate(self, prompts, sp):
        return self.engine.generate(prompts, sp)

    def sequence_logprobs(self, seqs, prompt_lens, temperature=1.0):
        """Log-probs of the tokens after each prompt.  All sequences of a call go through ONE packed, padding-free
        forward (chunks of at most 16 * max_model_len tokens), not one forward per sequence."""
        import torch

        from ..models.decoder import SeqCtx
        from ..ops import functional as ops

        outs = [None] * len(seqs)
        budget = 16 * self.max_model_len
        dev = self.model.device
        with torch.no_grad():
            i = 0
            while i < len(seqs):
                j, tot = i, 0
                while j < len(seqs) and (j == i or tot + len(seqs[j]) <= budget):
                    tot += len(seqs[j])
                    j += 1
                lens = [len(s) for s in seqs[i:j]]
                flat = torch.tensor([t for s in seqs[i:j] for t in s], device=dev)
                h = self.model.forward_hidden(flat, SeqCtx.from_lengths(lens, dev))
                starts = [0]
                for L in lens:
                    starts.append(starts[-1] + L)
                sel = torch.tensor([p for k, L in enumerate(lens) for p in range(starts[k] + prompt_lens[i + k] - 1, starts[k] + L - 1)],
                                   dtype=torch.long, device=dev)
                if sel.numel():
                    lp, _ = ops.lm_head_logprobs(h[sel], self.model.lm_head_weight, flat[sel + 1], temperature,
                                                 compute_entropy=False)
                    lp = lp.float().cpu().numpy()
                else:
                    lp = np.zeros(0, dtype=np.float32)
                o = 0
                for k, L in enumerate(lens):
                    n = L - prompt_lens[i + k]
                    outs[i + k] = lp[o:o + n]
                    o += n
                i = j
        return outs

    def _named_views(self):
        if self._named is None:
            self._named = self.model.state_dict_hf()  # views that alias the fused storage: built once, not per tensor
        return self._named

    def update_named_param(self, name, tensor):
        import torch

        sd = self._named_views()
        if name not in sd:
            raise KeyError(name)
        with torch.no_grad():
            sd[name].copy_(tensor.to(sd[name].device, sd[name].dtype))
        self._weights_changed()

    def update_packed(self, meta: dict, blob) -> int:
        """``blob``: a flat uint8 tensor (host or device) laid out as ``meta`` says; every tensor is copied into the
        live parameter it names."""
        import torch

        sd = self._named_views()
        with torch.no_grad():
            for m in meta["tensors"]:
                if m["name"] not in sd:
                    raise KeyError(m["name"])
                dst = sd[m["name"]]
                dt = getattr(torch, _DTYPES.get(m["dtype"], m["dtype"].replace("torch.", "")))
                src = blob[m["offset"]:m["offset"] + m["nbytes"]].view(dt).view(m["shape"])
                dst.copy_(src.to(dst.device, dst.dtype, non_blocking=True))
        self._weights_changed()
        return len(meta["tensors"])

    def update_ipc(self, meta: dict, ipc: dict) -> int:
        """Device-to-device: the trainer shares a CUDA IPC handle of its packed buffer; it is opened here and copied
        from without touching host memory."""
        import torch
        from torch.multiprocessing.reductions import rebuild_cuda_tensor

        blob = rebuild_cuda_tensor(torch.Tensor, (ipc["nbytes"],), (1,), 0, torch.UntypedStorage, torch.uint8,
                                   ipc["device"], base64.b64decode(ipc["handle"]), ipc["storage_size_bytes"],
                                   ipc["storage_offset_bytes"], False, base64.b64decode(ipc["ref_counter_handle"]),
                                   ipc["ref_counter_offset"], base64.b64decode(ipc["event_handle"]), ipc["event_sync_required"])
        n = self.update_packed(meta, blob)
        torch.cuda.synchronize()
        del blob
        return n

    def _weights_changed(self):
        if hasattr(self.engine, "sync_weights") and getattr(self.engine, "tp", 1) > 1:
            self.engine.sync_weights()  # tensor-parallel engines keep repacked slices


def _to_sampling(r: dict, eos):
    from ..rollout.sampling import SamplingParams

    gk = r.get("generation_kwargs") or {}
    return SamplingParams(n=r.get("n", 1), temperature=r.get("temperature", 1.0), top_p=r.get("top_p", 1.0),
                          top_k=max(r.get("top_k", 0), 0), min_p=r.get("min_p", 0.0),
                          repetition_penalty=r.get("repetition_penalty", 1.0), max_tokens=r.get("max_tokens", 16),
                          eos_token_id=eos, **{k: v for k, v in gk.items() if k in ("seed", "greedy", "eos_prob_floor")})


def llm_worker(a: ServeArguments, dp_rank: int, tp_rank: int, conn, rendezvous_port: int):
    """One engine process of a data-parallel replica (trl/scripts/vllm_serve.py:332-385): builds its engine on its own
    GPU, then serves commands from the parent over a pipe until it is told to shut down or the pipe closes."""
    import os

    import torch

    tp = a.tensor_parallel_size
    dev = dp_rank * tp + tp_rank
    group = None
    if tp > 1:
        import torch.distributed as td

        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(rendezvous_port + dp_rank), RANK=str(tp_rank),
                          WORLD_SIZE=str(tp), LOCAL_RANK=str(dev))
        torch.cuda.set_device(dev)
        td.init_process_group("nccl", rank=tp_rank, world_size=tp)
        group = td.group.WORLD
    holder = EngineHolder(a, device_index=dev if torch.cuda.is_available() else 0, tp_group=group)
    conn.send({"status": "ready", "eos": getattr(holder.tok, "eos_token_id", None) if holder.tok is not None
               else holder.model.config.eos_token_id})
    while True:
        try:
            cmd = conn.recv()
        except (EOFError, KeyboardInterrupt):
            break
        kind = cmd["type"]
        try:
            if kind == "shutdown":
                break
            if kind == "generate":
                outs = holder.generate(cmd["prompts"], _to_sampling(cmd["request"], cmd["eos"]))
                conn.send({"ok": [(o.prompt_ids, o.token_ids, o.logprobs) for o in outs]})
            elif kind == "logprobs":
                conn.send({"ok": holder.sequence_logprobs(cmd["sequences"], cmd["prompt_lengths"], cmd["temperature"])})
            elif kind == "update_named":
                holder.update_named_param(cmd["name"], cmd["tensor"])
                conn.send({"ok": 1})
            elif kind == "update_packed":
                import torch as _t

                conn.send({"ok": holder.update_packed(cmd["meta"], _t.frombuffer(bytearray(cmd["blob"]), dtype=_t.uint8))})
            elif kind == "update_ipc":
                conn.send({"ok": holder.update_ipc(cmd["meta"], cmd["ipc"])})
            elif kind == "reset_prefix_cache":
                if hasattr(holder.engine, "reset_prefix_cache"):
                    holder.engine.reset_prefix_cache()
                conn.send({"ok": 1})
            else:
                conn.send({"error": f"unknown command {kind!r}"})
        except Exception as e:  # noqa: BLE001  (reported to the parent, the worker keeps serving)
            conn.send({"error": f"{type(e).__name__}: {e}"})
    if tp > 1:
        import torch.distributed as td

        td.destroy_process_group()


class WorkerPool:
    """The engines behind the HTTP front end: one in-process engine (``data_parallel_size == tensor_parallel_size == 1``)
    or ``data_parallel_size`` replicas of ``tensor_parallel_size`` spawned processes each, commanded over pipes."""

    def __init__(self, a: ServeArguments, holder: EngineHolder | None = None):
        self.a, self.dp, self.tp = a, a.data_parallel_size, a.tensor_parallel_size
        self.local = holder
        self.conns, self.procs = [], []
        self.max_model_len = a.max_model_len or 2048
        if holder is None and self.dp == 1 and self.tp == 1:
            self.local = EngineHolder(a)
        if self.local is not None:
            self.eos = getattr(self.local.tok, "eos_token_id", None) if self.local.tok is not None \
                else self.local.model.config.eos_token_id
            self.tok, self.world_size = self.local.tok, self.local.world_size
            return
        import multiprocessing as mp
        import socket

        ctx = mp.get_context("spawn")
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        for d in range(self.dp):
            row = []
            for t in range(self.tp):
                parent, child = ctx.Pipe()
                p = ctx.Process(target=llm_worker, args=(a, d, t, child, port), daemon=True)
                p.start()
                self.procs.append(p)
                row.append(parent)
            self.conns.append(row)
        ready = [c.recv() for row in self.conns for c in row]  # blocks until every engine is built
        self.eos = ready[0]["eos"]
        self.world_size = self.dp * self.tp
        self.tok = None
        import os

        if os.path.isdir(a.model):
            from transformers import AutoTokenizer

            self.tok = AutoTokenizer.from_pretrained(a.model)

    @staticmethod
    def _result(msg):
        if "error" in msg:
            raise RuntimeError(msg["error"])
        return msg["ok"]

    def generate(self, prompt_ids: list, request: dict) -> list:
        """-> [(prompt_ids, completion_ids, logprobs)] in request order (``n`` per prompt)."""
        if self.local is not None:
            outs = self.local.generate(prompt_ids, _to_sampling(request, self.eos))
            return [(o.prompt_ids, o.token_ids, o.logprobs) for o in outs]
        # prompts are cut over the replicas, and inside a replica over its tensor-parallel ranks (every rank of a TP
        # group passes its share and gets the completions of its share back: the group runs the union)
        slots = [c for row in self.conns for c in row]
        chunks = chunk_list(prompt_ids, len(slots))
        if self.tp > 1 and any(len(c) == 0 for c in chunks):  # every rank of a TP group must join the collective call
            chunks = [c or [prompt_ids[0]] for c in chunks]
            pad = [len(c) == 0 for c in chunk_list(prompt_ids, len(slots))]
        else:
            pad = [False] * len(slots)
        for c, ch in zip(slots, chunks):
            if ch:
                c.send({"type": "generate", "prompts": ch, "request": request, "eos": self.eos})
        out = []
        for c, ch, is_pad in zip(slots, chunks, pad):
            if ch:
                res = self._result(c.recv())
                if not is_pad:
                    out += res
        return out

    def sequence_logprobs(self, sequences, prompt_lengths, temperature):
        if self.local is not None:
            return self.local.sequence_logprobs(sequences, prompt_lengths, temperature)
        heads = [row[0] for row in self.conns] if self.tp == 1 else [self.conns[0][0]]
        idx = chunk_list(list(range(len(sequences))), len(heads))
        for c, ix in zip(heads, idx):
            if ix:
                c.send({"type": "logprobs", "sequences": [sequences[i] for i in ix],
                        "prompt_lengths": [prompt_lengths[i] for i in ix], "temperature": temperature})
        out = [None] * len(sequences)
        for c, ix in zip(heads, idx):
            if ix:
                for i, lp in zip(ix, self._result(c.recv())):
                    out[i] = lp
        return out

    def broadcast(self, cmd: dict):
        if self.local is not None:
            kind = cmd["type"]
            if kind == "update_named":
                return self.local.update_named_param(cmd["name"], cmd["tensor"])
            if kind == "update_packed":
                import torch

                return self.local.update_packed(cmd["meta"], torch.frombuffer(bytearray(cmd["blob"]), dtype=torch.uint8))
            if kind == "update_ipc":
                return self.local.update_ipc(cmd["meta"], cmd["ipc"])
            if kind == "reset_prefix_cache" and hasattr(self.local.engine, "reset_prefix_cache"):
                return self.local.engine.reset_prefix_cache()
            return None
        slots = [c for row in self.conns for c in row]
        for c in slots:
            c.send(cmd)
        return [self._result(c.recv()) for c in slots]

    def close(self):
        for row in self.conns:
            for c in row:
                try:
                    c.send({"type": "shutdown"})
                except Exception:  # noqa: BLE001
                    pass
        for p in self.procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()  # this exact child


class LogprobBatcher:
    """``/get_sequence_logprobs`` requests that arrive within ``window_s`` of each other (5 ms) are scored in one
    engine call, up to ``token_budget`` tokens (``max_model_len x data_parallel_size``); a request that does not fit
    waits for the next batch (trl/scripts/vllm_serve.py:462-485,857-871)."""

    def __init__(self, pool: WorkerPool, window_s: float = 0.005):
        self.pool, self.window = pool, window_s
        self.budget = pool.max_model_len * max(1, pool.dp)
        self.pending: list = []
        self.task = None
        self.batches = 0

    async def submit(self, sequences, prompt_lengths, temperature):
        import asyncio

        fut = asyncio.get_running_loop().create_future()
        self.pending.append((sequences, prompt_lengths, temperature, fut))
        if self.task is None or self.task.done():
            self.task = asyncio.ensure_future(self._drain())
        return await fut

    async def _drain(self):
        import asyncio

        while self.pending:
            await asyncio.sleep(self.window)
            batch, tokens, temp = [], 0, None
            rest = []
            for item in self.pending:
                n = sum(len(s) for s in item[0])
                same = temp is None or item[2] == temp
                if same and (not batch or tokens + n <= self.budget):
                    batch.append(item)
                    tokens += n
                    temp = item[2]
                else:
                    rest.append(item)
            self.pending = rest
            seqs = [s for it in batch for s in it[0]]
            pls = [p for it in batch for p in it[1]]
            try:
                res = await asyncio.get_running_loop().run_in_executor(None, self.pool.sequence_logprobs, seqs, pls, temp)
                self.batches += 1
                o = 0
                for it in batch:
                    it[3].set_result(res[o:o + len(it[0])])
                    o += len(it[0])
            except Exception as e:  # noqa: BLE001
                for it in batch:
                    if not it[3].done():
                        it[3].set_exception(e)


try:  # request models live at module level so FastAPI can resolve the postponed annotations
    from pydantic import BaseModel
except Exception:  # pragma: no cover
    BaseModel = object
try:
    from fastapi import Request
except Exception:  # pragma: no cover
    Request = object


class GenerateRequest(BaseModel):
    prompts: list
    n: int = 1
    repetition_penalty: float = 1.0
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    max_tokens: int = 16
    logprobs: Optional[int] = 0
    generation_kwargs: dict = {}

class ChatRequest(GenerateRequest):
    prompts: list = []
    messages: list = []
    chat_template_kwargs: dict = {}
    tools: Optional[list] = None

class LogprobRequest(BaseModel):
    sequences: list
    prompt_lengths: list
    temperature: float = 1.0

class UpdateRequest(BaseModel):
    name: str
    dtype: str
    shape: list
    data: Optional[str] = None


def build_app(holder_or_pool):
    """FastAPI application over a :class:`WorkerPool` (an :class:`EngineHolder` is wrapped into a one-engine pool)."""
    from fastapi import FastAPI

    pool = holder_or_pool if isinstance(holder_or_pool, WorkerPool) else WorkerPool(ServeArguments(), holder=holder_or_pool)
    app = FastAPI()
    batcher = LogprobBatcher(pool)
    app.state.pool, app.state.logprob_batcher = pool, batcher

    def _run(prompt_ids, r):
        req = r.model_dump() if hasattr(r, "model_dump") else r.dict()
        outs = pool.generate(prompt_ids, req)
        return {"prompt_ids": [o[0] for o in outs][::r.n] if r.n else [], "completion_ids": [o[1] for o in outs],
                "logprobs": [[[lp] for lp in o[2]] for o in outs],
                "logprob_token_ids": [[[t] for t in o[1]] for o in outs]}

    @app.get("/health/")
    async def health():
        return {"status": "ok"}

    @app.get("/get_world_size/")
    async def world():
        return {"world_size": pool.world_size}

    @app.post("/generate/")
    async def generate(r: GenerateRequest):
        ids = [p if isinstance(p, list) else pool.tok(text=p)["input_ids"] for p in r.prompts]
        return _run(ids, r)

    @app.post("/chat/")
    async def chat(r: ChatRequest):
        if pool.tok is None:
            return {"error": "chat needs a tokenizer (serve a checkpoint directory)"}
        ids = [pool.tok.apply_chat_template(m, tools=r.tools, add_generation_prompt=True, tokenize=True,
                                            return_dict=True, **r.chat_template_kwargs)["input_ids"] for m in r.messages]
        return _run(ids, r)

    @app.post("/get_sequence_logprobs/")
    async def seq_logprobs(r: LogprobRequest):
        lps = await batcher.submit(r.sequences, r.prompt_lengths, r.temperature)
        enc = []
        for a in lps:
            buf = io.BytesIO()
            np.save(buf, np.asarray(a, dtype=np.float32))
            enc.append(base64.b64encode(buf.getvalue()).decode())
        return {"logprobs_b64": enc}

    @app.post("/init_communicator/")
    async def init_comm(req: dict):
        """Weight pushes need no side communicator here.  The answer tells the client which transports the server takes
        and on which device it runs, so that the client can pick CUDA IPC (same box, device to device) or the packed
        binary body; like the reference (vllm_serve.py:84-93) it names the device so a caller can refuse a clash."""
        import torch

        cuda = torch.cuda.is_available()
        return {"transports": (["ipc"] if cuda else []) + ["packed", "named"], "device": "cuda" if cuda else "cpu",
                "world_size": pool.world_size}

    @app.post("/update_named_param/")
    async def update(r: UpdateRequest):
        import torch

        if r.data is None:
            return {"message": "no data"}
        arr = np.load(io.BytesIO(base64.b64decode(r.data)), allow_pickle=False)
        t = torch.from_numpy(arr)
        if r.dtype == "torch.bfloat16":
            t = t.view(torch.bfloat16) if t.dtype == torch.int16 else t.to(torch.bfloat16)
        pool.broadcast({"type": "update_named", "name": r.name, "tensor": t.reshape(r.shape)})
        return {"message": f"updated {r.name}"}

    @app.post("/update_packed/")
    async def update_packed(request: Request):
        """Many tensors in one binary body: 8-byte little-endian metadata length, the JSON metadata of
        :func:`pack_tensors`, then the raw bytes.  No base64, no JSON around the payload, no per-tensor request."""
        import json as _json

        body = await request.body()
        n = int.from_bytes(body[:8], "little")
        meta = _json.loads(body[8:8 + n].decode())
        res = pool.broadcast({"type": "update_packed", "meta": meta, "blob": bytes(body[8 + n:])})
        return {"message": f"updated {len(meta['tensors'])} tensors", "workers": 1 if not isinstance(res, list) else len(res)}

    @app.post("/update_ipc/")
    async def update_ipc(req: dict):
        """Device-to-device weight update: ``req["ipc"]`` describes a CUDA IPC handle of the trainer's packed buffer
        (plain fields, no pickled objects), ``req["meta"]`` its layout.  Same box only."""
        pool.broadcast({"type": "update_ipc", "meta": req["meta"], "ipc": req["ipc"]})
        return {"message": f"updated {len(req['meta']['tensors'])} tensors device to device"}

    @app.post("/reset_prefix_cache/")
    async def reset():
        pool.broadcast({"type": "reset_prefix_cache"})
        return {"message": "ok"}

    @app.post("/close_communicator/")
    async def close():
        return {"message": "ok"}

    return app


def make_parser():
    from .utils import TrlParser

    return TrlParser([ServeArguments], prog="trl vllm-serve")


def main(argv=None) -> int:
    import uvicorn

    (a,) = make_parser().parse_args_and_config(argv)
    pool = WorkerPool(a)
    try:
        uvicorn.run(build_app(pool), host=a.host, port=a.port, log_level=a.log_level)
    finally:
        pool.close()
    return 0


if __name__ == "__main__":
    main()
