"""``trl vllm-serve`` / ``trl rollout-serve``: the rollout engine behind an HTTP API.

Endpoints and payloads follow trl/scripts/vllm_serve.py (:533-660 ``/generate``, ``/chat``, :857-871
``/get_sequence_logprobs``, :1124-1177 communicator / ``/update_named_param``, ``/reset_prefix_cache``,
``/health``, ``/get_world_size``).  Differences: the engine is this framework's own (paged KV, CUDA-graph
decode on GPUs, the eager generator on CPU); weights arrive as raw tensors in the request body (base64) instead
of a side NCCL broadcast, because trainer and server share one box and the colocated mode needs no transfer at all.
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


class EngineHolder:
    def __init__(self, a: ServeArguments):
        import torch

        from ..models.hf_io import load_model
        from ..rollout.engine import EagerGenerator, RolloutEngine

        cuda = torch.cuda.is_available()
        dt = (torch.bfloat16 if cuda else torch.float32) if a.dtype == "auto" else a.dtype
        self.model = load_model(a.model, dtype=dt, device="cuda" if cuda else None).eval()
        self.tok = None
        import os

        if os.path.isdir(a.model):
            from transformers import AutoTokenizer

            self.tok = AutoTokenizer.from_pretrained(a.model)
        self.engine = RolloutEngine(self.model, a.max_num_seqs, a.max_model_len or 2048) if cuda else EagerGenerator(self.model)
        self.world_size = a.tensor_parallel_size * a.data_parallel_size

    def generate(self, prompts, sp):
        return self.engine.generate(prompts, sp)

    def sequence_logprobs(self, seqs, prompt_lens, temperature=1.0):
        import torch

        from ..models.decoder import SeqCtx
        from ..ops import functional as ops

        outs = []
        with torch.no_grad():
            for ids, pl in zip(seqs, prompt_lens):
                flat = torch.tensor(ids, device=self.model.device)
                ctx = SeqCtx.from_lengths([len(ids)], self.model.device)
                h = self.model.forward_hidden(flat, ctx)
                lp, _ = ops.lm_head_logprobs(h[pl - 1:-1], self.model.lm_head_weight, flat[pl:], temperature,
                                             compute_entropy=False)
                outs.append(lp.float().cpu().numpy())
        return outs

    def update_named_param(self, name, tensor):
        import torch

        from ..models.hf_io import load_hf_state_dict

        sd = self.model.state_dict_hf()
        if name not in sd:
            raise KeyError(name)
        with torch.no_grad():
            sd[name].copy_(tensor.to(sd[name].device, sd[name].dtype))  # HF-named views alias the fused storage


try:  # request models live at module level so FastAPI can resolve the postponed annotations
    from pydantic import BaseModel
except Exception:  # pragma: no cover
    BaseModel = object


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


def build_app(holder: EngineHolder):
    from fastapi import FastAPI

    from ..rollout.sampling import SamplingParams

    app = FastAPI()

    def _run(prompt_ids, r):
        eos = getattr(holder.tok, "eos_token_id", None) if holder.tok is not None else holder.model.config.eos_token_id
        sp = SamplingParams(n=r.n, temperature=r.temperature, top_p=r.top_p, top_k=max(r.top_k, 0), min_p=r.min_p,
                            repetition_penalty=r.repetition_penalty, max_tokens=r.max_tokens, eos_token_id=eos,
                            **{k: v for k, v in r.generation_kwargs.items() if k in ("seed", "greedy", "eos_prob_floor")})
        outs = holder.generate(prompt_ids, sp)
        return {"prompt_ids": [o.prompt_ids for o in outs][::r.n] if r.n else [], "completion_ids": [o.token_ids for o in outs],
                "logprobs": [[[lp] for lp in o.logprobs] for o in outs],
                "logprob_token_ids": [[[t] for t in o.token_ids] for o in outs]}

    @app.get("/health/")
    async def health():
        return {"status": "ok"}

    @app.get("/get_world_size/")
    async def world():
        return {"world_size": holder.world_size}

    @app.post("/generate/")
    async def generate(r: GenerateRequest):
        ids = [p if isinstance(p, list) else holder.tok(text=p)["input_ids"] for p in r.prompts]
        return _run(ids, r)

    @app.post("/chat/")
    async def chat(r: ChatRequest):
        if holder.tok is None:
            return {"error": "chat needs a tokenizer (serve a checkpoint directory)"}
        ids = [holder.tok.apply_chat_template(m, tools=r.tools, add_generation_prompt=True, tokenize=True,
                                              return_dict=True, **r.chat_template_kwargs)["input_ids"] for m in r.messages]
        return _run(ids, r)

    @app.post("/get_sequence_logprobs/")
    async def seq_logprobs(r: LogprobRequest):
        lps = holder.sequence_logprobs(r.sequences, r.prompt_lengths, r.temperature)
        enc = []
        for a in lps:
            buf = io.BytesIO()
            np.save(buf, a.astype(np.float32))
            enc.append(base64.b64encode(buf.getvalue()).decode())
        return {"logprobs_b64": enc}

    @app.post("/init_communicator/")
    async def init_comm(req: dict):
        return {"message": "weights travel in the request body; no side communicator is needed"}

    @app.post("/update_named_param/")
    async def update(r: UpdateRequest):
        import torch

        if r.data is None:
            return {"message": "no data"}
        arr = np.load(io.BytesIO(base64.b64decode(r.data)), allow_pickle=False)
        t = torch.from_numpy(arr)
        if r.dtype == "torch.bfloat16":
            t = t.view(torch.bfloat16) if t.dtype == torch.int16 else t.to(torch.bfloat16)
        holder.update_named_param(r.name, t.reshape(r.shape))
        return {"message": f"updated {r.name}"}

    @app.post("/reset_prefix_cache/")
    async def reset():
        if hasattr(holder.engine, "reset_prefix_cache"):
            holder.engine.reset_prefix_cache()
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
    uvicorn.run(build_app(EngineHolder(a)), host=a.host, port=a.port, log_level=a.log_level)
    return 0


if __name__ == "__main__":
    main()
