"""HTTP client of the rollout server (API of trl/generation/vllm_client.py:58-745: ``generate``, ``chat``,
``init_communicator``, ``update_named_param``, ``update_model_params``, ``get_sequence_logprobs``,
``reset_prefix_cache``, ``close_communicator``), with the same retry policy (5 retries, backoff 2 s on
500/502/503) and health polling with a timeout."""
from __future__ import annotations

import base64
import io
import time

import numpy as np

from ..scripts.rollout_serve import chunk_list  # noqa: F401  (re-exported)


class RolloutClient:
    def __init__(self, base_url: str | None = None, host: str = "127.0.0.1", server_port: int = 8000,
                 group_port: int = 51216, connection_timeout: float = 0.0):
        import requests
        from requests.adapters import HTTPAdapter
        from urllib3.util.retry import Retry

        self.session = requests.Session()
        retry = Retry(total=5, connect=5, read=5, status=3, status_forcelist=[500, 502, 503], backoff_factor=2,
                      allowed_methods=["POST", "GET"])
        self.session.mount("http://", HTTPAdapter(max_retries=retry))
        self.session.mount("https://", HTTPAdapter(max_retries=retry))
        self.base_url = (base_url or f"http://{host}:{server_port}").rstrip("/")
        self.check_server(connection_timeout)

    def check_server(self, total_timeout: float = 0.0, retry_interval: float = 2.0):
        import requests

        start = time.time()
        while True:
            try:
                r = requests.get(f"{self.base_url}/health/", timeout=5)
                if r.status_code == 200:
                    return
            except requests.exceptions.RequestException as e:
                if time.time() - start >= total_timeout:
                    raise ConnectionError(f"The rollout server can't be reached at {self.base_url} after "
                                          f"{total_timeout} seconds. Make sure it is running "
                                          "(`trl vllm-serve --model <path>`).") from e
            time.sleep(retry_interval)

    def _post(self, path, payload):
        r = self.session.post(f"{self.base_url}/{path}/", json=payload)
        if r.status_code != 200:
            raise Exception(f"Request failed: {r.status_code}, {r.text}")
        return r.json()

    def generate(self, prompts, n=1, repetition_penalty=1.0, temperature=1.0, top_p=1.0, top_k=0, min_p=0.0,
                 max_tokens=16, logprobs=0, generation_kwargs=None, **unused):
        return self._post("generate", dict(prompts=prompts, n=n, repetition_penalty=repetition_penalty,
                                           temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p,
                                           max_tokens=max_tokens, logprobs=logprobs, generation_kwargs=generation_kwargs or {}))

    def chat(self, messages, n=1, max_tokens=16, temperature=1.0, tools=None, chat_template_kwargs=None, **kw):
        return self._post("chat", dict(messages=messages, n=n, max_tokens=max_tokens, temperature=temperature, tools=tools,
                                       chat_template_kwargs=chat_template_kwargs or {}, generation_kwargs=kw.get("generation_kwargs", {})))

    def get_sequence_logprobs(self, sequences, prompt_lengths, temperature=1.0, chunk_size: int = 64):
        out = []
        for s in range(0, len(sequences), chunk_size):
            res = self._post("get_sequence_logprobs", dict(sequences=sequences[s:s + chunk_size],
                                                           prompt_lengths=prompt_lengths[s:s + chunk_size],
                                                           temperature=temperature))
            out += [np.load(io.BytesIO(base64.b64decode(b))) for b in res["logprobs_b64"]]
        return out

    def init_communicator(self, device=0):
        """Asks the server which weight transports it takes (``ipc``: CUDA IPC, device to device on one box;
        ``packed``: one binary body for many tensors; ``named``: one tensor per request) and remembers them."""
        info = self._post("init_communicator", {"device": str(device)})
        self.transports = info.get("transports", ["named"])
        self.server_device = info.get("device", "cpu")
        return info

    def update_named_param(self, name: str, weights):
        import torch

        w = weights.detach().cpu().contiguous()
        arr = w.view(torch.int16).numpy() if w.dtype == torch.bfloat16 else w.numpy()
        buf = io.BytesIO()
        np.save(buf, arr)
        return self._post("update_named_param", dict(name=name, dtype=str(weights.dtype), shape=list(weights.shape),
                                                     data=base64.b64encode(buf.getvalue()).decode()))

    def update_packed(self, named: list, chunk_bytes: int = 256 << 20) -> int:
        """Pushes ``[(name, tensor)]`` in binary bodies of at most ``chunk_bytes``: no base64, no JSON around the
        payload, one request per chunk instead of one per tensor."""
        import json

        import torch

        from ..scripts.rollout_serve import pack_tensors

        sent, group, size = 0, [], 0

        def flush():
            nonlocal group, size, sent
            if not group:
                return
            meta, parts = pack_tensors(group)
            blob = bytearray(meta["total"])
            for m, part in zip(meta["tensors"], parts):
                blob[m["offset"]:m["offset"] + m["nbytes"]] = part.cpu().numpy().tobytes()
            head = json.dumps(meta).encode()
            r = self.session.post(f"{self.base_url}/update_packed/", data=len(head).to_bytes(8, "little") + head + bytes(blob),
                                  headers={"Content-Type": "application/octet-stream"})
            if r.status_code != 200:
                raise Exception(f"Request failed: {r.status_code}, {r.text}")
            sent += len(group)
            group, size = [], 0

        for name, t in named:
            nb = t.numel() * t.element_size()
            if group and size + nb > chunk_bytes:
                flush()
            group.append((name, t))
            size += nb
        flush()
        return sent

    def update_ipc(self, named: list) -> int:
        """Device-to-device push on one box: the tensors are packed into one CUDA buffer whose IPC handle travels in
        the request (plain fields); the server opens it and copies into its parameters without touching host memory.
        The buffer is kept until the server has answered."""
        import torch
        from torch.multiprocessing.reductions import reduce_tensor

        from ..scripts.rollout_serve import pack_tensors

        meta, parts = pack_tensors(named)
        dev = parts[0].device
        flat = torch.empty(meta["total"], dtype=torch.uint8, device=dev)
        for m, part in zip(meta["tensors"], parts):
            flat[m["offset"]:m["offset"] + m["nbytes"]].copy_(part)
        torch.cuda.synchronize(dev)
        _, args = reduce_tensor(flat)
        (_, _, _, _, _, _, device, handle, storage_size, storage_offset, _, ref_handle, ref_offset, event_handle,
         event_sync) = args
        b64 = lambda b: base64.b64encode(bytes(b)).decode()  # noqa: E731
        ipc = {"nbytes": meta["total"], "device": int(device), "handle": b64(handle), "storage_size_bytes": int(storage_size),
               "storage_offset_bytes": int(storage_offset), "ref_counter_handle": b64(ref_handle),
               "ref_counter_offset": int(ref_offset), "event_handle": b64(event_handle), "event_sync_required": bool(event_sync)}
        self._post("update_ipc", {"meta": meta, "ipc": ipc})
        del flat
        return len(named)

    def update_model_params(self, model, transport: str | None = None) -> int:
        """Pushes every parameter (HF names).  ``transport``: ``"ipc"`` | ``"packed"`` | ``"named"``; by default the
        fastest one the server and the tensors allow (CUDA tensors + a CUDA server on this box -> IPC)."""
        sd = model.state_dict_hf() if hasattr(model, "state_dict_hf") else dict(model.named_parameters())
        named = [(k, v.detach()) for k, v in sd.items()]
        if transport is None:
            if not hasattr(self, "transports"):
                try:
                    self.init_communicator()
                except Exception:  # noqa: BLE001  (an older server: one tensor per request)
                    self.transports = ["named"]
            local = self.base_url.split("//")[-1].split(":")[0] in ("127.0.0.1", "localhost")
            cuda = bool(named) and named[0][1].is_cuda
            transport = "ipc" if ("ipc" in self.transports and cuda and local) else (
                "packed" if "packed" in self.transports else "named")
        if transport == "ipc":
            return self.update_ipc(named)
        if transport == "packed":
            return self.update_packed(named)
        for name, p in named:
            self.update_named_param(name, p)
        return len(named)

    def reset_prefix_cache(self):
        return self._post("reset_prefix_cache", {})

    def close_communicator(self):
        return self._post("close_communicator", {})


VLLMClient = RolloutClient
