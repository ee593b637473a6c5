"""``RolloutGeneration`` (alias ``VLLMGeneration``): the generate / sync_weights facade the online
trainers talk to (role of trl/generation/vllm_generation.py:111-704).

``mode="colocate"``  an in-process :class:`~trl_b200.rollout.engine.RolloutEngine` that reads the policy's
                     weights in place (``sync_weights`` is a no-op at TP=1, the reshard kernel at TP>1).
``mode="server"``    rank 0 talks to ``trl vllm-serve`` over HTTP; prompts are gathered to rank 0, completions
                     broadcast back and sliced per rank (vllm_generation.py:551-609).
"""
from __future__ import annotations

from ..parallel import dist as D
from ..rollout.sampling import SamplingParams


def extract_logprobs(outputs):
    """Engine outputs -> (logprobs, token ids) as nested lists [seq][token][rank]; NaN becomes None."""
    lps, ids = [], []
    for o in outputs:
        lps.append([[None if (lp != lp) else float(lp)] for lp in o.logprobs])
        ids.append([[int(t)] for t in o.token_ids])
    return lps, ids


class RolloutGeneration:
    def __init__(self, model, mode: str = "colocate", tensor_parallel_size: int = 1, max_num_seqs: int = 64,
                 max_model_len: int = 2048, server_base_url=None, server_host="127.0.0.1", server_port=8000,
                 server_timeout: float = 240.0, **kw):
        self.model, self.mode = model, mode
        if mode == "server":
            self.client = None
            if D.is_main():
                from .client import RolloutClient

                self.client = RolloutClient(server_base_url, server_host, server_port, connection_timeout=server_timeout)
        elif mode == "colocate":
            if D.world_size() % tensor_parallel_size != 0:
                raise ValueError(f"tensor_parallel_size ({tensor_parallel_size}) must divide world size ({D.world_size()})")
            if model.device.type == "cuda":
                from ..rollout.engine import RolloutEngine

                self.engine = RolloutEngine(model, max_num_seqs, max_model_len)
            else:
                from ..rollout.engine import EagerGenerator

                self.engine = EagerGenerator(model)
        else:
            raise ValueError("mode must be 'server' or 'colocate'")

    def sync_weights(self):
        if self.mode == "server":
            if D.is_main():
                self.client.update_model_params(self.model)
                self.client.reset_prefix_cache()
            D.barrier()
        else:
            if hasattr(self.engine, "sync_weights"):
                self.engine.sync_weights()

    def generate(self, prompts: list[list[int]], sp: SamplingParams):
        """Returns (prompt_ids, completion_ids, logprobs, logprob_token_ids) for this rank's prompts."""
        if self.mode == "colocate":
            outs = self.engine.generate(prompts, sp)
            lps, ids = extract_logprobs(outs)
            return [o.prompt_ids for o in outs], [o.token_ids for o in outs], lps, ids
        allp = D.gather_object(prompts)
        payload = [None]
        if D.is_main():
            res = self.client.generate(allp, n=sp.n, temperature=sp.temperature, top_p=sp.top_p, top_k=sp.top_k,
                                       min_p=sp.min_p, max_tokens=sp.max_tokens, repetition_penalty=sp.repetition_penalty)
            payload = [res]
        D.broadcast_object_list(payload)
        res = payload[0]
        per = len(prompts) * sp.n
        sl = slice(D.rank() * per, (D.rank() + 1) * per)
        rep = [p for p in prompts for _ in range(sp.n)]
        return rep, res["completion_ids"][sl], res["logprobs"][sl], res["logprob_token_ids"][sl]


VLLMGeneration = RolloutGeneration
