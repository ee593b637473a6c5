"""Generation through a rollout server (``vllm_mode="server"``): the object the online trainers use in place of the
in-process engine.

Same interface as the engines (``generate(prompts, sampling_params)`` -> completions, ``sync_weights()``), carried over
the HTTP client.  With several training processes the prompts of all ranks are gathered, the main process talks to the
server, and every rank gets its own slice of the completions back; weights are pushed by the main process only (the
client picks CUDA IPC, packed binary bodies or one tensor per request, whatever the server offers), followed by a
prefix-cache reset.  The reference does the same around its vLLM client
(trl/generation/vllm_generation.py:444-501 weight sync, :636-699 gather / generate / broadcast / slice)."""
from __future__ import annotations

from ..parallel import dist as D
from ..rollout.engine import Completion
from ..rollout.sampling import SamplingParams


class ServerRollout:
    def __init__(self, model, base_url: str | None = None, host: str = "127.0.0.1", port: int = 8000,
                 timeout: float = 240.0, client=None):
        self.model = model
        self.client = client
        if self.client is None and D.is_main():
            from .client import RolloutClient

            host = "127.0.0.1" if host in ("0.0.0.0", "", None) else host
            self.client = RolloutClient(base_url=base_url, host=host, server_port=port, connection_timeout=timeout)
            self.client.init_communicator()
        self.stats = {"requests": 0, "generated_tokens": 0}

    def generate(self, prompts, sp: SamplingParams, images=None) -> list[Completion]:
        if images is not None:
            raise NotImplementedError("image prompts through the rollout server")
        mine = [list(p) for p in prompts]
        counts = D.gather_object([len(mine)])
        everyone = D.gather_object(mine)
        payload = [None]
        if D.is_main():
            res = self.client.generate(everyone, n=sp.n, repetition_penalty=sp.repetition_penalty, temperature=sp.temperature,
                                       top_p=sp.top_p, top_k=sp.top_k or 0, min_p=sp.min_p, max_tokens=sp.max_tokens,
                                       generation_kwargs={"seed": sp.seed, "greedy": sp.greedy,
                                                          "eos_prob_floor": sp.eos_prob_floor})
            comp, lps = res["completion_ids"], res["logprobs"]
            if len(comp) != len(everyone) * sp.n:
                raise RuntimeError(f"the server returned {len(comp)} completions for {len(everyone)} prompts x {sp.n}")
            payload[0] = (comp, [[x[0] if isinstance(x, (list, tuple)) else x for x in seq] for seq in lps])
            self.stats["requests"] += 1
        D.broadcast_object_list(payload, src=0)
        comp, lps = payload[0]
        start = sum(counts[:D.rank()]) * sp.n
        outs = []
        for j, p in enumerate(mine):
            for k in range(sp.n):
                i = start + j * sp.n + k
                ids = list(comp[i])
                stop = sp.eos_token_id is not None and bool(ids) and ids[-1] == sp.eos_token_id
                outs.append(Completion(p, ids, [float(x) for x in lps[i]], "stop" if stop else "length"))
                self.stats["generated_tokens"] += len(ids)
        return outs

    def sync_weights(self, model=None):
        """Pushes the policy's current weights to the server (main process); every rank waits for it."""
        if D.is_main():
            self.client.update_model_params(model if model is not None else self.model)
            self.client.reset_prefix_cache()
        D.barrier()

    def reset_prefix_cache(self):
        if D.is_main():
            self.client.reset_prefix_cache()
