"""2-rank worker (gloo): generation through a rollout server with several training processes.  The main process is the
only one that talks to the (fake) server; every rank must get the completions of its own prompts, in order."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from trl_b200.generation.server_rollout import ServerRollout
from trl_b200.parallel import dist as D
from trl_b200.rollout.sampling import SamplingParams


class FakeClient:
    """Completion of a prompt = its token ids reversed, then the sample index; log-probs = -position."""

    def __init__(self):
        self.calls, self.pushed, self.resets = [], 0, 0

    def generate(self, prompts, n=1, **kw):
        self.calls.append((len(prompts), n, kw.get("max_tokens"), kw.get("generation_kwargs", {}).get("seed")))
        comp, lps = [], []
        for p in prompts:
            for k in range(n):
                ids = list(reversed(p)) + [k]
                comp.append(ids)
                lps.append([[-float(i)] for i in range(len(ids))])
        return {"prompt_ids": prompts, "completion_ids": comp, "logprobs": lps}

    def update_model_params(self, model):
        self.pushed += 1

    def reset_prefix_cache(self):
        self.resets += 1


def main():
    D.init_process_group(use_cpu=True)
    rank = D.rank()
    client = FakeClient() if D.is_main() else None
    eng = ServerRollout(model=object(), client=client)
    mine = [[10 + rank, 11, 12], [20 + rank]] if rank == 0 else [[30, 31], [40], [50, 51, 52, 53]]  # 2 and 3 prompts
    sp = SamplingParams(n=2, max_tokens=7, temperature=1.0, eos_token_id=0, seed=5)
    outs = eng.generate(mine, sp)
    assert len(outs) == len(mine) * 2
    for j, p in enumerate(mine):
        for k in range(2):
            o = outs[j * 2 + k]
            assert o.prompt_ids == p and o.token_ids == list(reversed(p)) + [k], (rank, j, k, o)
            assert o.logprobs == [-float(i) for i in range(len(p) + 1)]
            assert o.finish_reason == ("stop" if k == 0 else "length")  # sample 0 ends with the eos id 0
    eng.sync_weights()
    if D.is_main():
        assert client.calls == [(5, 2, 7, 5)] and client.pushed == 1 and client.resets == 1
        print("SERVER_ROLLOUT_OK")
    D.barrier()


if __name__ == "__main__":
    main()
