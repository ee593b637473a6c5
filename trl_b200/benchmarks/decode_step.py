"""Where one decode step of the rollout engine goes: device time per kernel (PyTorch profiler, eager launches) and the
wall time of the captured step (CUDA graph replays, CUDA events).

    python -m trl_b200.benchmarks.decode_step [--model qwen2.5-7b] [--batch 64] [--ctx 512]

With dependent launch the kernels of the chain overlap: a kernel's profiled duration includes the time it waits for
its predecessor, so the per-kernel times add up to more than the step."""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--steps", type=int, default=4)
    a = ap.parse_args()
    from torch.profiler import ProfilerActivity, profile

    from trl_b200.models.configuration import preset
    from trl_b200.models.decoder import CausalLM
    from trl_b200.rollout.engine import RolloutEngine
    from trl_b200.rollout.sampling import SamplingParams

    cfg = preset(a.model, eos_token_id=1, pad_token_id=0)
    model = CausalLM(cfg, dtype=torch.bfloat16, device="cuda").eval()
    n, new = 8, 64
    plen = a.ctx - new
    eng = RolloutEngine(model, max_num_seqs=a.batch, max_model_len=a.ctx + 16, poll_every=16)
    prompts = [torch.randint(2, cfg.vocab_size, (plen,)).tolist() for _ in range(a.batch // n)]
    sp = SamplingParams(n=n, max_tokens=new, eos_token_id=None, seed=1)
    eng.generate(prompts, sp)  # fills the cache and captures the graph

    def reset(frac=1.0):
        eng.seq_lens.fill_(a.ctx - 2)
        eng.finished.zero_()
        if frac < 1:
            eng.seq_lens[int(a.batch * frac):] = -1

    with torch.no_grad():
        reset()
        for _ in range(3):
            eng._decode_step(sp, a.ctx)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(a.steps):
                eng._decode_step(sp, a.ctx)
            torch.cuda.synchronize()
    ev = sorted((e for e in prof.key_averages() if e.device_time_total > 0), key=lambda e: -e.device_time_total)
    rows = [{"kernel": e.key[:80], "calls_per_step": e.count / a.steps, "us_per_step": round(e.device_time_total / a.steps, 1)}
            for e in ev[:12]]
    out = {"model": a.model, "batch": a.batch, "context": a.ctx, "kernels": rows,
           "sum_of_kernel_times_us_per_step": round(sum(e.device_time_total for e in ev) / a.steps, 1),
           "kernels_in_graph": eng._graph_kernels}
    g = eng._graph
    for frac in (1.0, 0.25):
        reset(frac)
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(32):
            reset(frac)
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        out[f"graph_replay_ms_per_step_active_{frac}"] = round(e0.elapsed_time(e1) / 32, 3)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
