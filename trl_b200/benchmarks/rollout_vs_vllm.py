"""Rollout generation of the GRPO benchmark configuration: this framework's engine against vLLM on the same GPU.

    python -m trl_b200.benchmarks.rollout_vs_vllm --engine ours
    python -m trl_b200.benchmarks.rollout_vs_vllm --engine vllm        # needs the installed vllm package to start here
    # tensor parallel over 2 GPUs, 128 sequences (64 per GPU, as in the GRPO benchmark):
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m trl_b200.benchmarks.rollout_vs_vllm --engine ours
    python -m trl_b200.benchmarks.rollout_vs_vllm --engine vllm --tp 2 --prompts 16

Work: random-init Qwen2.5-7B architecture in bf16, 8 prompts of 256 uniform-random token ids, 8 completions each
(64 sequences), at most 1024 new tokens, temperature 1.  Completion lengths follow the benchmark's end-of-sequence
floor (probability 1/512 per step, capped at 1024): our engine applies the floor while sampling; vLLM gets one request
per completion with ``ignore_eos`` and a ``max_tokens`` drawn from the same capped geometric law (seeded), which is the
same amount of decode work in distribution without a custom logits processor.  Timed: wall clock around the generate
call after one warm-up call, synchronised on both sides.  One JSON line per engine.

Each engine runs in its own process (``--engine``) because both want most of the GPU's memory.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time


def _lengths(n: int, floor: float, cap: int, seed: int) -> list[int]:
    import random

    rng = random.Random(seed)
    out = []
    for _ in range(n):
        k = 1
        while k < cap and rng.random() >= floor:
            k += 1
        out.append(k)
    return out


def run_ours(a) -> dict:
    import torch

    from trl_b200.models.configuration import preset
    from trl_b200.models.decoder import CausalLM
    from trl_b200.rollout.engine import RolloutEngine
    from trl_b200.rollout.sampling import SamplingParams

    cfg = preset(a.model, eos_token_id=1, pad_token_id=0)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = 0
    if world > 1:  # launched through torch.distributed.run: one tensor-parallel group over all ranks
        import torch.distributed as td

        from trl_b200.parallel import dist as D
        from trl_b200.rollout.tp_engine import TPRolloutEngine

        D.init_process_group()
        rank = D.rank()
        torch.cuda.set_device(D.local_rank())
    torch.manual_seed(0)
    model = CausalLM(cfg, dtype=torch.bfloat16, device="cuda").eval()
    if world > 1:
        eng = TPRolloutEngine(model, td.group.WORLD, max_num_seqs=a.prompts * a.n, max_model_len=a.prompt_len + a.max_new + 16)
    else:
        eng = RolloutEngine(model, max_num_seqs=a.prompts * a.n, max_model_len=a.prompt_len + a.max_new + 16)
    g = torch.Generator().manual_seed(1 + rank)  # every rank brings its own prompts; the group decodes the union
    prompts = [torch.randint(2, cfg.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(a.prompts)]
    sp = SamplingParams(n=a.n, max_tokens=a.max_new, temperature=1.0, eos_token_id=1, eos_prob_floor=a.eos_floor, seed=3)
    eng.generate(prompts, sp)  # warm-up: graph capture
    times, toks = [], []
    for it in range(a.iters):
        sp.seed = 100 + it
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = eng.generate(prompts, sp)
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
        toks.append(sum(len(o.token_ids) for o in outs))
    i = sorted(range(len(times)), key=lambda k: times[k])[len(times) // 2]
    n_tok = toks[i]
    if world > 1:  # tokens of all ranks' completions in the median iteration
        t = torch.tensor([float(x) for x in toks], device="cuda")
        td.all_reduce(t)
        n_tok = int(t[i])
        td.barrier()
        if rank != 0:
            td.destroy_process_group()
            return {}
        td.destroy_process_group()
    return {"engine": "trl_b200 " + (f"TPRolloutEngine (TP{world})" if world > 1 else "RolloutEngine"),
            "generate_s": round(times[i], 3), "generated_tokens": n_tok, "tokens_per_s": round(n_tok / times[i], 1),
            "decode_steps": eng.stats.get("decode_steps")}


def run_vllm(a) -> dict:
    import torch
    from vllm import LLM, SamplingParams

    from trl_b200.models.configuration import preset

    cfg = preset(a.model, eos_token_id=1, pad_token_id=0)
    d = tempfile.mkdtemp(prefix="vllm_cfg_")
    hf = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": cfg.hidden_size,
          "intermediate_size": cfg.intermediate_size, "num_hidden_layers": cfg.num_hidden_layers,
          "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads,
          "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta,
          "max_position_embeddings": 32768, "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "bfloat16",
          "bos_token_id": 0, "eos_token_id": 1}
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", tensor_parallel_size=a.tp,
              max_model_len=a.prompt_len + a.max_new + 16, max_num_seqs=a.prompts * a.n, gpu_memory_utilization=0.6,
              enable_prefix_caching=True, seed=0)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(2, cfg.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(a.prompts)]
    times, toks = [], []
    for it in range(a.iters + 1):  # the first call is the warm-up
        lens = _lengths(a.prompts * a.n, a.eos_floor, a.max_new, seed=100 + it)
        reqs = [{"prompt_token_ids": prompts[i // a.n]} for i in range(a.prompts * a.n)]
        sps = [SamplingParams(n=1, temperature=1.0, max_tokens=L, ignore_eos=True, detokenize=False, seed=it * 1000 + i)
               for i, L in enumerate(lens)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(reqs, sps, use_tqdm=False)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if it:
            times.append(dt)
            toks.append(sum(len(o.outputs[0].token_ids) for o in outs))
    i = sorted(range(len(times)), key=lambda k: times[k])[len(times) // 2]
    import vllm

    return {"engine": f"vllm {vllm.__version__} (dummy weights, prefix caching, TP{a.tp})", "generate_s": round(times[i], 3),
            "generated_tokens": toks[i], "tokens_per_s": round(toks[i] / times[i], 1)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--engine", choices=["ours", "vllm"], default="ours")
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--n", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--max-new", type=int, default=1024)
    ap.add_argument("--eos-floor", type=float, default=1.0 / 512)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--tp", type=int, default=1)
    a = ap.parse_args()
    try:
        rec = run_ours(a) if a.engine == "ours" else run_vllm(a)
    except Exception as e:  # noqa: BLE001  (an engine that cannot start here is a result too)
        rec = {"engine": a.engine, "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
    if not rec:
        return 0
    seqs = a.prompts * a.n * (int(os.environ.get("WORLD_SIZE", "1")) if a.engine == "ours" else 1)
    rec["config"] = {"model": f"{a.model} (random init)", "sequences": seqs, "prompt_len": a.prompt_len,
                     "max_new_tokens": a.max_new, "eos_prob_floor": a.eos_floor, "dtype": "bf16"}
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
