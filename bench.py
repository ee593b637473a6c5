"""Headline benchmark: one GRPO optimizer step (rollout generation + reward + reference
log-probs + policy forward/backward + optimizer) on the Qwen2.5-7B architecture.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 3 --warmup 3

Work per GPU is fixed (weak scaling): 8 prompts x 8 completions = 64 sequences per GPU and step,
i.e. 64 prompts / 512 completions per step on 8 GPUs.  Prompts are 256 uniform-random token ids,
completions are sampled at temperature 1.0 with an end-of-sequence probability floor of 1/512
and at most 1024 new tokens; the reward is the fraction of even token ids minus 0.001 x length.
Weights are random-init (no checkpoints or datasets are reachable).  Rank 0 prints one JSON line.

``value`` is device-timed (CUDA events, max over ranks) around ``Trainer.optimizer_step``;
``e2e`` is the same metric through the public ``GRPOTrainer.train()`` call, wall-clock, with
the per-step host->device copy of the prompts from pinned memory and the device->host read of
the loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
os.environ.setdefault("TRL_B200_PROFILE_MAX_OVER_RANKS", "1")  # phases_s: a phase is as slow as its slowest rank
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts-per-gpu", type=int, default=8)
    ap.add_argument("--num-generations", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--max-new", type=int, default=1024)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--rollout-tp", type=int, default=0, help="0 = 2 when more than one GPU, else 1")
    ap.add_argument("--layers", type=int, default=None, help="debug only: truncating the model invalidates the number")
    ap.add_argument("--grad-ckpt", default="on", choices=["on", "off"],
                    help="activation checkpointing (an out-of-memory warm-up step switches it back on)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the DPO / SFT Llama-3-8B rows that are measured after the headline and reported under "
                         "'extras'")
    ap.add_argument("--shard", default=None,
                    help="engine shard mode (default: zero2 with more than one GPU, else ddp); full_shard_stream holds "
                         "1 / N of every layer per GPU for models whose training state does not fit otherwise")
    ap.add_argument("--meta-init", action="store_true",
                    help="with --shard full_shard_stream: build the policy on the meta device (initialised slice by slice)")
    ap.add_argument("--ckpt-layers", default="all",
                    help="with checkpointing on: 'all' (default) recomputes every layer; n recomputes only the first n "
                         "layers and keeps the activations of the rest; 'auto' lets the trainer measure in the first two "
                         "warm-up steps how many layers fit (gradient_checkpointing_kwargs={'num_layers': 'auto'}).  With "
                         "micro-batches of varying length keeping activations did not pay here: the allocator's "
                         "remapping cost what the recomputation saved")
    return ap.parse_args()


def reference_arm():
    """The reference needs accelerate (not installed, not in the offline wheelhouse)."""
    line = {"impl": "reference"}
    try:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref"))
        from trl import GRPOTrainer  # noqa: F401

        line["unavailable"] = "reference imports, but no vLLM/accelerate launch path is wired for it here"
    except Exception as e:  # noqa: BLE001
        line["unavailable"] = f"reference cannot import its trainers offline: {type(e).__name__}: {str(e)[:160]}"
    print(json.dumps(line))
    return 0


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms during the timed region (read-only)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class SyntheticTokenizer:
    """Stand-in processing class for token-id prompts: only the attributes the trainer touches."""

    def __init__(self, vocab: int):
        self.vocab_size, self.pad_token, self.eos_token = vocab, "<pad>", "<eos>"
        self.pad_token_id, self.eos_token_id = 0, 1
        self.chat_template = None

    def batch_decode(self, ids, **kw):
        return ["" for _ in ids]

    def save_pretrained(self, path):
        pass


def even_fraction_reward(completion_ids, **kw):
    out = []
    for ids in completion_ids:
        n = max(1, len(ids))
        out.append(sum(1 for t in ids if t % 2 == 0) / n - 0.001 * len(ids))
    return out


def main():
    a = parse()
    if a.impl == "reference":
        return reference_arm()
    import torch

    from trl_b200.models.configuration import preset
    from trl_b200.models.decoder import CausalLM
    from trl_b200.ops import cuda as K
    from trl_b200.parallel import dist as D
    from trl_b200.trainer.grpo_config import GRPOConfig
    from trl_b200.trainer.grpo_trainer import GRPOTrainer

    D.init_process_group()
    world, rank = D.world_size(), D.rank()
    dev = torch.device("cuda", D.local_rank())
    torch.cuda.set_device(dev)
    torch.manual_seed(1234)  # same weights on every rank
    overrides = {"num_hidden_layers": a.layers} if a.layers else {}
    cfg = preset(a.model, eos_token_id=1, pad_token_id=0, **overrides)
    if a.meta_init and a.shard != "full_shard_stream":
        raise SystemExit("--meta-init needs --shard full_shard_stream")
    model = CausalLM(cfg, dtype=torch.bfloat16, device="meta" if a.meta_init else dev)
    tok = SyntheticTokenizer(cfg.vocab_size)
    g = torch.Generator().manual_seed(99)
    n_prompts = a.prompts_per_gpu * world * (a.steps + a.warmup + a.steps + 2)
    rows = [{"prompt": torch.randint(2, cfg.vocab_size, (a.prompt_len,), generator=g).tolist()} for _ in range(n_prompts)]
    per_rank = a.prompts_per_gpu * a.num_generations
    ga = per_rank // a.micro_batch
    out_dir = tempfile.mkdtemp(prefix="bench_grpo_")
    rollout_tp = a.rollout_tp or (2 if world > 1 else 1)
    grad_ckpt = a.grad_ckpt == "on"
    shard_mode = a.shard or ("zero2" if world > 1 else "ddp")
    if a.ckpt_layers in ("all", None) or shard_mode == "full_shard_stream":
        ckpt_kwargs = None
    elif a.ckpt_layers == "auto":
        if a.warmup < 3:
            raise SystemExit("--ckpt-layers auto settles in the first two steps: use --warmup >= 3 or --ckpt-layers all")
        ckpt_kwargs = {"num_layers": "auto"}
    else:
        ckpt_kwargs = {"num_layers": int(a.ckpt_layers)}
    args = GRPOConfig(output_dir=out_dir, per_device_train_batch_size=a.micro_batch, gradient_accumulation_steps=ga,
                      num_generations=a.num_generations, max_completion_length=a.max_new, temperature=1.0, beta=0.04,
                      epsilon=0.2, learning_rate=1e-6, max_steps=a.steps, logging_steps=1, save_strategy="no",
                      bf16=True, use_vllm=True, vllm_mode="colocate", eos_prob_floor=1.0 / 512, shuffle_dataset=False,
                      shard_mode=a.shard or ("zero2" if world > 1 else "ddp"), report_to="none", seed=7,
                      vllm_importance_sampling_correction=False, gradient_checkpointing=grad_ckpt,
                      gradient_checkpointing_kwargs=ckpt_kwargs,
                      vllm_tensor_parallel_size=rollout_tp)
    trainer = GRPOTrainer(model, even_fraction_reward, args, train_dataset=rows, processing_class=tok)
    trainer.callback_handler.callbacks = [c for c in trainer.callback_handler.callbacks
                                          if type(c).__name__ != "PrinterCallback"]
    trainer.create_optimizer_and_scheduler(a.steps + a.warmup)
    trainer.engine.zero_grad()
    loader = iter(trainer.get_train_dataloader())
    model.train()

    def one_step():
        batches = [next(loader) for _ in range(ga)]
        n0 = trainer._total_train_tokens
        loss, gnorm, _ = trainer.optimizer_step(batches)
        trainer.state.global_step += 1
        return loss, trainer._total_train_tokens - n0

    for _ in range(a.warmup):
        try:
            one_step()
        except torch.cuda.OutOfMemoryError:
            # not enough room without recomputation after all: switch it on (all ranks see the same sizes only
            # approximately, so the decision is made job-wide below) and repeat the step
            grad_ckpt = True
            oom = torch.ones(1, device=dev)
        else:
            oom = torch.zeros(1, device=dev)
        D.all_reduce(oom, "max")
        if float(oom) > 0:
            grad_ckpt = True
            model.gradient_checkpointing_enable()
            trainer.engine.zero_grad()
            trainer._buffered_inputs = None
            torch.cuda.empty_cache()
    K.check_status(dev)
    comm_check = trainer.engine.comm_selfcheck() if world > 1 and hasattr(trainer.engine, "comm_selfcheck") else None
    gen0 = trainer._total_generated_tokens
    torch.cuda.synchronize()
    D.barrier()
    clocks = ClockSampler(D.local_rank())
    if rank == 0:
        clocks.start()
    launches0 = K.LAUNCHES[0]
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.reset_peak_memory_stats()
    ev0.record()
    seq_tokens = 0
    for _ in range(a.steps):
        _, ntok = one_step()
        seq_tokens += ntok  # prompt + completion tokens of all ranks (already gathered)
    ev1.record()
    torch.cuda.synchronize()
    D.barrier()
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    D.all_reduce(ms, "max")
    gen_local = torch.tensor([float(trainer._total_generated_tokens - gen0)], device=dev)  # already job-wide
    clk = clocks.stop() if rank == 0 else {}
    launches = K.LAUNCHES[0] - launches0
    K.check_status(dev)
    peak_gb = torch.cuda.max_memory_allocated() / 2**30
    step_s = float(ms) / 1e3 / a.steps
    total_tokens = float(seq_tokens) + float(gen_local)  # trained (prompt+completion) + generated tokens, whole job
    value = total_tokens / (float(ms) / 1e3)

    e2e = None
    if not a.no_e2e:
        # public API: GRPOTrainer.train() for `steps` more optimizer steps, wall clock
        trainer.args.max_steps = trainer.state.global_step + a.steps
        trainer._buffered_inputs = None
        t_tok0, g0 = trainer._total_train_tokens, trainer._total_generated_tokens
        start_step = trainer.state.global_step

        torch.cuda.synchronize()
        D.barrier()
        t0 = time.perf_counter()
        trainer.train()
        torch.cuda.synchronize()
        D.barrier()
        dt = torch.tensor([time.perf_counter() - t0], device=dev)
        D.all_reduce(dt, "max")
        gl = torch.tensor([float(trainer._total_generated_tokens - g0)], device=dev)
        e_tokens = float(trainer._total_train_tokens - t_tok0) + float(gl)
        h2d = per_rank // a.num_generations * a.prompt_len * 8 + trainer._rollout.block_table_host.numel() * 4
        e2e = {"value": e_tokens / float(dt), "unit": "tokens/s", "step_s": float(dt) / a.steps,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(4 + per_rank * a.max_new * 8 // 16),
               "steps": trainer.state.global_step - start_step}
    if rank == 0:
        line = {
            "metric": "grpo_gen_plus_train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": float(ms) / a.steps, "step_s": step_s,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": f"{a.model} (random init)" + (f" TRUNCATED to {a.layers} layers" if a.layers else ""),
                       "global_batch": per_rank * world, "prompts_per_step": a.prompts_per_gpu * world,
                       "num_generations": a.num_generations, "seq_len": a.prompt_len + a.max_new,
                       "prompt_len": a.prompt_len, "max_new_tokens": a.max_new, "eos_prob_floor": 1.0 / 512,
                       "beta": 0.04, "epsilon": 0.2, "loss_type": "dapo", "micro_batch": a.micro_batch, "activation_checkpointing": (bool(grad_ckpt) if not (grad_ckpt and getattr(model, "checkpoint_num_layers", None) is not None) else f"first {model.checkpoint_num_layers} layers"),
                       "parallelism": f"dp{world} {args.shard_mode}, rollout tp{rollout_tp} x {world // rollout_tp} replicas "
                                      f"(colocated)",
                       "l2_policy": "inputs larger than L2: every step streams >=15 GB of weights",
                       "tokens_counted": "generated completion tokens + trained (prompt+completion) tokens"},
            "gpu_launches": int(launches), "clocks": clk, "peak_mem_gib": round(peak_gb, 1),
            "generated_tokens_per_step": float(gen_local) / a.steps,
        }
        if comm_check is not None:
            line["comm_selfcheck"] = comm_check
        if e2e is not None:
            line["e2e"] = e2e
            hist = [h for h in trainer.state.log_history if any(k.startswith("profiling/") for k in h)]
            if hist:
                keys = sorted({k for h in hist for k in h if k.startswith("profiling/") or k == "step_time"})
                line["phases_s"] = {k.replace("profiling/Time taken: GRPOTrainer.", ""): round(
                    sum(h.get(k, 0.0) for h in hist[-a.steps:]) / max(1, len(hist[-a.steps:])), 3) for k in keys}
        rs = getattr(trainer._rollout, "stats", None)
        if rs and "t_decode" in rs:  # only with TRL_B200_ROLLOUT_TIMING=1 (diagnostic: it adds host syncs)
            line["rollout_sections_s_total"] = {k: round(v, 3) for k, v in rs.items() if k.startswith("t_")}
            line["rollout_decode_steps_total"] = rs.get("decode_steps")
    else:
        line = None
    # ---- the DPO / SFT rows: measured after everything of the headline has been released -----------------------------
    master_port = int(os.environ.get("MASTER_PORT", "29500"))
    D.barrier()
    if D.is_initialized():
        import torch.distributed as td

        td.destroy_process_group()
    extras = None
    if not a.no_extras and not a.layers:
        del trainer, model, loader
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        free_gib = torch.cuda.mem_get_info()[0] / 2**30
        extras = run_extras(world, rank, dev.index, master_port)
        if extras is not None:
            extras["free_gib_after_headline"] = round(free_gib, 1)
    if rank == 0:
        if extras is not None:
            line["extras"] = extras
        print(json.dumps(line))
    return 0


def run_extras(world: int, rank: int, local_rank: int, master_port: int) -> dict:
    """DPO (2 pairs per GPU, lengths U[64,512], frozen reference) and packed SFT (8192 tokens per GPU) on the
    Llama-3-8B architecture with the full-shard engine, each in child processes of its own (one per rank, on this
    rank's GPU, with its own rendezvous), so that a failure there cannot take the headline number with it."""
    out = {}
    shard = "full_shard" if world > 1 else "ddp"
    for i, (task, key) in enumerate((("dpo", f"dpo_llama3_8b_{shard}_tok_s"), ("sft", f"sft_llama3_8b_{shard}_tok_s"))):
        # the launcher's agent-store variables must not reach the children: with them rank 0 would not open the
        # rendezvous store on the new port and every rank would wait for it
        env = {k: v for k, v in os.environ.items() if not k.startswith("TORCHELASTIC_")}
        env.update(RANK=str(rank), LOCAL_RANK=str(local_rank), WORLD_SIZE=str(world),
                   MASTER_ADDR=os.environ.get("MASTER_ADDR", "127.0.0.1"), MASTER_PORT=str(master_port + 37 + i))
        if out.get("_timed_out"):
            out[key] = None
            out[key + "_note"] = "skipped: the previous child run exceeded its time limit"
            continue
        cmd = [sys.executable, "-m", "trl_b200.benchmarks.train_throughput", "--task", task, "--model", "llama-3-8b",
               "--shard", shard, "--steps", "3", "--warmup", "2"]
        p = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                             cwd=os.path.dirname(os.path.abspath(__file__)))
        try:
            so, se = p.communicate(timeout=200)
        except subprocess.TimeoutExpired:
            p.kill()  # this exact child, nothing else
            so, se = p.communicate()
            out[key] = None
            out[key + "_note"] = "child run exceeded 200 s"
            out["_timed_out"] = True
            continue
        if rank != 0:
            continue
        rec = None
        for ln in so.splitlines():
            if ln.startswith("{"):
                try:
                    rec = json.loads(ln)
                except ValueError:
                    pass
        if p.returncode == 0 and rec is not None:
            out[key] = rec["value"]
            out[key + "_detail"] = {k: rec.get(k) for k in ("ms_per_step", "steps", "warmup", "n_gpus", "peak_mem_gib", "config")}
        else:
            out[key] = None
            out[key + "_note"] = (se.strip().splitlines() or ["no output"])[-1][:200]
    out.pop("_timed_out", None)
    return out


if __name__ == "__main__":
    sys.exit(main())
