"""Training-throughput rows besides the GRPO headline: DPO (sigmoid, frozen reference copy) and packed SFT.

    python -m trl_b200.benchmarks.train_throughput --task dpo --model llama-3-8b --shard full_shard
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29611 \
        -m trl_b200.benchmarks.train_throughput --task dpo --model llama-3-8b --shard full_shard

Synthetic token ids, random-init weights of the named architecture, bf16 compute with fp32 master weights.  Timed
with CUDA events over K optimizer steps after W warm-up steps, max over ranks; rank 0 prints one JSON line.  Every
step streams all weights (>= 15 GB), far more than L2, so no explicit flush is needed.
"""
from __future__ import annotations

import argparse
import json
import math
import tempfile

import torch


def _lengths(g, n, lo, hi, log_uniform=False):
    if log_uniform:
        u = torch.rand(n, generator=g)
        return [int(math.exp(math.log(lo) + float(x) * (math.log(hi) - math.log(lo)))) for x in u]
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


class SyntheticTokenizer:
    """Stand-in processing class for token-id datasets: only the attributes the trainers touch."""

    def __init__(self, vocab: int):
        self.vocab_size, self.pad_token, self.eos_token = vocab, "<pad>", "<eos>"
        self.pad_token_id, self.eos_token_id = 0, 1
        self.chat_template = None

    def batch_decode(self, ids, **kw):
        return ["" for _ in ids]

    def save_pretrained(self, path):
        pass


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--task", choices=["dpo", "sft"], default="dpo")
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--shard", default=None, help="ddp | zero2 | full_shard | full_shard_stream (default: full_shard when "
                                                  "world > 1)")
    ap.add_argument("--activation-offloading", action="store_true",
                    help="SFT: keep the checkpointed layer inputs in pinned host memory between forward and backward")
    ap.add_argument("--meta-init", action="store_true",
                    help="with full_shard_stream: build the model on the meta device and initialise every layer inside "
                         "the engine's slots, so the whole model never exists on one GPU (Llama-3-70B)")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--pairs-per-gpu", type=int, default=2)
    ap.add_argument("--tokens-per-gpu", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None, help="debug only: a truncated model is not the named config")
    ap.add_argument("--kernel-table", type=int, default=0, metavar="N",
                    help="after the timed steps, run one more step under the PyTorch profiler and add the N kernels with "
                         "the most device time to the JSON line (`top_kernels`: name, calls, total ms, share)")
    a = ap.parse_args()

    from trl_b200.models.configuration import preset
    from trl_b200.models.decoder import CausalLM
    from trl_b200.ops import cuda as K
    from trl_b200.parallel import dist as D

    D.init_process_group()
    world, rank = D.world_size(), D.rank()
    on_gpu = torch.cuda.is_available()  # the CPU path exists to check the script itself with a tiny preset
    dev = torch.device("cuda", D.local_rank()) if on_gpu else torch.device("cpu")
    if on_gpu:
        torch.cuda.set_device(dev)
    torch.manual_seed(1234)
    cfg = preset(a.model, **({"num_hidden_layers": a.layers} if a.layers else {}))
    if a.meta_init and (a.task != "sft" or (a.shard or "") != "full_shard_stream"):
        raise SystemExit("--meta-init goes with --task sft --shard full_shard_stream (DPO also needs a whole reference model)")
    model = CausalLM(cfg, dtype=torch.bfloat16 if on_gpu else torch.float32, device="meta" if a.meta_init else dev)
    tok = SyntheticTokenizer(cfg.vocab_size)
    shard = a.shard or ("full_shard" if world > 1 else "ddp")
    out_dir = tempfile.mkdtemp(prefix="bench_train_")
    g = torch.Generator().manual_seed(17)
    n_steps_total = 2 * a.steps + a.warmup + 2
    common = dict(output_dir=out_dir, max_steps=a.steps, logging_steps=1, save_strategy="no", bf16=on_gpu, report_to="none",
                  shard_mode=shard, gradient_checkpointing=True, seed=3, gradient_accumulation_steps=1)
    if a.task == "dpo":
        from trl_b200.trainer.dpo_config import DPOConfig
        from trl_b200.trainer.dpo_trainer import DPOTrainer

        n = a.pairs_per_gpu * world * n_steps_total
        pl, cl, rl = (_lengths(g, n, 64, 512) for _ in range(3))
        rows = [{"prompt_ids": torch.randint(2, cfg.vocab_size, (p,), generator=g).tolist(),
                 "chosen_ids": torch.randint(2, cfg.vocab_size, (c,), generator=g).tolist(),
                 "rejected_ids": torch.randint(2, cfg.vocab_size, (r,), generator=g).tolist()} for p, c, r in zip(pl, cl, rl)]
        args = DPOConfig(per_device_train_batch_size=a.pairs_per_gpu, learning_rate=5e-7, beta=0.1, loss_type="sigmoid",
                         max_length=None, **common)
        trainer = DPOTrainer(model, args=args, train_dataset=rows, processing_class=tok)
        metric = "dpo_train_tokens_per_s"
    else:
        from trl_b200.trainer.sft_config import SFTConfig
        from trl_b200.trainer.sft_trainer import SFTTrainer

        rows = []
        for _ in range(world * n_steps_total):  # one packed 8192-token sample per GPU and step
            left, docs = a.tokens_per_gpu, []
            while left > 0:
                L = min(left, _lengths(g, 1, 128, a.tokens_per_gpu, log_uniform=True)[0])
                docs.append(L)
                left -= L
            ids = torch.randint(2, cfg.vocab_size, (a.tokens_per_gpu,), generator=g).tolist()
            rows.append({"input_ids": ids, "seq_lengths": docs})
        args = SFTConfig(per_device_train_batch_size=1, learning_rate=1e-5, max_length=a.tokens_per_gpu, packing=False,
                         padding_free=True, activation_offloading=a.activation_offloading, **common)
        trainer = SFTTrainer(model, args, train_dataset=rows, processing_class=tok)
        metric = "sft_train_tokens_per_s"
    trainer.callback_handler.callbacks = [c for c in trainer.callback_handler.callbacks if type(c).__name__ != "PrinterCallback"]
    trainer.create_optimizer_and_scheduler(a.steps + a.warmup)
    trainer.engine.zero_grad()
    loader = iter(trainer.get_train_dataloader())
    model.train()

    def one_step():
        batch = next(loader)  # host tensors; counted on the host, no device sync
        am = batch.get("attention_mask")
        n = int(am.sum()) if am is not None else int(batch["input_ids"].numel())
        trainer.optimizer_step([batch])
        trainer.state.global_step += 1
        return n

    for _ in range(a.warmup):
        one_step()
    l0 = K.LAUNCHES[0]
    tokens = 0
    if on_gpu:
        K.check_status(dev)
        torch.cuda.synchronize()
        D.barrier()
        torch.cuda.reset_peak_memory_stats()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(a.steps):
            tokens += one_step()
        ev1.record()
        torch.cuda.synchronize()
        D.barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        K.check_status(dev)
    else:
        import time

        t0 = time.perf_counter()
        for _ in range(a.steps):
            tokens += one_step()
        ms = torch.tensor([(time.perf_counter() - t0) * 1e3])
    top = None
    if a.kernel_table and on_gpu:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            one_step()
            torch.cuda.synchronize()
        ev = [e for e in prof.key_averages() if getattr(e, "device_time_total", 0) > 0]
        total = sum(e.device_time_total for e in ev) or 1.0
        ev.sort(key=lambda e: -e.device_time_total)
        top = [{"kernel": e.key[:90], "calls": int(e.count), "ms": round(e.device_time_total / 1e3, 3),
                "share": round(e.device_time_total / total, 4)} for e in ev[: a.kernel_table]]
        top.append({"kernel": "(all kernels of the profiled step)", "calls": int(sum(e.count for e in ev)),
                    "ms": round(total / 1e3, 3), "share": 1.0})
    D.all_reduce(ms, "max")
    tok_t = torch.tensor([float(tokens)], device=dev)
    D.all_reduce(tok_t, "sum")
    tokens = float(tok_t)
    if rank == 0:
        print(json.dumps({
            "metric": metric, "value": float(tokens) / (float(ms) / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": float(ms) / a.steps, "higher_is_better": True,
            "scaling": "weak", "dtype": "bf16" if on_gpu else "fp32 (cpu)", "data": "synthetic",
            "config": {"model": f"{a.model} (random init)" + (f" TRUNCATED to {a.layers} layers" if a.layers else ""),
                       "task": a.task, "parallelism": f"dp{world} {shard}",
                       "per_gpu": f"{a.pairs_per_gpu} pairs, lengths U[64,512]" if a.task == "dpo"
                       else f"{a.tokens_per_gpu} packed tokens, doc lengths log-uniform [128,{a.tokens_per_gpu}]",
                       "l2_policy": "inputs larger than L2 (all weights streamed every step)"},
            **({"top_kernels": top} if top else {}),
            "gpu_launches": int(K.LAUNCHES[0] - l0), "peak_mem_gib": round(torch.cuda.max_memory_allocated() / 2**30, 1) if on_gpu else None}))
    D.barrier()
    if D.is_initialized():
        import torch.distributed as td

        td.destroy_process_group()


if __name__ == "__main__":
    main()
