"""GRPO with rule-based rewards (answer accuracy + <think> format) on prompts with a "solution" column.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/scripts/grpo_math.py \
        --model /path/to/qwen2.5-7b-instruct --data math.jsonl --out out/grpo
The rollout engine runs inside the training processes (``use_vllm=True, vllm_mode="colocate"``); with
``vllm_tensor_parallel_size=2`` pairs of GPUs share one decode replica.
"""
import argparse
import json

from trl_b200 import GRPOConfig, GRPOTrainer
from trl_b200.rewards import accuracy_reward, think_format_reward


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", required=True)
    ap.add_argument("--out", default="out/grpo")
    ap.add_argument("--tp", type=int, default=1)
    a = ap.parse_args()
    rows = [json.loads(line) for line in open(a.data)]  # {"prompt": [...messages...] or str, "solution": "..."}
    cfg = GRPOConfig(output_dir=a.out, per_device_train_batch_size=8, gradient_accumulation_steps=8, num_generations=8,
                     max_completion_length=1024, temperature=1.0, beta=0.0, learning_rate=1e-6, bf16=True, use_vllm=True,
                     vllm_mode="colocate", vllm_tensor_parallel_size=a.tp, shard_mode="zero2", logging_steps=1,
                     log_completions=True, report_to="none")
    trainer = GRPOTrainer(a.model, [accuracy_reward, think_format_reward], cfg, train_dataset=rows)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
