"""Worker: GRPO on two gloo ranks with either zero2 (generation reads the policy in place) or streamed full shard
(generation reads a whole replica refreshed from the slices); writes the logged trajectory (rank 0)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from trl_b200.parallel import dist as D
from trl_b200.testing import make_dataset, make_tiny_model, make_tiny_tokenizer
from trl_b200.trainer.grpo_config import GRPOConfig
from trl_b200.trainer.grpo_trainer import GRPOTrainer


def reward(completion_ids, **kw):
    return [float(sum(c) % 7) for c in completion_ids]


def main():
    out, mode, kind = sys.argv[1], sys.argv[2], sys.argv[3]
    D.init_process_group(use_cpu=True)
    torch.manual_seed(0)
    model = make_tiny_model("tiny-qwen3-moe" if kind == "moe" else "tiny-qwen2", seed=0)
    args = GRPOConfig(output_dir=out + "_o", per_device_train_batch_size=4, num_generations=4, max_completion_length=5,
                      max_steps=3, logging_steps=1, learning_rate=1e-3, use_cpu=True, save_strategy="no", report_to="none",
                      beta=0.04, shard_mode=mode, gradient_checkpointing=True, shuffle_dataset=False, seed=11)
    tr = GRPOTrainer(model, reward, args, train_dataset=make_dataset("standard_prompt_only", 16),
                     processing_class=make_tiny_tokenizer())
    tr.train()
    if mode == "full_shard_stream":  # policy slices, a whole generation replica, and a sliced frozen reference
        assert tr._gen_model is not None and tr._ref_stream is not None and tr._ref_stream.frozen
        assert all(l.master.numel() == l.numel // 2 for l in tr._ref_stream.layers)
    if D.is_main():
        hist = [{k: h[k] for k in ("loss", "grad_norm", "reward", "kl")} for h in tr.state.log_history if "reward" in h]
        with open(out, "w") as f:
            json.dump(hist, f)
    D.barrier()


if __name__ == "__main__":
    main()
