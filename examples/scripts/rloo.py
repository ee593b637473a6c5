"""RLOO with a rule-based reward on prompt-only data (JSON lines with "prompt").

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/scripts/rloo.py \
        --model /path/to/model --data prompts.jsonl --out out/rloo
"""
from _common import parser, pick

from trl_b200 import RLOOConfig, RLOOTrainer


def brevity_reward(completion_ids, **kw):
    """Shorter completions score higher (a stand-in for a task reward)."""
    return [-0.01 * len(c) for c in completion_ids]


def main():
    a = parser(__doc__, "out/rloo").parse_args()
    model, tok, rows, kw = pick(a, "standard_prompt_only", per_device_train_batch_size=8, gradient_accumulation_steps=4,
                                learning_rate=1e-6, bf16=True, logging_steps=1, report_to="none", use_vllm=True,
                                shard_mode="zero2")
    cfg = RLOOConfig(output_dir=a.out, num_generations=4, max_completion_length=8 if a.smoke else 512, beta=0.05, **kw)
    trainer = RLOOTrainer(model, brevity_reward, cfg, train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
