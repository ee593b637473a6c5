"""GRPO of a vision-language model on image prompts with a rule-based reward.

Each JSON line: {"image": "img.png", "prompt": [{"role": "user", "content": "..."}], "solution": "..."}

    python examples/scripts/grpo_vlm.py --model /path/to/llava-checkpoint --data prompts.jsonl --out out/grpo_vlm
"""
from _common import load_rows, parser
from dpo_vlm import smoke_setup

from trl_b200 import GRPOConfig, GRPOTrainer, VisionLanguageModel


def contains_solution(completions, solution=None, **kw):
    """1 when the reference answer appears in the completion text, else 0."""
    texts = [c[0]["content"] if isinstance(c, list) else c for c in completions]
    return [float(s is not None and str(s).lower() in t.lower()) for t, s in zip(texts, solution or [None] * len(texts))]


def main():
    a = parser(__doc__, "out/grpo_vlm").parse_args()
    if a.smoke:
        model, proc, pairs = smoke_setup()
        rows = [{"image": r["images"][0], "prompt": r["prompt"], "solution": r["chosen"][0]["content"]} for r in pairs]
        kw = dict(use_cpu=True, max_steps=2, learning_rate=1e-3, per_device_train_batch_size=4, num_generations=4,
                  max_completion_length=6)
    else:
        from trl_b200.scripts.utils import load_processing_class

        model = VisionLanguageModel.from_pretrained(a.model, dtype="bfloat16")
        proc, rows = load_processing_class(a.model), load_rows(a.data)
        kw = dict(bf16=True, learning_rate=1e-6, per_device_train_batch_size=8, gradient_accumulation_steps=4,
                  num_generations=8, max_completion_length=256, use_vllm=True)
    cfg = GRPOConfig(output_dir=a.out, beta=0.0, logging_steps=1, save_strategy="no", report_to="none", **kw)
    trainer = GRPOTrainer(model, contains_solution, cfg, train_dataset=rows, processing_class=proc)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
