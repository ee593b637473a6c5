"""Generalised knowledge distillation: a student learns from a teacher on a mix of dataset completions and its own
generations (JSON lines with "prompt" and "completion").

    python examples/scripts/gkd.py --model /path/to/student --teacher /path/to/teacher --data sft.jsonl --out out/gkd
"""
from _common import parser, pick

from trl_b200.experimental.gkd import GKDConfig, GKDTrainer


def main():
    ap = parser(__doc__, "out/gkd")
    ap.add_argument("--teacher", default=None)
    a = ap.parse_args()
    model, tok, rows, kw = pick(a, "standard_prompt_completion", per_device_train_batch_size=4, gradient_accumulation_steps=4,
                                learning_rate=1e-5, bf16=True, logging_steps=10, report_to="none")
    if a.smoke:
        from trl_b200.testing import make_tiny_model

        teacher = make_tiny_model("tiny-qwen2", seed=1)
    else:
        teacher = a.teacher or a.model
    cfg = GKDConfig(output_dir=a.out, lmbda=0.5, beta=0.5, temperature=0.9, max_new_tokens=8 if a.smoke else 256, **kw)
    trainer = GKDTrainer(model, teacher, cfg, train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
