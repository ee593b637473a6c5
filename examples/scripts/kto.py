"""KTO on unpaired feedback (JSON lines with "prompt", "completion", "label": true / false).

    python examples/scripts/kto.py --model /path/to/model --data feedback.jsonl --out out/kto
"""
from _common import parser, pick

from trl_b200 import KTOConfig, KTOTrainer


def main():
    a = parser(__doc__, "out/kto").parse_args()
    model, tok, rows, kw = pick(a, "standard_unpaired_preference", per_device_train_batch_size=4, gradient_accumulation_steps=4,
                                learning_rate=5e-7, bf16=True, logging_steps=10, report_to="none")
    cfg = KTOConfig(output_dir=a.out, beta=0.1, desirable_weight=1.0, undesirable_weight=1.0, **kw)
    trainer = KTOTrainer(model, args=cfg, train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
