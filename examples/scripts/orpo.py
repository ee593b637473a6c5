"""ORPO: supervised loss on the chosen answer plus an odds-ratio penalty, no reference model.

    python examples/scripts/orpo.py --model /path/to/model --data prefs.jsonl --out out/orpo
"""
from _common import parser, pick

from trl_b200.experimental.orpo import ORPOConfig, ORPOTrainer


def main():
    a = parser(__doc__, "out/orpo").parse_args()
    model, tok, rows, kw = pick(a, "conversational_preference", per_device_train_batch_size=4, gradient_accumulation_steps=4,
                                learning_rate=8e-6, bf16=True, logging_steps=10, report_to="none")
    trainer = ORPOTrainer(model, ORPOConfig(output_dir=a.out, beta=0.1, **kw), train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
