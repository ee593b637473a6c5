"""BCO (experimental): unpaired feedback ({"prompt", "completion", "label": true | false}) trained as a binary
classifier of the implicit reward against a running mean.

    python examples/scripts/bco.py --model /path/to/model --data feedback.jsonl --out out/bco
"""
from _common import parser, pick

from trl_b200.experimental.bco import BCOConfig, BCOTrainer


def main():
    a = parser(__doc__, "out/bco").parse_args()
    model, tok, rows, kw = pick(a, "standard_unpaired_preference", per_device_train_batch_size=8, learning_rate=5e-7,
                                bf16=True, logging_steps=10, report_to="none")
    trainer = BCOTrainer(model, args=BCOConfig(output_dir=a.out, beta=0.1, **kw), train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
