"""Bradley-Terry reward model on preference pairs (JSON lines with "chosen", "rejected" and optionally "prompt").

    python examples/scripts/reward_modeling.py --model /path/to/model --data prefs.jsonl --out out/rm
The checkpoint gets a one-label score head; `center_rewards_coefficient` keeps the scores centred.
"""
from _common import parser, pick

from trl_b200 import RewardConfig, RewardTrainer


def main():
    a = parser(__doc__, "out/rm").parse_args()
    model, tok, rows, kw = pick(a, "standard_preference", per_device_train_batch_size=8, learning_rate=1e-5, bf16=True,
                                logging_steps=10, report_to="none")
    if a.smoke:
        from trl_b200.testing import make_tiny_model

        model = make_tiny_model("tiny-qwen2", num_labels=1)
    cfg = RewardConfig(output_dir=a.out, center_rewards_coefficient=0.01, max_length=1024, **kw)
    trainer = RewardTrainer(model, args=cfg, train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
