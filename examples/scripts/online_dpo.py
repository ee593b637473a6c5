"""Online DPO (experimental): two samples per prompt from the current policy, ranked by a reward function (or a
pairwise judge); the better one becomes "chosen" and the DPO loss is taken against the frozen reference.

    python examples/scripts/online_dpo.py --model /path/to/model --data prompts.jsonl --out out/online_dpo
"""
from _common import parser, pick

from trl_b200.experimental.online_dpo import OnlineDPOConfig, OnlineDPOTrainer


def brevity(completions, **kw):
    return [-len(c if isinstance(c, str) else c[-1]["content"]) / 100.0 for c in completions]


def main():
    a = parser(__doc__, "out/online_dpo").parse_args()
    model, tok, rows, kw = pick(a, "standard_prompt_only", per_device_train_batch_size=8, learning_rate=5e-7, bf16=True,
                                logging_steps=1, report_to="none")
    cfg = OnlineDPOConfig(output_dir=a.out, max_new_tokens=8 if a.smoke else 128, missing_eos_penalty=1.0, **kw)
    trainer = OnlineDPOTrainer(model, reward_funcs=brevity, args=cfg, train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
