"""XPO and Nash-MD (experimental): online preference optimisation with two completions per prompt, one from the
policy and one from the reference (XPO) or from a geometric mixture of policy and reference (Nash-MD), ranked by a
reward function.

    python examples/scripts/xpo_nash_md.py --algo xpo --model /path/to/model --data prompts.jsonl --out out/xpo
"""
from _common import parser, pick


def concise(completions, **kw):
    return [-len(c if isinstance(c, str) else c[-1]["content"]) / 100.0 for c in completions]


def main():
    ap = parser(__doc__, "out/xpo")
    ap.add_argument("--algo", choices=["xpo", "nash_md"], default="xpo")
    a = ap.parse_args()
    if a.algo == "xpo":
        from trl_b200.experimental.xpo import XPOConfig as Config, XPOTrainer as Trainer
        extra = dict(alpha=[1e-5])
    else:
        from trl_b200.experimental.nash_md import NashMDConfig as Config, NashMDTrainer as Trainer
        extra = dict(mixture_coef=0.5)
    model, tok, rows, kw = pick(a, "standard_prompt_only", per_device_train_batch_size=8, learning_rate=5e-7, bf16=True,
                                logging_steps=1, report_to="none")
    kw["max_new_tokens"] = 8 if a.smoke else 128
    trainer = Trainer(model, reward_funcs=concise, args=Config(output_dir=a.out, **kw, **extra), train_dataset=rows,
                      processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
