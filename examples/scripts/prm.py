"""Process reward model: token classification at the end of every reasoning step
(JSON lines with "prompt", "completions": [step, ...], "labels": [bool, ...]).

    python examples/scripts/prm.py --model /path/to/model --data steps.jsonl --out out/prm
"""
from _common import parser, pick

from trl_b200.experimental.prm import PRMConfig, PRMTrainer


def main():
    a = parser(__doc__, "out/prm").parse_args()
    model, tok, rows, kw = pick(a, "standard_stepwise_supervision", per_device_train_batch_size=8, learning_rate=1e-5,
                                bf16=True, logging_steps=10, report_to="none")
    if a.smoke:
        from trl_b200.testing import make_tiny_model

        model = make_tiny_model("tiny-qwen2", num_labels=2)
    trainer = PRMTrainer(model, PRMConfig(output_dir=a.out, step_separator="\n", **kw), train_dataset=rows,
                         processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
