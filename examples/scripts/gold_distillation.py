"""GOLD (experimental): on-policy distillation from a teacher that may use another tokenizer.  With
`--cross-tokenizer` the ULD loss aligns student and teacher tokens by the characters they cover and compares the
sorted probability vectors; otherwise the generalised Jensen-Shannon divergence on the shared vocabulary is used.

    python examples/scripts/gold_distillation.py --model /path/to/student --teacher /path/to/teacher \
        --data prompt_completion.jsonl --out out/gold [--cross-tokenizer]
"""
from _common import parser, pick

from trl_b200.experimental.gold import GOLDConfig, GOLDTrainer


def main():
    ap = parser(__doc__, "out/gold")
    ap.add_argument("--teacher", default=None, help="teacher checkpoint directory")
    ap.add_argument("--cross-tokenizer", action="store_true")
    a = ap.parse_args()
    model, tok, rows, kw = pick(a, "standard_prompt_completion", per_device_train_batch_size=4, learning_rate=1e-5,
                                bf16=True, logging_steps=10, report_to="none")
    if a.smoke:
        from trl_b200.testing import make_tiny_model

        teacher, teacher_tok = make_tiny_model("tiny-qwen2", seed=1), tok
    else:
        from trl_b200.scripts.utils import load_processing_class

        if not a.teacher:
            raise SystemExit("--teacher is required")
        teacher, teacher_tok = a.teacher, load_processing_class(a.teacher)
    cfg = GOLDConfig(output_dir=a.out, lmbda=0.5, beta=0.5, use_uld_loss=a.cross_tokenizer or a.smoke,
                     uld_use_hybrid_loss=True, max_new_tokens=8 if a.smoke else 128, **kw)
    trainer = GOLDTrainer(model, teacher, cfg, teacher_processing_class=teacher_tok, train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
