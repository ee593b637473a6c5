"""Reference-free preference optimisation: CPO, or SimPO / AlphaPO through `--loss simpo`.

    python examples/scripts/cpo_simpo.py --model /path/to/model --data prefs.jsonl --out out/cpo --loss simpo
"""
from _common import parser, pick

from trl_b200.experimental.cpo import CPOConfig, CPOTrainer


def main():
    ap = parser(__doc__, "out/cpo")
    ap.add_argument("--loss", default="sigmoid", help="sigmoid | hinge | ipo | simpo | alphapo")
    a = ap.parse_args()
    model, tok, rows, kw = pick(a, "standard_preference", per_device_train_batch_size=4, gradient_accumulation_steps=4,
                                learning_rate=5e-7, bf16=True, logging_steps=10, report_to="none")
    extra = dict(cpo_alpha=0.0, simpo_gamma=0.5) if a.loss in ("simpo", "alphapo") else {}
    cfg = CPOConfig(output_dir=a.out, loss_type=a.loss, beta=0.1 if a.loss == "sigmoid" else 2.0, **extra, **kw)
    trainer = CPOTrainer(model, cfg, train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
