"""DPO on a local preference dataset (JSON lines with "prompt", "chosen", "rejected").

    python examples/scripts/dpo.py --model /path/to/model --data prefs.jsonl --out out/dpo --loss sigmoid
"""
import argparse
import json

from trl_b200 import DPOConfig, DPOTrainer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", required=True)
    ap.add_argument("--out", default="out/dpo")
    ap.add_argument("--loss", default="sigmoid")
    ap.add_argument("--beta", type=float, default=0.1)
    a = ap.parse_args()
    rows = [json.loads(line) for line in open(a.data)]
    cfg = DPOConfig(output_dir=a.out, per_device_train_batch_size=2, gradient_accumulation_steps=8, learning_rate=5e-7,
                    beta=a.beta, loss_type=a.loss, bf16=True, max_length=1024, logging_steps=10, report_to="none")
    trainer = DPOTrainer(a.model, args=cfg, train_dataset=rows)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
