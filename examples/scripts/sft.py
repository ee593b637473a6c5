"""Supervised fine-tuning on a local dataset (JSON lines with a "messages" or "text" column).

    python examples/scripts/sft.py --model /path/to/qwen2.5-0.5b --data train.jsonl --out out/sft
    python -m trl_b200.cli.main sft --model_name_or_path ... --dataset_name train.jsonl --output_dir out/sft \
        --num_processes 8 --accelerate_config zero2
"""
import argparse
import json

from trl_b200 import SFTConfig, SFTTrainer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", required=True)
    ap.add_argument("--out", default="out/sft")
    ap.add_argument("--packing", action="store_true")
    a = ap.parse_args()
    rows = [json.loads(line) for line in open(a.data)]
    cfg = SFTConfig(output_dir=a.out, per_device_train_batch_size=4, gradient_accumulation_steps=4, learning_rate=2e-5,
                    num_train_epochs=1, bf16=True, packing=a.packing, max_length=2048, logging_steps=10, save_strategy="epoch",
                    report_to="none")
    trainer = SFTTrainer(a.model, cfg, train_dataset=rows)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
