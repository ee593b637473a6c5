"""Online DPO (experimental): two samples per prompt from the current policy, ranked by a reward function."""
import argparse
import json

from trl_b200.experimental.online_dpo import OnlineDPOConfig, OnlineDPOTrainer


def brevity(completions, **kw):
    return [-len(c) / 100.0 for c in completions]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", required=True)
    ap.add_argument("--out", default="out/online_dpo")
    a = ap.parse_args()
    rows = [json.loads(line) for line in open(a.data)]
    cfg = OnlineDPOConfig(output_dir=a.out, per_device_train_batch_size=8, max_new_tokens=128, bf16=True, report_to="none")
    OnlineDPOTrainer(a.model, reward_funcs=brevity, args=cfg, train_dataset=rows).train()


if __name__ == "__main__":
    main()
