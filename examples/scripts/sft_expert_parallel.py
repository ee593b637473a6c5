"""Supervised fine-tuning of a mixture-of-experts model with expert parallelism: every rank keeps
`num_experts / world` experts of every layer, tokens travel to their experts and back inside the MoE block.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/scripts/sft_expert_parallel.py \
        --model /path/to/qwen3-moe --data train.jsonl --out out/sft_ep

`--smoke` runs a tiny random Qwen3-MoE on CPU in one process (ep_size 1: the same code path without the exchange).
"""
from _common import parser, pick

from trl_b200 import SFTConfig, SFTTrainer


def main():
    a = parser(__doc__, "out/sft_ep").parse_args()
    model, tok, rows, kw = pick(a, "standard_language_modeling", per_device_train_batch_size=2, gradient_accumulation_steps=8,
                                learning_rate=1e-5, bf16=True, logging_steps=10, report_to="none")
    if a.smoke:
        from trl_b200.testing import make_tiny_model

        model = make_tiny_model("tiny-qwen3-moe")
        ep = 1
    else:
        import os

        ep = int(os.environ.get("WORLD_SIZE", "1"))
    cfg = SFTConfig(output_dir=a.out, ep_size=ep, packing=not a.smoke, max_length=64 if a.smoke else 4096, **kw)
    trainer = SFTTrainer(model, cfg, train_dataset=rows, processing_class=tok)
    trainer.train()
    trainer.save_model(a.out)  # the experts of all ranks are gathered into one checkpoint


if __name__ == "__main__":
    main()
