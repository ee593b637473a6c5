"""DPO of a vision-language model (LLaVA checkpoint layout) on image preference pairs.

Each JSON line: {"images": ["img.png"], "prompt": [{"role": "user", "content": "..."}],
                 "chosen": [{"role": "assistant", "content": "..."}], "rejected": [{"role": "assistant", "content": "..."}]}

    python examples/scripts/dpo_vlm.py --model /path/to/llava-checkpoint --data prefs.jsonl --out out/dpo_vlm
"""
from _common import load_rows, parser

from trl_b200 import DPOConfig, DPOTrainer, VisionLanguageModel, VisionProcessor


def smoke_setup():
    import numpy as np

    from trl_b200.models.vision import tiny_vlm_arch
    from trl_b200.testing import make_tiny_tokenizer

    proc = VisionProcessor(make_tiny_tokenizer(), image_size=28, image_seq_length=4)
    model = VisionLanguageModel(tiny_vlm_arch("tiny-qwen2", image_token_index=proc.image_token_id))
    rs, rows = np.random.RandomState(0), []
    for i in range(16):
        bright = i % 2
        img = (rs.rand(28, 28, 3) * 60 + (160 if bright else 10)).astype("uint8")
        good, bad = ("day", "night") if bright else ("night", "day")
        rows.append({"images": [img], "prompt": [{"role": "user", "content": "is it day or night"}],
                     "chosen": [{"role": "assistant", "content": good}], "rejected": [{"role": "assistant", "content": bad}]})
    return model, proc, rows


def main():
    a = parser(__doc__, "out/dpo_vlm").parse_args()
    if a.smoke:
        model, proc, rows = smoke_setup()
        kw = dict(use_cpu=True, max_steps=2, learning_rate=1e-3, per_device_train_batch_size=4)
    else:
        from trl_b200.scripts.utils import load_processing_class

        model = VisionLanguageModel.from_pretrained(a.model, dtype="bfloat16")
        proc, rows = load_processing_class(a.model), load_rows(a.data)  # image paths are opened by the processor
        kw = dict(bf16=True, learning_rate=5e-7, per_device_train_batch_size=2, gradient_accumulation_steps=8)
    cfg = DPOConfig(output_dir=a.out, beta=0.1, logging_steps=1, save_strategy="no", report_to="none", **kw)
    trainer = DPOTrainer(model, args=cfg, train_dataset=rows, processing_class=proc)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
