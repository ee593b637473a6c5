"""Supervised fine-tuning of a vision-language model (LLaVA or Qwen2-VL checkpoint layout) on image conversations.

Each JSON line: {"images": ["path/to/img.png", ...], "messages": [{"role": "user", "content": "..."}, ...]}

    python examples/scripts/sft_vlm.py --model /path/to/llava-checkpoint --data train.jsonl --out out/sft_vlm

Without --model a tiny random model and synthetic images are used (a smoke run on CPU); --family qwen2_vl picks the
dynamic-resolution model (images keep their size, multimodal RoPE) instead of the LLaVA composition.
"""
import argparse
import json


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None)
    ap.add_argument("--data", default=None)
    ap.add_argument("--out", default="out/sft_vlm")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--family", choices=["llava", "qwen2_vl"], default="llava", help="tiny model of the smoke run")
    a = ap.parse_args()

    from trl_b200 import SFTConfig, SFTTrainer, VisionLanguageModel, VisionProcessor

    if a.model:
        from PIL import Image

        from trl_b200.scripts.utils import load_processing_class

        from trl_b200 import load_model

        model = load_model(a.model, dtype="bfloat16")  # llava or qwen2_vl, by the checkpoint's model_type
        processor = load_processing_class(a.model)
        rows = []
        for line in open(a.data):
            r = json.loads(line)
            r["images"] = [Image.open(p).convert("RGB") for p in r.get("images", [])]
            rows.append(r)
        cpu = False
    else:
        import numpy as np

        from trl_b200.models.vision import tiny_vlm_arch
        from trl_b200.testing import make_tiny_tokenizer

        tok = make_tiny_tokenizer()
        if a.family == "qwen2_vl":
            from trl_b200 import DynamicResolutionProcessor, Qwen2VLModel
            from trl_b200.models.vision_qwen import tiny_qwen2_vl_arch

            processor = DynamicResolutionProcessor(tok, min_pixels=28 * 28, max_pixels=56 * 56)
            arch = tiny_qwen2_vl_arch()
            arch.image_token_id = processor.image_token_id
            arch.text.vocab_size = max(arch.text.vocab_size, len(tok))
            model = Qwen2VLModel(arch)
        else:
            processor = VisionProcessor(tok, image_size=28, image_seq_length=4)
            model = VisionLanguageModel(tiny_vlm_arch("tiny-qwen2", image_token_index=processor.image_token_id))
        rs = np.random.RandomState(0)
        rows = []
        for i in range(32):
            bright = i % 2
            img = (rs.rand(28, 28 * (1 + (i // 2) % 2), 3) * 60 + (160 if bright else 10)).astype("uint8")
            rows.append({"images": [img], "messages": [{"role": "user", "content": "is it day or night"},
                                                       {"role": "assistant", "content": "day" if bright else "night"}]})
        cpu = True
    cfg = SFTConfig(output_dir=a.out, per_device_train_batch_size=4, learning_rate=2e-5 if a.model else 3e-3,
                    max_steps=a.steps, logging_steps=1, save_strategy="no", report_to="none", use_cpu=cpu, bf16=not cpu,
                    max_length=None)
    trainer = SFTTrainer(model, cfg, train_dataset=rows, processing_class=processor)
    trainer.train()
    trainer.save_model(a.out)  # model.safetensors + config.json (llava layout) + tokenizer / preprocessor files


if __name__ == "__main__":
    main()
