"""Writes tiny random checkpoints of every native model family (HF safetensors layout + tokenizer) for offline tests and
CI, the role of scripts/generate_tiny_models/ in the reference (there: hub uploads such as tiny-Qwen2ForCausalLM-2.5 with
hidden 8, 2 layers).

    python examples/scripts/generate_tiny_models.py --out tiny_models [--families tiny-qwen2 tiny-llama ...]

Each directory loads with `trl_b200.load_model(path)` and with `transformers.AutoModelForCausalLM.from_pretrained(path)`.
"""
import argparse
import os


def main():
    from trl_b200.models.configuration import PRESETS, preset
    from trl_b200.models.decoder import CausalLM
    from trl_b200.models.vision import VisionLanguageModel, tiny_vlm_arch
    from trl_b200.models.vision_processing import VisionProcessor
    from trl_b200.testing import make_tiny_tokenizer

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default="tiny_models")
    ap.add_argument("--families", nargs="*", default=sorted(k for k in PRESETS if k.startswith("tiny-")))
    ap.add_argument("--reward-heads", action="store_true", help="also write <family>-reward with a one-label score head")
    ap.add_argument("--no-vlm", action="store_true")
    a = ap.parse_args()
    import torch

    for name in a.families:
        torch.manual_seed(0)
        tok = make_tiny_tokenizer()
        path = os.path.join(a.out, name)
        CausalLM(preset(name, eos_token_id=tok.eos_token_id, pad_token_id=tok.pad_token_id)).save_pretrained(path)
        tok.save_pretrained(path)
        print("wrote", path)
        if a.reward_heads:
            CausalLM(preset(name, num_labels=1, pad_token_id=tok.pad_token_id)).save_pretrained(path + "-reward")
            tok.save_pretrained(path + "-reward")
            print("wrote", path + "-reward")
    if not a.no_vlm:
        tok = make_tiny_tokenizer()
        proc = VisionProcessor(tok, image_size=28, image_seq_length=4)
        path = os.path.join(a.out, "tiny-llava")
        VisionLanguageModel(tiny_vlm_arch("tiny-llama", image_token_index=proc.image_token_id)).save_pretrained(path)
        proc.save_pretrained(path)
        print("wrote", path)
        from trl_b200.models.vision_processing import DynamicResolutionProcessor
        from trl_b200.models.vision_qwen import Qwen2VLModel, tiny_qwen2_vl_arch

        tok = make_tiny_tokenizer()
        proc = DynamicResolutionProcessor(tok, min_pixels=28 * 28, max_pixels=112 * 112)
        arch = tiny_qwen2_vl_arch()
        arch.image_token_id = proc.image_token_id
        arch.text.vocab_size = max(arch.text.vocab_size, len(tok))
        path = os.path.join(a.out, "tiny-qwen2-vl")
        Qwen2VLModel(arch).save_pretrained(path)
        proc.save_pretrained(path)
        print("wrote", path)


if __name__ == "__main__":
    main()
