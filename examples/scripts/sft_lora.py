"""Supervised fine-tuning of LoRA adapters; the output directory holds adapter_model.safetensors + adapter_config.json.

    python examples/scripts/sft_lora.py --model /path/to/model --data train.jsonl --out out/sft_lora
"""
from _common import parser, pick

from trl_b200 import LoraConfig, SFTConfig, SFTTrainer


def main():
    a = parser(__doc__, "out/sft_lora").parse_args()
    model, tok, rows, kw = pick(a, "conversational_language_modeling", per_device_train_batch_size=4,
                                gradient_accumulation_steps=4, learning_rate=1e-4, bf16=True, logging_steps=10,
                                report_to="none")
    lora = LoraConfig(r=16, lora_alpha=32, lora_dropout=0.0, target_modules=["q_proj", "k_proj", "v_proj", "o_proj",
                                                                              "gate_proj", "up_proj", "down_proj"])
    trainer = SFTTrainer(model, SFTConfig(output_dir=a.out, assistant_only_loss=False, **kw), train_dataset=rows,
                         processing_class=tok, peft_config=lora)
    trainer.train()
    trainer.save_model(a.out)


if __name__ == "__main__":
    main()
