"""trl_b200: a Blackwell-native post-training framework with TRL's public surface
(exports of trl/__init__.py:28-73)."""
__version__ = "0.1.0.dev0"

_import_structure = {
    "chat_template_utils": ["add_response_schema", "clone_chat_template", "get_training_chat_template",
                            "supports_tool_calling", "parse_response", "is_chat_template_prefix_preserving"],
    "data_utils": ["apply_chat_template", "extract_prompt", "is_conversational", "is_conversational_from_value",
                   "maybe_apply_chat_template", "maybe_convert_to_chatml", "maybe_extract_prompt",
                   "maybe_unpair_preference_dataset", "pack_dataset", "prepare_multimodal_messages",
                   "prepare_multimodal_messages_vllm", "unpair_preference_dataset", "truncate_dataset"],
    "models.utils": ["create_reference_model", "unwrap_model_for_generation"],
    "models.decoder": ["CausalLM"],
    "models.hf_io": ["load_model"],
    "models.vision": ["VisionLanguageModel", "VlmArch", "VisionArch"],
    "models.vision_processing": ["VisionProcessor", "DynamicResolutionProcessor"],
    "models.vision_qwen": ["Qwen2VLModel", "Qwen2VLArch", "QwenVisionArch"],
    "models.configuration": ["ModelArch", "preset"],
    "models.lora": ["LoraConfig", "get_peft_model"],
    "scripts.utils": ["DatasetMixtureConfig", "ScriptArguments", "TrlParser", "get_dataset", "init_zero_verbose"],
    "trainer.callbacks": ["BEMACallback", "LogCompletionsCallback", "RichProgressCallback", "SyncRefModelCallback",
                          "WeaveCallback"],
    "trainer.dpo_config": ["DPOConfig"],
    "trainer.dpo_trainer": ["DPOTrainer"],
    "trainer.grpo_config": ["GRPOConfig", "RLOOConfig"],
    "trainer.grpo_trainer": ["GRPOTrainer"],
    "trainer.kto_trainer": ["KTOConfig", "KTOTrainer"],
    "trainer.model_config": ["ModelConfig"],
    "trainer.reward_trainer": ["RewardConfig", "RewardTrainer"],
    "trainer.rloo_trainer": ["RLOOTrainer"],
    "trainer.sft_config": ["SFTConfig"],
    "trainer.sft_trainer": ["SFTTrainer"],
    "trainer.utils": ["get_peft_config", "get_quantization_config"],
    "rollout.engine": ["RolloutEngine", "EagerGenerator"],
    "rollout.sampling": ["SamplingParams"],
    "loop.trainer": ["Trainer"],
    "loop.training_args": ["TrainingArguments"],
    "loop.state": ["TrainerCallback", "TrainerState", "TrainerControl"],
}

from . import _compat as _compat_mod  # noqa: E402
from ._lazy_module import lazy_exports  # noqa: E402

_compat_mod.apply()

__getattr__, __dir__, __all__ = lazy_exports(__name__, _import_structure, globals())
