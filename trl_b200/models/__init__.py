from .activation_offloading import get_act_offloading_ctx_manager
from .configuration import PRESETS, ModelArch, preset
from .decoder import CausalLM, SeqCtx
from .hf_io import load_model
from .lora import LoraConfig, get_peft_model
from .vision import VisionArch, VisionLanguageModel, VlmArch
from .vision_processing import DynamicResolutionProcessor, VisionProcessor
from .vision_qwen import Qwen2VLArch, Qwen2VLModel, QwenVisionArch
from .utils import (create_reference_model, disable_gradient_checkpointing, prepare_deepspeed, prepare_fsdp,
                    unwrap_model_for_generation)

__all__ = ["CausalLM", "SeqCtx", "ModelArch", "preset", "PRESETS", "load_model", "LoraConfig", "get_peft_model",
           "get_act_offloading_ctx_manager", "prepare_deepspeed", "prepare_fsdp", "unwrap_model_for_generation",
           "create_reference_model", "disable_gradient_checkpointing", "VisionLanguageModel", "VlmArch", "VisionArch",
           "VisionProcessor"]
