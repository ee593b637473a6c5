"""``trl grpo`` training script: parse (ScriptArguments, GRPOConfig, ModelConfig, DatasetMixtureConfig),
load the tokenizer and dataset from local paths, train, save.  Skeleton of trl/scripts/grpo.py."""
from __future__ import annotations

import dataclasses
import os
from typing import Optional

from trl_b200.scripts.utils import ScriptArguments


@dataclasses.dataclass
class GRPOScriptArguments(ScriptArguments):
    reward_model_name_or_path: Optional[str] = None
    reward_funcs: Optional[list] = None


def main(script_args, training_args, model_args, dataset_args):
    from trl_b200 import GRPOTrainer, get_peft_config, get_quantization_config
    from trl_b200.scripts.utils import load_processing_class, load_script_dataset

    get_quantization_config(model_args)
    training_args.model_init_kwargs = dict(dtype=model_args.dtype)
    # tokenizer, or a processor for vision-language checkpoints; presets get the offline ChatML fixture
    tokenizer = load_processing_class(model_args.model_name_or_path)
    dataset = load_script_dataset(script_args, dataset_args)
    eval_ds = dataset[script_args.dataset_test_split] if (
        training_args.eval_strategy != "no" and script_args.dataset_test_split in dataset) else None
    from trl_b200.scripts.grpo import resolve_reward_funcs

    reward_funcs = resolve_reward_funcs(script_args)
    trainer = GRPOTrainer(model=model_args.model_name_or_path, reward_funcs=reward_funcs, args=training_args,
                  train_dataset=dataset[script_args.dataset_train_split], eval_dataset=eval_ds,
                  processing_class=tokenizer, peft_config=get_peft_config(model_args))
    trainer.train()
    trainer.save_model(training_args.output_dir)
    if training_args.push_to_hub:
        trainer.push_to_hub(dataset_name=script_args.dataset_name)


reward_funcs_registry = None


def resolve_reward_funcs(script_args):
    """Names from the built-in registry, dotted import paths (``pkg.mod.func``), and/or a reward model path."""
    import importlib

    from trl_b200 import rewards as R

    registry = {
        "accuracy_reward": R.accuracy_reward,
        "reasoning_accuracy_reward": R.reasoning_accuracy_reward,
        "think_format_reward": R.think_format_reward,
        "get_cosine_scaled_reward": R.get_cosine_scaled_reward(),
        "get_repetition_penalty_reward": R.get_repetition_penalty_reward(ngram_size=3, max_penalty=-1.0),
        "get_soft_overlong_punishment": R.get_soft_overlong_punishment(max_completion_len=1280, soft_punish_cache=256),
    }
    funcs = []
    if getattr(script_args, "reward_model_name_or_path", None):
        funcs.append(script_args.reward_model_name_or_path)
    for name in getattr(script_args, "reward_funcs", None) or []:
        if name in registry:
            funcs.append(registry[name])
        elif "." in name:
            mod, fn = name.rsplit(".", 1)
            funcs.append(getattr(importlib.import_module(mod), fn))
        else:
            raise ValueError(f"Could not load reward function '{name}'. Expected one of {list(registry)} or a dotted path.")
    if not funcs:
        raise ValueError("provide --reward_funcs and/or --reward_model_name_or_path")
    return funcs


def make_parser(subparsers=None):
    from trl_b200 import DatasetMixtureConfig, ModelConfig, TrlParser, GRPOConfig
    from trl_b200.scripts.utils import ScriptArguments

    dataclass_types = (GRPOScriptArguments, GRPOConfig, ModelConfig, DatasetMixtureConfig)
    if subparsers is not None:
        return subparsers.add_parser("grpo", help="Run the GRPO training script", dataclass_types=dataclass_types)
    return TrlParser(dataclass_types)


if __name__ == "__main__":
    parser = make_parser()
    script_args, training_args, model_args, dataset_args = parser.parse_args_and_config(fail_with_unknown_args=False)[:4]
    main(script_args, training_args, model_args, dataset_args)
