"""``trl reward`` training script: parse (ScriptArguments, RewardConfig, ModelConfig, DatasetMixtureConfig),
load the tokenizer and dataset from local paths, train, save.  Skeleton of trl/scripts/reward.py."""
from __future__ import annotations

import os


def main(script_args, training_args, model_args, dataset_args):
    from trl_b200 import RewardTrainer, get_peft_config, get_quantization_config
    from trl_b200.scripts.utils import load_processing_class, load_script_dataset

    get_quantization_config(model_args)
    training_args.model_init_kwargs = dict(dtype=model_args.dtype)
    # tokenizer, or a processor for vision-language checkpoints; presets get the offline ChatML fixture
    tokenizer = load_processing_class(model_args.model_name_or_path)
    dataset = load_script_dataset(script_args, dataset_args)
    eval_ds = dataset[script_args.dataset_test_split] if (
        training_args.eval_strategy != "no" and script_args.dataset_test_split in dataset) else None
    trainer = RewardTrainer(model=model_args.model_name_or_path, args=training_args,
                            train_dataset=dataset[script_args.dataset_train_split], eval_dataset=eval_ds,
                            processing_class=tokenizer, peft_config=get_peft_config(model_args))
    trainer.train()
    trainer.save_model(training_args.output_dir)
    if training_args.push_to_hub:
        trainer.push_to_hub(dataset_name=script_args.dataset_name)


def make_parser(subparsers=None):
    from trl_b200 import DatasetMixtureConfig, ModelConfig, TrlParser, RewardConfig
    from trl_b200.scripts.utils import ScriptArguments

    dataclass_types = (ScriptArguments, RewardConfig, ModelConfig, DatasetMixtureConfig)
    if subparsers is not None:
        return subparsers.add_parser("reward", help="Run the REWARD training script", dataclass_types=dataclass_types)
    return TrlParser(dataclass_types)


if __name__ == "__main__":
    parser = make_parser()
    script_args, training_args, model_args, dataset_args = parser.parse_args_and_config(fail_with_unknown_args=False)[:4]
    main(script_args, training_args, model_args, dataset_args)
