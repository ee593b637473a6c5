"""PPO with a value head (experimental): rollouts from the policy, a reward function on the completions, GAE
advantages, clipped policy and value losses.

    python examples/scripts/ppo.py --model /path/to/model --data prompts.jsonl --out out/ppo

Each JSON line: {"prompt": "..."} (or a list of chat messages).  `--smoke` runs a tiny random model on CPU.
"""
from _common import parser, pick

from trl_b200.experimental.ppo import PPOConfig, PPOTrainer


def brevity_and_closure(completions, completion_ids, **kw):
    """Short answers that end with a full stop score higher."""
    def text(c):
        return c if isinstance(c, str) else c[-1]["content"]
    return [(1.0 if text(c).rstrip().endswith(".") else 0.0) - len(ids) / 200.0 for c, ids in zip(completions, completion_ids)]


def main():
    a = parser(__doc__, "out/ppo").parse_args()
    model, tok, rows, kw = pick(a, "standard_prompt_only", per_device_train_batch_size=8, learning_rate=3e-6, bf16=True,
                                logging_steps=1, report_to="none")
    if a.smoke:
        kw.update(max_steps=4, response_length=6, num_mini_batches=2, num_ppo_epochs=2)
    else:
        from trl_b200.scripts.utils import load_processing_class

        tok = load_processing_class(a.model)
        kw.update(response_length=128, num_mini_batches=2, num_ppo_epochs=4, total_episodes=4096)
    cfg = PPOConfig(output_dir=a.out, kl_coef=0.05, missing_eos_penalty=1.0, **kw)
    trainer = PPOTrainer(cfg, tok, model, reward_funcs=brevity_and_closure, train_dataset=rows)
    trainer.train()
    trainer.save_model(a.out)  # the policy; the value head is stored next to it


if __name__ == "__main__":
    main()
