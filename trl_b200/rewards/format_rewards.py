"""Format rewards (trl/rewards/format_rewards.py)."""
import re

_THINK = re.compile(r"^<think>(?!.*<think>)(.*?)</think>.*$", re.DOTALL | re.MULTILINE)


def think_format_reward(completions: list, **kwargs) -> list[float]:
    """1.0 when the completion starts with exactly one ``<think>...</think>`` block, else 0.0."""
    return [1.0 if _THINK.match(c[0]["content"] if isinstance(c, list) else c) else 0.0 for c in completions]
