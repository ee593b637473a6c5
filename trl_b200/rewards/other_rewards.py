"""Length / repetition shaping rewards (trl/rewards/other_rewards.py).  The factories return picklable
callable objects with a ``__name__`` so they survive being sent to a spawned rollout worker."""
from __future__ import annotations


class _RepetitionPenalty:
    __name__ = "repetition_penalty_reward"

    def __init__(self, ngram_size: int, max_penalty: float):
        self.ngram_size, self.max_penalty = ngram_size, max_penalty

    def __call__(self, completion_ids: list[list[int]], **kwargs) -> list[float]:
        out = []
        n = self.ngram_size
        for ids in completion_ids:
            total = len(ids) - n + 1
            if total <= 0:
                out.append(0.0)
                continue
            uniq = len({tuple(ids[i:i + n]) for i in range(total)})
            frac = 1.0 - uniq / total
            out.append(frac * self.max_penalty if frac else 0.0)
        return out


def get_repetition_penalty_reward(ngram_size: int = 3, max_penalty: float = -1.0):
    """(1 - unique n-grams / total n-grams) * max_penalty over the completion token ids."""
    if max_penalty > 0:
        raise ValueError(f"max_penalty {max_penalty} should not be positive")
    return _RepetitionPenalty(ngram_size, max_penalty)


class _SoftOverlongPunishment:
    __name__ = "soft_overlong_punishment_reward"

    def __init__(self, max_completion_len: int, soft_punish_cache: int):
        self.max_completion_len, self.soft_punish_cache = max_completion_len, soft_punish_cache

    def __call__(self, completion_ids: list[list[int]], **kwargs) -> list[float]:
        lo = self.max_completion_len - self.soft_punish_cache
        out = []
        for ids in completion_ids:
            L = len(ids)
            if L <= lo:
                out.append(0.0)
            elif L <= self.max_completion_len:
                out.append((lo - L) / self.soft_punish_cache)
            else:
                out.append(-1.0)
        return out


def get_soft_overlong_punishment(max_completion_len: int, soft_punish_cache: int):
    """DAPO eq. 13: 0 up to L_max - L_cache, linear down to -1 at L_max, -1 beyond."""
    return _SoftOverlongPunishment(max_completion_len, soft_punish_cache)
