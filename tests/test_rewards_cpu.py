"""Reward functions against the literal cases of the reference's tests (tests/test_rewards.py)."""
import pickle

import pytest

from trl_b200.rewards import (get_cosine_scaled_reward, get_repetition_penalty_reward, get_soft_overlong_punishment,
                              think_format_reward)


def _chat(texts):
    return [[{"content": t}] for t in texts]


def test_think_format_valid_invalid_and_mixed():
    valid = ["<think>This is my reasoning.</think>This is my answer.",
             "<think>\nThis is my reasoning.\n</think>\nThis is my answer.",
             "<think>\nThis is\nmy reasoning.\n</think>\nThis is my answer.",
             "<think>\nThis is <some tag> my reasoning.</think>\nThis is my answer.",
             "<think></think>\nThis is my answer."]
    assert think_format_reward(_chat(valid)) == [1.0] * 5
    invalid = ["<think>\nThis is my reasoning.\nThis is my answer.", "<think>This is my reasoning.\nThis is my answer.",
               "This is my reasoning. This is my answer.", "This is my reasoning.\nThis is my answer.",
               "This is my reasoning.</think>\nThis is my answer.", "This is my reasoning.</think>This is my answer.",
               "This<think>is my reasoning.</think>\nThis is my answer.",
               "<think>This is<think>my reasoning.</think></think>This is my answer.",
               "<think>This is</think>\nmy\n<think>reasoning.</think>\nThis is my answer."]
    assert think_format_reward(_chat(invalid)) == [0.0] * 9
    assert think_format_reward(_chat([valid[0], valid[1], invalid[1], invalid[2]])) == [1.0, 1.0, 0.0, 0.0]


def test_soft_overlong_punishment():
    fn = get_soft_overlong_punishment(max_completion_len=100, soft_punish_cache=20)
    assert fn(completion_ids=[[1] * 50]) == [0]          # up to 80 tokens: no penalty
    assert fn([[1] * 110]) == [-1]                       # past the limit
    assert fn([[1] * 90])[0] == pytest.approx(-0.5)      # half way through the soft zone


def test_repetition_penalty_reward():
    fn = get_repetition_penalty_reward(ngram_size=2, max_penalty=-1.0)
    assert fn([[1, 2, 3, 4]]) == [0.0]
    assert fn([[5, 5, 5, 5, 5]]) == [pytest.approx(-0.75)]          # 4 bigrams, 1 distinct
    assert fn([[1, 2, 1, 2, 1, 2]]) == [pytest.approx(-0.6)]        # 5 bigrams, 2 distinct
    assert fn([[1, 2, 3, 4], [5, 5, 5, 5, 5], [9]]) == [pytest.approx(0.0), pytest.approx(-0.75), pytest.approx(0.0)]
    assert fn([[5, 5, 5, 5, 5]], prompts=["x"], completions=_chat(["5 5 5 5 5"])) == [pytest.approx(-0.75)]
    tri = get_repetition_penalty_reward(ngram_size=3, max_penalty=-1.0)
    assert tri([[1, 2]]) == [0.0] and tri([[1, 2, 3]]) == [0.0] and tri([[]]) == [0.0]
    assert fn([[1, 2, 3, 1, 2, 3]]) == [pytest.approx(-0.4)] and tri([[1, 2, 3, 1, 2, 3]]) == [pytest.approx(-0.25)]
    assert get_repetition_penalty_reward(ngram_size=2, max_penalty=-0.5)([[5, 5, 5, 5, 5]]) == [pytest.approx(-0.375)]
    with pytest.raises(ValueError):
        get_repetition_penalty_reward(ngram_size=2, max_penalty=0.5)
    again = pickle.loads(pickle.dumps(fn))                          # crosses to the rollout worker process
    assert again([[5, 5, 5, 5, 5]]) == [pytest.approx(-0.75)] and again.__name__ == "repetition_penalty_reward"


def test_accuracy_reward_cases():
    import threading

    from trl_b200.rewards import accuracy_reward

    boxed = [[{"content": r"\boxed{\frac{63}{400}}"}]] * 2
    assert accuracy_reward(boxed, [r"\frac{63}{400}", "63/400"]) == [1.0, 1.0]
    assert accuracy_reward([[{"content": r"\boxed{\frac{64}{400}}"}]], [r"\frac{63}{400}"]) == [0.0]
    assert accuracy_reward([[{"content": r"\boxed{3}"}]], ["6"]) == [0.0]
    # a gold solution that does not parse: the sample is skipped (None), whatever the completion says
    got = accuracy_reward([[{"content": "Answer is forty two."}], [{"content": r"Some other content. \boxed{43}."}]],
                          ["Answer is forty two.", "Answer is forty three."])
    assert got == [None, None]
    out, err = [], []

    def target():
        try:
            out.extend(accuracy_reward([[{"content": r"\boxed{\frac{1}{3}}"}]], [r"\frac{1}{3}"]))
        except Exception as e:  # noqa: BLE001
            err.append(e)
    t = threading.Thread(target=target)
    t.start()
    t.join()
    assert not err and out == [1.0]


def test_reasoning_accuracy_reward_cases():
    from trl_b200.rewards import reasoning_accuracy_reward

    sol = r"\frac{63}{400}"
    assert reasoning_accuracy_reward([[{"content": r"<think> Reasoning content </think> \boxed{\frac{63}{400}}"}],
                                      [{"content": r"Reasoning content </think> \boxed{\frac{63}{400}}"}]], [sol, sol]) == [1.0, 1.0]
    assert reasoning_accuracy_reward([[{"content": r"<REASONING_START> Reasoning content </REASONING_END> \boxed{\frac{63}{400}}"}]],
                                     [sol], reasoning_delimiters=["</REASONING_END>"]) == [1.0]
    assert reasoning_accuracy_reward([[{"content": r"<think> Reasoning content </think> \boxed{\frac{64}{400}}"}]], [sol]) == [0.0]
    # the answer inside the reasoning does not count; an unfinished reasoning block scores zero
    assert reasoning_accuracy_reward([[{"content": r"<think> My answer is \boxed{42} </think> Some other text."}],
                                      [{"content": r"<think> The answer is \boxed{42} </think> Here's a wrong answer: \boxed{43}."}]],
                                     [r"\boxed{42}", r"\boxed{42}"]) == [0.0, 0.0]
    assert reasoning_accuracy_reward([[{"content": r"<think> Incomplete reasoning without closing tag"}],
                                      [{"content": r"Correct answer \frac{63}{400} but completely missing reasoning content"}]],
                                     [sol, sol]) == [0.0, 0.0]
    assert reasoning_accuracy_reward([[{"content": r"<think> Reasoning content </think> \boxed{42}"}]], ["forty two"]) == [None]


def test_cosine_scaled_reward_cases():
    third, half = [{"content": r"\boxed{\frac{1}{3}}"}], [{"content": r"\boxed{\frac{1}{2}}"}]
    gold = [r"\frac{1}{3}"] * 2
    fn = get_cosine_scaled_reward(max_len=100)
    assert fn([third, third], gold, [[1] * 25, [1] * 75]) == [pytest.approx(0.92678, abs=1e-4), pytest.approx(0.57322, abs=1e-4)]
    assert fn([half, half], gold, [[1] * 25, [1] * 75]) == [pytest.approx(-0.92678, abs=1e-4), pytest.approx(-0.57322, abs=1e-4)]
    assert fn([third, half], gold, [[1] * 50, [1] * 50]) == [pytest.approx(0.75), pytest.approx(-0.75)]
    assert fn([third, third], gold, [[], [1] * 100]) == [pytest.approx(1.0), pytest.approx(0.5)]
    assert fn([half, half], gold, [[], [1] * 100]) == [pytest.approx(-1.0), pytest.approx(-0.5)]
    assert fn([third, half], gold, [[1] * 200, [1] * 200]) == [pytest.approx(0.5), pytest.approx(-0.5)]   # clamped past max_len
    assert fn([[{"content": r"\boxed{42}"}]], ["forty two"], [[1] * 50]) == [None]
    wide = get_cosine_scaled_reward(max_len=100, min_value_correct=0.0, max_value_correct=2.0)
    assert wide([third], gold[:1], [[1] * 50]) == [pytest.approx(1.0)]
    again = pickle.loads(pickle.dumps(fn))
    assert again([third], gold[:1], [[1] * 50]) == [pytest.approx(0.75)] and again.__name__ == "cosine_scaled_reward"
