"""Collators against literal expected batches (the vectors of the reference's collator unit tests:
tests/test_sft_trainer.py:97-262, tests/test_dpo_trainer.py:44-135, tests/test_reward_trainer.py:34-120,
tests/test_kto_trainer.py:146-230)."""
import torch

from trl_b200.trainer.sft_trainer import DataCollatorForLanguageModeling

T = torch.tensor


def _eq(result, **want):
    assert set(result.keys()) == set(want), (set(result.keys()), set(want))
    for k, v in want.items():
        assert torch.equal(result[k], T(v)), (k, result[k], v)


def test_language_modeling_padded_batches():
    ex = [{"input_ids": [1, 2, 3], "labels": [1, 2, 3]}, {"input_ids": [4, 5], "labels": [4, 5]}]
    c = DataCollatorForLanguageModeling(pad_token_id=0)
    want = dict(input_ids=[[1, 2, 3], [4, 5, 0]], attention_mask=[[1, 1, 1], [1, 1, 0]], labels=[[1, 2, 3], [4, 5, -100]])
    _eq(c(ex), **want)
    _eq(c([{"input_ids": [1, 2, 3]}, {"input_ids": [4, 5]}]), **want)  # labels default to the ids, padding masked
    # provided labels are used as they are: mask columns next to them change nothing
    _eq(c([{**ex[0], "completion_mask": [0, 0, 1], "assistant_masks": [0, 0, 1]},
           {**ex[1], "completion_mask": [0, 1], "assistant_masks": [0, 1]}]), **want)
    # seq_lengths without padding_free is ignored
    _eq(c([{**ex[0], "seq_lengths": [1, 2]}, {**ex[1], "seq_lengths": [2]}]), **want)
    _eq(DataCollatorForLanguageModeling(pad_token_id=0, pad_to_multiple_of=4)(ex),
        input_ids=[[1, 2, 3, 0], [4, 5, 0, 0]], attention_mask=[[1, 1, 1, 0], [1, 1, 0, 0]],
        labels=[[1, 2, 3, -100], [4, 5, -100, -100]])
    _eq(DataCollatorForLanguageModeling(pad_token_id=999)(ex), input_ids=[[1, 2, 3], [4, 5, 999]],
        attention_mask=[[1, 1, 1], [1, 1, 0]], labels=[[1, 2, 3], [4, 5, -100]])
    _eq(c([{"input_ids": [1, 2, 3, 4], "labels": [1, 2, 3, 4]}]), input_ids=[[1, 2, 3, 4]], attention_mask=[[1, 1, 1, 1]],
        labels=[[1, 2, 3, 4]])


def test_language_modeling_padding_free_and_packed_batches():
    ex = [{"input_ids": [1, 2, 3], "labels": [1, 2, 3]}, {"input_ids": [4, 5], "labels": [4, 5]}]
    c = DataCollatorForLanguageModeling(pad_token_id=0, padding_free=True)
    want = dict(input_ids=[[1, 2, 3, 4, 5]], position_ids=[[0, 1, 2, 0, 1]], labels=[[-100, 2, 3, -100, 5]])
    _eq(c(ex), **want)
    _eq(c([{"input_ids": [1, 2, 3]}, {"input_ids": [4, 5]}]), **want)
    packed = [{"input_ids": [1, 2, 3, 4, 5, 6], "seq_lengths": [3, 3], "labels": [1, 2, 3, 4, 5, 6]},
              {"input_ids": [7, 8, 9, 10, 11], "seq_lengths": [4, 1], "labels": [7, 8, 9, 10, 11]}]
    _eq(c(packed), input_ids=[[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]], position_ids=[[0, 1, 2, 0, 1, 2, 0, 1, 2, 3, 0]],
        labels=[[-100, 2, 3, -100, 5, 6, -100, 8, 9, 10, -100]])
    _eq(DataCollatorForLanguageModeling(pad_token_id=0, padding_free=True, pad_to_multiple_of=4)(ex),
        input_ids=[[1, 2, 3, 4, 5, 0, 0, 0]], position_ids=[[0, 1, 2, 0, 1, 0, 0, 0]],
        labels=[[-100, 2, 3, -100, 5, -100, -100, -100]])
    pos = DataCollatorForLanguageModeling.get_position_ids_from_packed_seq_lengths
    assert [p.tolist() for p in pos([[5]])] == [[0, 1, 2, 3, 4]]
    assert [p.tolist() for p in pos([[3, 2]])] == [[0, 1, 2, 0, 1]]
    assert [p.tolist() for p in pos([[2, 2], [3]])] == [[0, 1, 0, 1], [0, 1, 2]]


def test_dpo_preference_batches():
    from trl_b200.trainer.dpo_trainer import DataCollatorForPreference

    c = DataCollatorForPreference(pad_token_id=0)
    out = c([{"prompt_ids": [1, 2, 3], "chosen_ids": [4, 5], "rejected_ids": [6]},
             {"prompt_ids": [7, 8], "chosen_ids": [9, 10], "rejected_ids": [11, 12, 13]}])
    _eq(out, input_ids=[[1, 2, 3, 4, 5], [7, 8, 9, 10, 0], [1, 2, 3, 6, 0], [7, 8, 11, 12, 13]],
        attention_mask=[[1, 1, 1, 1, 1], [1, 1, 1, 1, 0], [1, 1, 1, 1, 0], [1, 1, 1, 1, 1]],
        completion_mask=[[0, 0, 0, 1, 1], [0, 0, 1, 1, 0], [0, 0, 0, 1, 0], [0, 0, 1, 1, 1]])
    out = c([{"prompt_ids": [1, 2], "chosen_ids": [3], "rejected_ids": [4], "ref_chosen_logps": 0.1, "ref_rejected_logps": 0.2},
             {"prompt_ids": [5], "chosen_ids": [6, 7], "rejected_ids": [8, 9], "ref_chosen_logps": 0.3, "ref_rejected_logps": 0.4}])
    assert set(out) == {"input_ids", "attention_mask", "completion_mask", "ref_chosen_logps", "ref_rejected_logps"}
    torch.testing.assert_close(out["ref_chosen_logps"], T([0.1, 0.3]))
    torch.testing.assert_close(out["ref_rejected_logps"], T([0.2, 0.4]))
    out = DataCollatorForPreference(pad_token_id=0, pad_to_multiple_of=5)(
        [{"prompt_ids": [1], "chosen_ids": [2], "rejected_ids": [3]},
         {"prompt_ids": [4, 5], "chosen_ids": [6, 7], "rejected_ids": [8, 9]}])
    assert set(out) == {"input_ids", "attention_mask", "completion_mask"}
    assert out["input_ids"].tolist() == [[1, 2, 0, 0, 0], [4, 5, 6, 7, 0], [1, 3, 0, 0, 0], [4, 5, 8, 9, 0]]


def test_reward_preference_batches():
    from trl_b200.trainer.reward_trainer import DataCollatorForPreference

    ex = [{"chosen_ids": [1, 2, 3], "rejected_ids": [4, 5]}, {"chosen_ids": [6, 7], "rejected_ids": [8]}]
    out = DataCollatorForPreference(pad_token_id=0)(ex)
    assert out["input_ids"].tolist() == [[1, 2, 3], [6, 7, 0], [4, 5, 0], [8, 0, 0]]
    assert out["attention_mask"].tolist() == [[1, 1, 1], [1, 1, 0], [1, 1, 0], [1, 0, 0]]
    out = DataCollatorForPreference(pad_token_id=0, pad_to_multiple_of=4)(ex)
    assert out["input_ids"].tolist() == [[1, 2, 3, 0], [6, 7, 0, 0], [4, 5, 0, 0], [8, 0, 0, 0]]
    assert out["attention_mask"].tolist() == [[1, 1, 1, 0], [1, 1, 0, 0], [1, 1, 0, 0], [1, 0, 0, 0]]
    out = DataCollatorForPreference(pad_token_id=0)(ex[:1])
    assert out["input_ids"].tolist() == [[1, 2, 3], [4, 5, 0]] and out["attention_mask"].tolist() == [[1, 1, 1], [1, 1, 0]]
    out = DataCollatorForPreference(pad_token_id=999)(ex)
    assert out["input_ids"].tolist() == [[1, 2, 3], [6, 7, 999], [4, 5, 999], [8, 999, 999]]
    out = DataCollatorForPreference(pad_token_id=0)([{**ex[0], "margin": 0.1}, {**ex[1], "margin": 0.2}])
    assert out["input_ids"].tolist() == [[1, 2, 3], [6, 7, 0], [4, 5, 0], [8, 0, 0]]
    torch.testing.assert_close(out["margin"], T([0.1, 0.2]))


def test_kto_unpaired_preference_batches():
    from trl_b200.trainer.kto_trainer import DataCollatorForUnpairedPreference

    c = DataCollatorForUnpairedPreference(pad_token_id=0)
    out = c([{"prompt_ids": [1, 2, 3], "completion_ids": [4, 5], "KL_completion_ids": [6], "label": True},
             {"prompt_ids": [7, 8], "completion_ids": [9, 10], "KL_completion_ids": [11, 12, 13], "label": False}])
    _eq(out, input_ids=[[1, 2, 3, 4, 5], [7, 8, 9, 10, 0]], attention_mask=[[1, 1, 1, 1, 1], [1, 1, 1, 1, 0]],
        completion_mask=[[0, 0, 0, 1, 1], [0, 0, 1, 1, 0]], KL_input_ids=[[1, 2, 3, 6, 0], [7, 8, 11, 12, 13]],
        KL_attention_mask=[[1, 1, 1, 1, 0], [1, 1, 1, 1, 1]], KL_completion_mask=[[0, 0, 0, 1, 0], [0, 0, 1, 1, 1]],
        label=[True, False])
    out = c([{"prompt_ids": [1, 2], "completion_ids": [3], "KL_completion_ids": [4], "ref_logps": 0.1, "ref_KL_logps": 0.2,
              "label": True},
             {"prompt_ids": [5], "completion_ids": [6, 7], "KL_completion_ids": [8, 9], "ref_logps": 0.3, "ref_KL_logps": 0.4,
              "label": False}])
    assert set(out) == {"input_ids", "attention_mask", "completion_mask", "KL_input_ids", "KL_attention_mask",
                        "KL_completion_mask", "label", "ref_logps", "ref_KL_logps"}
    torch.testing.assert_close(out["ref_logps"], T([0.1, 0.3]))
    torch.testing.assert_close(out["ref_KL_logps"], T([0.2, 0.4]))
