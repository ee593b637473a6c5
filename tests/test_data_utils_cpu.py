"""Dataset-format helpers, packing and collators (literal expected outputs)."""
import pytest
import torch

from trl_b200.data_utils import (_SegmentTree, apply_chat_template, extract_prompt, is_conversational,
                                 maybe_convert_to_chatml, maybe_extract_prompt, maybe_unpair_preference_dataset,
                                 pack_dataset, unpair_preference_dataset, bfd_assign)
from trl_b200.trainer.sft_trainer import DataCollatorForLanguageModeling


def test_padding_free_collate():
    c = DataCollatorForLanguageModeling(pad_token_id=0, padding_free=True)
    out = c([{"input_ids": [1, 2, 3]}, {"input_ids": [4, 5]}])
    assert out["input_ids"].tolist() == [[1, 2, 3, 4, 5]]
    assert out["position_ids"].tolist() == [[0, 1, 2, 0, 1]]
    assert out["labels"].tolist() == [[-100, 2, 3, -100, 5]]
    assert "attention_mask" not in out


def test_packed_collate_with_seq_lengths_and_pad_multiple():
    c = DataCollatorForLanguageModeling(pad_token_id=0, padding_free=True)
    out = c([{"input_ids": [1, 2, 3, 4, 5, 6], "seq_lengths": [3, 3]}, {"input_ids": [7, 8, 9, 10, 11], "seq_lengths": [4, 1]}])
    assert out["position_ids"].tolist() == [[0, 1, 2, 0, 1, 2, 0, 1, 2, 3, 0]]
    assert out["labels"].tolist() == [[-100, 2, 3, -100, 5, 6, -100, 8, 9, 10, -100]]
    c2 = DataCollatorForLanguageModeling(pad_token_id=99, padding_free=True, pad_to_multiple_of=4)
    o2 = c2([{"input_ids": [1, 2, 3]}, {"input_ids": [4, 5]}])
    assert o2["input_ids"].tolist() == [[1, 2, 3, 4, 5, 99, 99, 99]]
    assert o2["position_ids"].tolist() == [[0, 1, 2, 0, 1, 0, 0, 0]] and o2["labels"][0, 5:].tolist() == [-100] * 3


def test_padded_collate_and_completion_mask():
    c = DataCollatorForLanguageModeling(pad_token_id=0)
    out = c([{"input_ids": [1, 2, 3], "completion_mask": [0, 1, 1]}, {"input_ids": [4, 5], "completion_mask": [0, 1]}])
    assert out["input_ids"].tolist() == [[1, 2, 3], [4, 5, 0]] and out["attention_mask"].tolist() == [[1, 1, 1], [1, 1, 0]]
    assert out["labels"].tolist() == [[-100, 2, 3], [-100, 5, -100]]


def test_bfd_packing_literal():
    rows = [{"input_ids": [1, 2, 3]}, {"input_ids": [4, 5, 6, 7]}, {"input_ids": [8]}]
    out = pack_dataset(rows, 4, "bfd")
    assert [r["input_ids"] for r in out] == [[4, 5, 6, 7], [1, 2, 3, 8]]
    assert [r["seq_lengths"] for r in out] == [[4], [3, 1]]


def test_bfd_truncates_and_bfd_split_requeues():
    rows = [{"input_ids": [1, 2, 3, 4, 5]}, {"input_ids": [6, 7]}, {"input_ids": [8, 9, 10, 11]}, {"input_ids": [12]},
            {"input_ids": []}]
    a = pack_dataset(rows, 4, "bfd")
    assert [r["input_ids"] for r in a] == [[1, 2, 3, 4], [8, 9, 10, 11], [6, 7, 12]]
    assert [r["seq_lengths"] for r in a] == [[4], [4], [2, 1]]
    b = pack_dataset(rows, 4, "bfd_split")
    assert [r["input_ids"] for r in b] == [[1, 2, 3, 4], [8, 9, 10, 11], [6, 7, 5, 12]]
    assert [r["seq_lengths"] for r in b] == [[4], [4], [2, 1, 1]]
    w = pack_dataset(rows, 4, "wrapped")
    assert [r["input_ids"] for r in w] == [[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]]


def test_pack_dataset_hf_dataset_and_native_matches_python():
    from datasets import Dataset
    import random

    ds = Dataset.from_dict({"input_ids": [[1, 2, 3], [4, 5, 6, 7], [8]], "completion_mask": [[0, 1, 1], [0, 0, 1, 1], [1]]})
    out = pack_dataset(ds, 4, "bfd")
    assert out["input_ids"] == [[4, 5, 6, 7], [1, 2, 3, 8]] and out["completion_mask"] == [[0, 0, 1, 1], [0, 1, 1, 1]]
    rng = random.Random(0)
    lens = [rng.randint(1, 64) for _ in range(500)]
    bins = bfd_assign(lens, 64)
    assert sorted(i for b in bins for i in b) == list(range(500))
    assert all(sum(lens[i] for i in b) <= 64 for b in bins)
    assert len(bins) <= int(sum(lens) / 64 * 1.1) + 1


def test_segment_tree():
    t = _SegmentTree(10)
    for v in (5, 2, 8):
        t.add(v)
    assert t.search(3) == 5 and t.search(6) == 8 and t.search(1) == 2
    t.remove(5)
    assert t.search(3) == 8 and t.search(9) == 0


def test_conversational_and_chatml_conversion():
    assert is_conversational({"prompt": [{"role": "user", "content": "hi"}]})
    assert not is_conversational({"prompt": "hi"})
    ex = maybe_convert_to_chatml({"conversations": [{"from": "user", "value": "a"}, {"from": "assistant", "value": "b"}]})
    assert ex == {"messages": [{"role": "user", "content": "a"}, {"role": "assistant", "content": "b"}]}


def test_unpair_and_extract_prompt():
    rows = [{"prompt": "p", "chosen": "c", "rejected": "r"}]
    un = unpair_preference_dataset(rows)
    assert un == [{"prompt": "p", "completion": "c", "label": True}, {"prompt": "p", "completion": "r", "label": False}]
    assert maybe_unpair_preference_dataset([{"prompt": "p", "completion": "c", "label": True}])[0]["label"] is True
    e = extract_prompt({"chosen": "The sky is blue", "rejected": "The sky is green"})
    assert e == {"prompt": "The sky is", "chosen": " blue", "rejected": " green"}
    conv = {"chosen": [{"role": "user", "content": "q"}, {"role": "assistant", "content": "a"}],
            "rejected": [{"role": "user", "content": "q"}, {"role": "assistant", "content": "b"}]}
    m = maybe_extract_prompt(conv)
    assert m["prompt"] == [{"role": "user", "content": "q"}] and m["chosen"] == [{"role": "assistant", "content": "a"}]


def test_apply_chat_template_variants(tiny_tokenizer):
    tok = tiny_tokenizer
    p = [{"role": "user", "content": "the sky"}]
    c = [{"role": "assistant", "content": "is good"}]
    out = apply_chat_template({"prompt": p, "completion": c}, tok)
    assert out["prompt"].endswith("<|im_start|>assistant\n") and out["completion"].startswith("is good<|im_end|>")
    full = apply_chat_template({"messages": p + c}, tok)["text"]
    assert full == out["prompt"] + out["completion"]
    pref = apply_chat_template({"prompt": p, "chosen": c, "rejected": [{"role": "assistant", "content": "no"}]}, tok)
    assert pref["chosen"].startswith("is good") and pref["rejected"].startswith("no")
    with pytest.raises(KeyError):
        apply_chat_template({"prompt": p, "messages": p}, tok)


def test_prepare_multimodal_messages_cases():
    """The cases of tests/test_data_utils.py:48-270: images go to the first user turn, strings become text blocks,
    prepared turns keep their blocks (placeholders are filled), tool-call turns pass through."""
    from PIL import Image

    from trl_b200.data_utils import prepare_multimodal_messages

    img = Image.new("RGB", (10, 10), color="blue")
    user = lambda *blocks: {"role": "user", "content": list(blocks)}                 # noqa: E731
    txt = lambda s: {"type": "text", "text": s}                                      # noqa: E731
    out = prepare_multimodal_messages([{"role": "user", "content": "What color is the sky?"},
                                       {"role": "assistant", "content": "It is blue."},
                                       {"role": "user", "content": "How about the grass?"}], images=[img])
    assert out == [user({"type": "image", "image": img}, txt("What color is the sky?")),
                   {"role": "assistant", "content": [txt("It is blue.")]}, user(txt("How about the grass?"))]
    imgs = [Image.new("RGB", (10, 10), color=c) for c in ("red", "green", "blue")]
    out = prepare_multimodal_messages([{"role": "user", "content": "q"}, {"role": "assistant", "content": "a"}], images=imgs)
    assert out[0] == user(*[{"type": "image", "image": i} for i in imgs], txt("q"))
    out = prepare_multimodal_messages([{"role": "system", "content": "You are a helpful assistant"},
                                       {"role": "user", "content": "q"}], images=[img])
    assert out == [{"role": "system", "content": [txt("You are a helpful assistant")]}, user({"type": "image", "image": img}, txt("q"))]
    # already prepared: the image placeholder is filled, nothing else changes
    prepared = [{"role": "system", "content": [txt("s")]}, user({"type": "image"}, txt("q")),
                {"role": "assistant", "content": [txt("a")]}]
    assert prepare_multimodal_messages(prepared, images=[img]) == [
        {"role": "system", "content": [txt("s")]}, user({"type": "image", "image": img}, txt("q")),
        {"role": "assistant", "content": [txt("a")]}]
    mixed = [{"role": "user", "content": "q1"}, {"role": "assistant", "content": [txt("a")]}, {"role": "user", "content": "q2"}]
    assert prepare_multimodal_messages(mixed, images=[img]) == [user({"type": "image", "image": img}, txt("q1")),
                                                                {"role": "assistant", "content": [txt("a")]}, user(txt("q2"))]
    call = {"role": "assistant", "tool_calls": [{"type": "tool", "function": {"name": "get_current_weather",
                                                                               "arguments": {"location": "New York"}}}]}
    out = prepare_multimodal_messages([{"role": "user", "content": "weather?"}, call,
                                       {"role": "tool", "name": "get_current_weather", "content": "22.0"},
                                       {"role": "assistant", "content": "22 degrees."}])
    assert out == [user(txt("weather?")), call, {"role": "tool", "name": "get_current_weather", "content": [txt("22.0")]},
                   {"role": "assistant", "content": [txt("22 degrees.")]}]
    keep = [user({"type": "image", "image": img}, txt("q")), {"role": "assistant", "content": "a"}]
    assert prepare_multimodal_messages(keep) == [user({"type": "image", "image": img}, txt("q")),
                                                 {"role": "assistant", "content": [txt("a")]}]


def test_prepare_multimodal_messages_vllm_cases():
    import copy

    from PIL import Image

    from trl_b200.data_utils import prepare_multimodal_messages_vllm

    img = Image.new("RGB", (10, 10), color="blue")
    msgs = [{"role": "user", "content": [{"type": "text", "text": "q"}, {"type": "image", "image": img}]},
            {"role": "assistant", "content": [{"type": "text", "text": "It is blue."}]}]
    original = copy.deepcopy(msgs)
    out = prepare_multimodal_messages_vllm(msgs)
    assert msgs == original                                                  # the input is not touched
    assert out[0]["content"][0]["type"] == "text" and out[0]["content"][1]["type"] == "image_pil"
    assert "image" not in out[0]["content"][1] and isinstance(out[0]["content"][1]["image_pil"], Image.Image)
    assert out[1]["content"][0] == {"type": "text", "text": "It is blue."}
    plain = [{"role": "user", "content": [{"type": "text", "text": "q"}]}]
    res = prepare_multimodal_messages_vllm(plain)
    assert res == plain and res is not plain and res[0] is not plain[0]


def test_unpair_preference_dataset_cases():
    """tests/test_data_utils.py:1008-1107: map-style, iterable, dataset dict, extra columns, already unpaired."""
    from datasets import Dataset, DatasetDict

    from trl_b200.data_utils import maybe_unpair_preference_dataset, unpair_preference_dataset

    paired = Dataset.from_dict({"prompt": ["The sky is", "The sun is"], "chosen": [" blue.", " in the sky."],
                                "rejected": [" green.", " in the sea."]})
    want = {"prompt": ["The sky is", "The sun is", "The sky is", "The sun is"],
            "completion": [" blue.", " in the sky.", " green.", " in the sea."], "label": [True, True, False, False]}
    assert unpair_preference_dataset(paired).to_dict() == want
    extra = Dataset.from_dict({**paired.to_dict(), "extra": [1, 2]})
    assert unpair_preference_dataset(extra).to_dict() == {**want, "extra": [1, 2, 1, 2]}
    rows = list(unpair_preference_dataset(paired.to_iterable_dataset()))
    assert rows == [dict(zip(want, vals)) for vals in zip(*want.values())]
    rows = list(unpair_preference_dataset(extra.to_iterable_dataset()))
    want_x = {**want, "extra": [1, 2, 1, 2]}
    assert rows == [dict(zip(want_x, vals)) for vals in zip(*want_x.values())]
    assert unpair_preference_dataset(DatasetDict({"abc": paired}))["abc"].to_dict() == want
    assert maybe_unpair_preference_dataset(paired).to_dict() == want
    assert maybe_unpair_preference_dataset(DatasetDict({"abc": paired}))["abc"].to_dict() == want
    unpaired = Dataset.from_dict(want)
    assert maybe_unpair_preference_dataset(unpaired).to_dict() == want
    assert maybe_unpair_preference_dataset(DatasetDict({"abc": unpaired}))["abc"].to_dict() == want


def test_extract_prompt_cases_and_is_conversational():
    from trl_b200.data_utils import (extract_prompt, is_conversational, is_conversational_from_value, maybe_extract_prompt)

    implicit = {"chosen": [{"role": "user", "content": "What color is the sky?"}, {"role": "assistant", "content": "It is blue."}],
                "rejected": [{"role": "user", "content": "What color is the sky?"}, {"role": "assistant", "content": "It is green."}]}
    explicit = {"prompt": [{"role": "user", "content": "What color is the sky?"}],
                "chosen": [{"role": "assistant", "content": "It is blue."}],
                "rejected": [{"role": "assistant", "content": "It is green."}]}
    assert extract_prompt(implicit) == explicit and maybe_extract_prompt(implicit) == explicit
    assert maybe_extract_prompt(explicit) == explicit
    std_implicit, std_explicit = {"chosen": "The sky is blue.", "rejected": "The sky is green."}, \
        {"prompt": "The sky is", "chosen": " blue.", "rejected": " green."}
    assert extract_prompt(std_implicit) == std_explicit and maybe_extract_prompt(std_implicit) == std_explicit
    assert maybe_extract_prompt(std_explicit) == std_explicit
    sky = [{"role": "user", "content": "What color is the sky?"}]
    think = {"role": "assistant", "thinking": "The user asks the color of the sky...", "content": "It is blue."}
    call = {"role": "assistant", "tool_calls": [{"type": "function", "function": {"name": "get_color", "arguments": {"what": "sky"}}}]}
    for ex in ({"messages": sky + [{"role": "assistant", "content": "It is blue."}]}, {"prompt": sky},
               {"prompt": sky, "completion": [{"role": "assistant", "content": "It is blue."}]}, explicit, implicit,
               {"prompt": sky, "chosen": [call, {"role": "tool", "name": "get_color", "content": "blue"}], "rejected": [call]},
               {"prompt": sky, "completion": [think], "label": True},
               {"messages": [{"role": "system", "content": "Respond in a friendly manner."}] + sky + [think]}):
        assert is_conversational(ex), ex
    for ex in ({"prompt": "The sky is", "completion": " blue."}, {"text": "The sky is blue."}, {"prompt": "The sky is"},
               std_explicit, {"prompt": "The sky is", "completion": " blue.", "label": True}):
        assert not is_conversational(ex), ex
    assert is_conversational_from_value({"conversations": [{"from": "user", "value": "q"}, {"from": "assistant", "value": "a"}]})
    assert not is_conversational_from_value({"messages": sky}) and not is_conversational_from_value({"text": "x"})


def test_pack_dataset_reference_vectors():
    """tests/test_data_utils.py:1184-1325: wrapped / bfd / bfd_split on map-style and iterable datasets; the dataset's
    format survives, seq_lengths is added to the formatted columns."""
    from datasets import Dataset

    from trl_b200.data_utils import pack_dataset

    ex = {"input_ids": [[1, 2, 3], [4, 5, 6, 7], [8]], "attention_mask": [[0, 1, 1], [0, 0, 1, 1], [1]]}
    want = {"input_ids": [[1, 2, 3], [4, 5, 6], [7, 8]], "attention_mask": [[0, 1, 1], [0, 0, 1], [1, 1]]}
    ds = Dataset.from_dict(ex).with_format("numpy", dtype="float32")
    fmt = ds.format
    out = pack_dataset(ds, 3, strategy="wrapped")
    assert out.to_dict() == want and out.format == fmt
    it = Dataset.from_dict(ex).to_iterable_dataset().with_format("numpy")
    out = pack_dataset(it, 3, strategy="wrapped")
    assert next(iter(out.with_format(None).batch(batch_size=3))) == want
    assert out._formatting == it._formatting

    ex = {"input_ids": [[1, 2, 3], [4, 5, 6, 7], [8]]}
    want = {"input_ids": [[4, 5, 6, 7], [1, 2, 3, 8]], "seq_lengths": [[4], [3, 1]]}
    ds = Dataset.from_dict(ex).with_format("numpy", dtype="float32")
    fmt = ds.format
    out = pack_dataset(ds, 4, strategy="bfd")
    got_fmt = out.format
    assert out.to_dict() == want and "seq_lengths" in got_fmt["columns"]
    got_fmt["columns"].remove("seq_lengths")
    assert got_fmt == fmt
    it = Dataset.from_dict(ex).to_iterable_dataset().with_format("numpy")
    out = pack_dataset(it, 4, strategy="bfd")
    assert next(iter(out.with_format(None).batch(batch_size=3))) == want

    cases = [
        ({"input_ids": [[1, 2, 3, 4, 5], [6, 7], [8, 9, 10, 11], [12]]}, 4, "bfd_split",
         {"input_ids": [[1, 2, 3, 4], [8, 9, 10, 11], [6, 7, 5, 12]], "seq_lengths": [[4], [4], [2, 1, 1]]}),
        ({"col1": [[1, -2, 3, -4, 5, -6], [7, -8, 9], [-10, 11, -12], [13, -14, 15, -16]],
          "col2": [[-1, 2, -3, 4, -5, 6], [-7, 8, -9], [10, -11, 12], [-13, 14, -15, 16]]}, 4, "bfd_split",
         {"col1": [[1, -2, 3, -4], [13, -14, 15, -16], [7, -8, 9], [-10, 11, -12], [5, -6]],
          "col2": [[-1, 2, -3, 4], [-13, 14, -15, 16], [-7, 8, -9], [10, -11, 12], [-5, 6]],
          "seq_lengths": [[4], [4], [3], [3], [2]]}),
        ({"input_ids": [[1, 2, 3, 4, 5], [6], [7, 8, 9, 10], [11, 12, 13]]}, 5, "bfd_split",
         {"input_ids": [[1, 2, 3, 4, 5], [7, 8, 9, 10, 6], [11, 12, 13]], "seq_lengths": [[5], [4, 1], [3]]}),
        ({"input_ids": [[1, 2, 3, 4, 5], [6, 7], [8, 9, 10, 11], [12]]}, 4, "bfd",
         {"input_ids": [[1, 2, 3, 4], [8, 9, 10, 11], [6, 7, 12]], "seq_lengths": [[4], [4], [2, 1]]}),
        ({"input_ids": [[1, 2], [], [3, 4, 5], [], [6]]}, 4, "bfd_split",
         {"input_ids": [[3, 4, 5, 6], [1, 2]], "seq_lengths": [[3, 1], [2]]}),
    ]
    for ex, L, strat, want in cases:
        assert pack_dataset(Dataset.from_dict(ex), L, strategy=strat).to_dict() == want, (ex, strat)


def test_maybe_convert_to_chatml_cases():
    from trl_b200.data_utils import maybe_convert_to_chatml

    msgs = [{"role": "user", "content": "What color is the sky?"}, {"role": "assistant", "content": "It is blue."}]
    raw = [{"from": "user", "value": "What color is the sky?"}, {"from": "assistant", "value": "It is blue."}]
    assert maybe_convert_to_chatml({"conversations": raw}) == {"messages": msgs}
    assert maybe_convert_to_chatml({"prompt": raw[:1], "completion": raw[1:]}) == {"prompt": msgs[:1], "completion": msgs[1:]}
    assert maybe_convert_to_chatml({"text": "The sky is blue."}) == {"text": "The sky is blue."}
    assert maybe_convert_to_chatml({"messages": msgs}) == {"messages": msgs}


def test_apply_chat_template_generation_prompt_that_inserts_text_round_trips():
    """tests/test_data_utils.py:723-748: the completions are cut against the final (shortest) prompt, so a tag opened by
    the generation prompt stays with the completion that keeps it."""
    from trl_b200.data_utils import apply_chat_template
    from trl_b200.testing import make_tiny_tokenizer

    tok = make_tiny_tokenizer()
    tok.chat_template = ("{% for message in messages %}{{ message['role'] + ': ' + message['content'] + '\n' }}{% endfor %}"
                         "{% if add_generation_prompt %}{{ 'assistant: <think>' }}{% endif %}")
    ex = {"prompt": [{"role": "user", "content": "What is 2+2?"}],
          "chosen": [{"role": "assistant", "content": "<think>2+2=4</think>It is 4."}],
          "rejected": [{"role": "assistant", "content": "It is 4."}]}
    out = apply_chat_template(ex, tok)
    assert out["prompt"] + out["chosen"] == tok.apply_chat_template(ex["prompt"] + ex["chosen"], tokenize=False)
    assert out["prompt"] + out["rejected"] == tok.apply_chat_template(ex["prompt"] + ex["rejected"], tokenize=False)
    assert out["chosen"].startswith("<think>")
