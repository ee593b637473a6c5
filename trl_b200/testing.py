"""Offline fixtures: a local tokenizer with a ChatML template, tiny random-init
models, and synthetic datasets in each of the dataset formats the trainers
accept.  They stand in for the Hub-hosted tiny models and the ``zen`` dataset
the reference tests download (tests/test_sft_trainer.py:328-338).
"""
from __future__ import annotations

import random

import torch

from .models.configuration import ModelArch, preset
from .models.decoder import CausalLM

CHATML_TEMPLATE = (
    "{% for message in messages %}"
    "{{ '<|im_start|>' + message['role'] + '\n' }}"
    "{% if message['role'] == 'assistant' %}{% generation %}{{ message['content'] + '<|im_end|>' }}{% endgeneration %}"
    "{% else %}{{ message['content'] + '<|im_end|>' }}{% endif %}"
    "{{ '\n' }}"
    "{% endfor %}"
    "{% if add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}"
)

_WORDS = ("the of and to in is that for it as was with be by on not he this are or his from at which but have an had "
          "they you were their one all we can her has there been if more when will would who so no said what up its "
          "about into than them only other new some could time these two may then do first any my now such like our "
          "over man me even most made after also did many before must through years where much your way well down "
          "should because each just those people how too little state good very make world still own see men work "
          "long get here between both life being under never day same another know while last might us great old "
          "year off come since against go came right used take three beautiful explicit simple flat sparse "
          "readability special cases errors ambiguity obvious namespaces better ugly implicit complex complicated "
          "nested dense counts practicality purity silently silenced refuse guess dutch idea explain").split()


def make_tiny_tokenizer(vocab_size: int = 1024):
    """Word-level tokenizer (whitespace + punctuation) with ChatML special tokens; built locally."""
    from tokenizers import Tokenizer, models, pre_tokenizers, decoders
    from transformers import PreTrainedTokenizerFast

    specials = ["<|pad|>", "<|endoftext|>", "<|im_start|>", "<|im_end|>", "<unk>"]
    base = list(dict.fromkeys(list(_WORDS) + ["user", "assistant", "system", "tool", "\n", ".", ",", "?", "!", ":", "'",
                                              "<think>", "</think>"] + [str(i) for i in range(10)] +
                              [chr(c) for c in range(ord("a"), ord("z") + 1)] + [chr(c) for c in range(ord("A"), ord("Z") + 1)]))
    vocab = {t: i for i, t in enumerate(specials)}
    for w in base:
        if w not in vocab and len(vocab) < vocab_size:
            vocab[w] = len(vocab)
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split("\n", behavior="isolated"),
        pre_tokenizers.WhitespaceSplit(),
        pre_tokenizers.Punctuation(behavior="isolated"),
    ])
    # special tokens contain punctuation: registering them keeps them whole
    tok.add_special_tokens(specials[:4])
    tok.decoder = decoders.Fuse()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<|pad|>", eos_token="<|im_end|>",
                                   bos_token=None, unk_token="<unk>")
    fast.chat_template = CHATML_TEMPLATE
    return fast


def make_tiny_model(name: str = "tiny-qwen2", dtype=torch.float32, device=None, seed: int = 0, **overrides) -> CausalLM:
    torch.manual_seed(seed)
    cfg = preset(name, **overrides)
    return CausalLM(cfg, dtype=dtype, device=device)


def _sentence(rng: random.Random, lo=3, hi=12) -> str:
    return " ".join(rng.choice(_WORDS) for _ in range(rng.randint(lo, hi))) + "."


def make_dataset(kind: str, n: int = 20, seed: int = 0):
    """Synthetic rows in one of the reference's dataset formats; returns ``datasets.Dataset``."""
    from datasets import Dataset

    rng = random.Random(seed)
    rows = []
    for i in range(n):
        p, c, r = _sentence(rng), _sentence(rng), _sentence(rng)
        if kind == "standard_language_modeling":
            rows.append({"text": p + " " + c})
        elif kind == "conversational_language_modeling":
            rows.append({"messages": [{"role": "user", "content": p}, {"role": "assistant", "content": c}]})
        elif kind == "standard_prompt_only":
            rows.append({"prompt": p})
        elif kind == "conversational_prompt_only":
            rows.append({"prompt": [{"role": "user", "content": p}]})
        elif kind == "standard_prompt_completion":
            rows.append({"prompt": p, "completion": " " + c})
        elif kind == "conversational_prompt_completion":
            rows.append({"prompt": [{"role": "user", "content": p}], "completion": [{"role": "assistant", "content": c}]})
        elif kind == "standard_preference":
            rows.append({"prompt": p, "chosen": " " + c, "rejected": " " + r})
        elif kind == "conversational_preference":
            rows.append({"prompt": [{"role": "user", "content": p}], "chosen": [{"role": "assistant", "content": c}],
                         "rejected": [{"role": "assistant", "content": r}]})
        elif kind == "standard_implicit_prompt_preference":
            rows.append({"chosen": p + " " + c, "rejected": p + " " + r})
        elif kind == "conversational_implicit_prompt_preference":
            rows.append({"chosen": [{"role": "user", "content": p}, {"role": "assistant", "content": c}],
                         "rejected": [{"role": "user", "content": p}, {"role": "assistant", "content": r}]})
        elif kind == "standard_unpaired_preference":
            rows.append({"prompt": p, "completion": " " + c, "label": bool(i % 2)})
        elif kind == "conversational_unpaired_preference":
            rows.append({"prompt": [{"role": "user", "content": p}], "completion": [{"role": "assistant", "content": c}],
                         "label": bool(i % 2)})
        elif kind == "standard_stepwise_supervision":
            steps = [_sentence(rng) for _ in range(rng.randint(1, 4))]
            rows.append({"prompt": p, "completions": steps, "labels": [bool(rng.getrandbits(1)) for _ in steps]})
        else:
            raise ValueError(f"unknown dataset kind {kind!r}")
    return Dataset.from_list(rows)


def synthetic_token_batches(vocab: int, n_rows: int, seq_len: int, seed: int, min_len: int = 16):
    """Packed rows of uniform-random token ids with document lengths uniform in [min_len, seq_len]
    and a completion-only mask on the second half of every document."""
    g = torch.Generator().manual_seed(seed)
    rows = []
    for _ in range(n_rows):
        ids, lens, mask = [], [], []
        left = seq_len
        while left >= min_len:
            L = int(torch.randint(min_len, seq_len + 1, (1,), generator=g))
            L = min(L, left)
            ids.append(torch.randint(0, vocab, (L,), generator=g))
            m = torch.zeros(L, dtype=torch.long)
            m[L // 2:] = 1
            mask.append(m)
            lens.append(L)
            left -= L
        rows.append({"input_ids": torch.cat(ids).tolist(), "completion_mask": torch.cat(mask).tolist(),
                     "seq_lengths": lens})
    return rows
