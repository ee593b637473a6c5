"""Dataset-format helpers: conversational detection, chat templating, preference
(un)pairing, prompt extraction and sequence packing.

Behavioural parity with trl/data_utils.py (function names and results);
the packing core is a native best-fit-decreasing packer (``csrc/host_runtime.cpp``)
with a pure-Python fallback of the same algorithm.
"""
from __future__ import annotations

import copy
from collections import defaultdict
from typing import Any, Callable, Sequence

import numpy as np

try:  # datasets is optional at import time
    from datasets import Dataset, DatasetDict, IterableDataset
except Exception:  # pragma: no cover
    Dataset = DatasetDict = IterableDataset = None

_CONV_KEYS = ("prompt", "chosen", "rejected", "completion", "messages")
_TEMPLATE_KEYSETS = [
    {"messages"}, {"prompt"}, {"prompt", "completion"}, {"prompt", "chosen", "rejected"},
    {"chosen", "rejected"}, {"prompt", "completion", "label"},
]


# ---------------------------------------------------------------------------
# multimodal message normalisation
# ---------------------------------------------------------------------------
def prepare_multimodal_messages(messages: list[dict], images: list | None = None) -> list[dict]:
    """String contents become ``[{"type": "text", ...}]`` blocks; image placeholders are
    inserted into the first user turn and filled from ``images`` in order."""
    images = list(images or [])
    out = copy.deepcopy(messages)
    placed = False
    for m in out:
        c = m.get("content")
        if isinstance(c, str):
            if m["role"] == "user" and images and not placed:
                m["content"] = [{"type": "image"} for _ in images] + [{"type": "text", "text": c}]
                placed = True
            else:
                m["content"] = [{"type": "text", "text": c}]
    # placeholders still to fill: image blocks that carry no payload yet (turns without content, such as an assistant
    # turn that only holds tool calls, stay as they are)
    slots = [b for m in out for b in (m.get("content") or []) if isinstance(b, dict) and b.get("type") == "image"
             and b.get("image") is None]
    if len(slots) != len(images):
        raise ValueError(f"Number of images provided ({len(images)}) does not match number of image placeholders ({len(slots)}).")
    for b, img in zip(slots, images):
        b["image"] = img
    return out


def prepare_multimodal_messages_vllm(messages: list[dict]) -> list[dict]:
    """Rollout-engine flavour: ``{"type": "image", "image": x}`` -> ``{"type": "image_pil", "image_pil": x}``."""
    out = copy.deepcopy(messages)
    for m in out:
        if isinstance(m.get("content"), list):
            for b in m["content"]:
                if b.get("type") == "image":
                    b["type"] = "image_pil"
                    b["image_pil"] = b.pop("image", None)
    return out


# ---------------------------------------------------------------------------
# format detection / conversion
# ---------------------------------------------------------------------------
def is_conversational(example: dict[str, Any]) -> bool:
    for k in _CONV_KEYS:
        if k in example:
            v = example[k]
            return isinstance(v, list) and len(v) > 0 and isinstance(v[0], dict) and "role" in v[0]
    return False


def is_conversational_from_value(example: dict[str, Any]) -> bool:
    v = example.get("conversations")
    return isinstance(v, list) and len(v) > 0 and isinstance(v[0], dict) and "from" in v[0] and "value" in v[0]


def maybe_convert_to_chatml(example: dict[str, list]) -> dict[str, list]:
    """``from/value`` turns become ``role/content``; a ``conversations`` column is renamed ``messages``."""
    example = dict(example)
    for key in ("prompt", "completion", "chosen", "rejected", "messages", "conversations"):
        turns = example.get(key)
        if isinstance(turns, list):
            new = []
            for t in turns:
                if isinstance(t, dict) and "from" in t and "value" in t:
                    t = {**{k: v for k, v in t.items() if k not in ("from", "value")}, "role": t["from"], "content": t["value"]}
                new.append(t)
            example[key] = new
    if "conversations" in example:
        example["messages"] = example.pop("conversations")
    return example


def get_dataset_column_names(dataset) -> list[str]:
    if getattr(dataset, "column_names", None) is not None:
        return list(dataset.column_names)
    return list(next(iter(dataset)).keys())


# ---------------------------------------------------------------------------
# chat templates
# ---------------------------------------------------------------------------
def _common_prefix(a: str, b: str) -> str:
    n = min(len(a), len(b))
    i = 0
    while i < n and a[i] == b[i]:
        i += 1
    return a[:i]


def apply_chat_template(example: dict, processing_class, tools: list | None = None, **template_kwargs) -> dict[str, str]:
    tools = tools or None
    keys = {k for k in example if k in ("prompt", "chosen", "rejected", "completion", "messages", "label")}
    if keys not in _TEMPLATE_KEYSETS:
        raise KeyError(f"Invalid keys in the example: {keys}")
    kw = {**example.get("chat_template_kwargs", {}), **template_kwargs}
    render = lambda msgs, **extra: processing_class.apply_chat_template(msgs, tools=tools, tokenize=False, **extra, **kw)
    out: dict[str, Any] = {}
    if "messages" in example:
        out["text"] = render(example["messages"])
    if "prompt" in example:
        last = example["prompt"][-1]["role"]
        if last in ("user", "tool"):
            prompt = render(example["prompt"], add_generation_prompt=True, continue_final_message=False)
        elif last == "assistant":
            prompt = render(example["prompt"], add_generation_prompt=False, continue_final_message=True)
        else:
            raise ValueError(f"Invalid role in the last message: {last}")
        full = {}
        for k in ("chosen", "rejected", "completion"):
            if k in example:
                full[k] = render(example["prompt"] + example[k])
                # some templates alter the generation prompt once an answer follows:
                # keep only what both renderings share
                prompt = _common_prefix(prompt, full[k])
        out["prompt"] = prompt
        for k, v in full.items():
            out[k] = v[len(prompt):]
    else:
        for k in ("chosen", "rejected"):
            if k in example:
                out[k] = render(example[k])
    if "label" in example:
        out["label"] = example["label"]
    return out


def maybe_apply_chat_template(example: dict, tokenizer, tools: list | None = None, **template_kwargs) -> dict:
    if is_conversational(example):
        return apply_chat_template(example, tokenizer, tools, **template_kwargs)
    return example


def _tokenize(processing_class, inp, **kw):
    """Conversation -> ``apply_chat_template(tokenize=True, return_dict=True)``; text -> ``__call__``."""
    if isinstance(inp, list):
        out = processing_class.apply_chat_template(inp, tokenize=True, return_dict=True, **kw)
    else:
        out = processing_class(text=inp)
    ids = out["input_ids"]
    if len(ids) > 0 and isinstance(ids[0], (list, tuple)) and len(ids) == 1:  # VLM processors add a batch dim
        out = {k: (v[0] if isinstance(v, (list, tuple)) and len(v) == 1 else v) for k, v in out.items()}
    return dict(out)


# ---------------------------------------------------------------------------
# preference datasets
# ---------------------------------------------------------------------------
def _map(dataset, fn, batched=False, remove_columns=None, **kw):
    if Dataset is not None and isinstance(dataset, (Dataset, DatasetDict, IterableDataset)):
        if isinstance(dataset, IterableDataset):
            kw.pop("num_proc", None)
            kw.pop("desc", None)
        return dataset.map(fn, batched=batched, remove_columns=remove_columns, **kw)
    rows = list(dataset)
    if batched:
        cols = {k: [r[k] for r in rows] for k in rows[0]} if rows else {}
        res = fn(cols)
        n = len(next(iter(res.values()))) if res else 0
        return [{k: v[i] for k, v in res.items()} for i in range(n)]
    out = []
    for r in rows:
        nr = {**r, **fn(r)}
        for c in remove_columns or []:
            nr.pop(c, None)
        out.append(nr)
    return out


def _unpair_batch(batch: dict[str, list]) -> dict[str, list]:
    n = len(batch["chosen"])
    res = {"completion": list(batch["chosen"]) + list(batch["rejected"]), "label": [True] * n + [False] * n}
    for name, col in batch.items():  # the prompt and every extra column ride along with both halves
        if name not in ("chosen", "rejected"):
            res[name] = list(col) * 2
    return res


def unpair_preference_dataset(dataset, num_proc: int | None = None, desc: str | None = None):
    """(prompt, chosen, rejected) rows -> twice as many (prompt, completion, label) rows."""
    kw = {}
    if Dataset is not None and isinstance(dataset, (Dataset, DatasetDict)):
        kw = dict(num_proc=num_proc, desc=desc)
    return _map(dataset, _unpair_batch, batched=True, remove_columns=["chosen", "rejected"], **kw)


def maybe_unpair_preference_dataset(dataset, num_proc: int | None = None, desc: str | None = None):
    cols = get_dataset_column_names(dataset[next(iter(dataset))] if isinstance(dataset, dict) else dataset)
    if "chosen" in cols and "rejected" in cols:
        return unpair_preference_dataset(dataset, num_proc, desc)
    return dataset


def extract_prompt(example: dict[str, Sequence]) -> dict[str, Sequence]:
    """Split the longest shared prefix of ``chosen`` / ``rejected`` off as the prompt."""
    ch, rj = example["chosen"], example["rejected"]
    n = min(len(ch), len(rj))
    idx = n
    for i in range(n):
        if ch[i] != rj[i]:
            idx = i
            if isinstance(ch, str) and i > 0 and ch[i - 1] == " ":
                idx = i - 1  # keep the separating space with the completions
            break
    return {"prompt": ch[:idx], "chosen": ch[idx:], "rejected": rj[idx:]}


def maybe_extract_prompt(example: dict[str, list]) -> dict[str, list]:
    if "chosen" not in example or "rejected" not in example:
        return example
    if "prompt" in example:
        cp = is_conversational({"chosen": example["chosen"]})
        pp = is_conversational({"prompt": example["prompt"]})
        if cp == pp:  # prompt already separate
            return example
    return {**example, **extract_prompt({"chosen": example["chosen"], "rejected": example["rejected"]})}


# ---------------------------------------------------------------------------
# packing
# ---------------------------------------------------------------------------
class _SegmentTree:
    """Max-tree over capacities 1..maxval; ``search(v)`` = smallest stored capacity >= v (0 if none)."""

    def __init__(self, maxval: int):
        self.maxval = maxval
        self.size = 1
        while self.size < maxval:
            self.size *= 2
        self.tree = [0] * (2 * self.size)

    def _set(self, val, present):
        i = self.size + val - 1
        self.tree[i] = val if present else 0
        i //= 2
        while i >= 1:
            self.tree[i] = max(self.tree[2 * i], self.tree[2 * i + 1])
            i //= 2

    def add(self, val):
        assert 0 < val <= self.maxval
        self._set(val, True)

    def remove(self, val):
        assert 0 < val <= self.maxval
        self._set(val, False)

    def search(self, val):
        assert 0 < val <= self.maxval
        i = 1
        while i < self.size:
            if self.tree[2 * i] >= val:
                i = 2 * i
            else:
                i = 2 * i + 1
        return self.tree[i]


def bfd_assign(lengths: Sequence[int], seq_length: int) -> list[list[int]]:
    """Best-fit-decreasing: returns bins as lists of item indices (items sorted by length desc, stable)."""
    try:
        from ._native import host_runtime

        hr = host_runtime()
        if hr is not None:
            return hr.bfd_assign(lengths, seq_length)
    except Exception:
        pass
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    tree = _SegmentTree(seq_length)
    tree.add(seq_length)
    space_to_bins: dict[int, list] = defaultdict(list)
    bins: list[dict] = []
    for i in order:
        L = lengths[i]
        space = tree.search(L)
        if space < seq_length:
            b = space_to_bins[space].pop(0)
        else:
            b = {"ids": [], "space": seq_length}
            bins.append(b)
        b["ids"].append(i)
        if space < seq_length and not space_to_bins[space]:
            tree.remove(space)
        b["space"] -= L
        if b["space"] > 0:
            if not space_to_bins[b["space"]]:
                tree.add(b["space"])
            space_to_bins[b["space"]].append(b)
    return [b["ids"] for b in bins]


def _pack_columns(columns: dict[str, list], seq_length: int, strategy: str) -> dict[str, list]:
    names = [k for k, v in columns.items() if len(v) and isinstance(v[0], (list, tuple, np.ndarray))]
    if not names:
        return columns
    key = "input_ids" if "input_ids" in names else names[0]
    if strategy == "wrapped":
        out = {}
        for k in names:
            flat = [x for row in columns[k] for x in row]
            out[k] = [flat[i:i + seq_length] for i in range(0, len(flat), seq_length)]
        return out
    # build fragments (row, start, end)
    frags = []
    for r, row in enumerate(columns[key]):
        n = len(row)
        if n == 0:
            continue
        if strategy == "bfd_split":
            for s in range(0, n, seq_length):
                frags.append((r, s, min(n, s + seq_length)))
        else:
            frags.append((r, 0, min(n, seq_length)))
    bins = bfd_assign([e - s for _, s, e in frags], seq_length)
    out = {k: [] for k in names}
    out["seq_lengths"] = []
    for b in bins:
        for k in names:
            row = []
            for j in b:
                r, s, e = frags[j]
                row.extend(columns[k][r][s:e])
            out[k].append(row)
        out["seq_lengths"].append([frags[j][2] - frags[j][1] for j in b])
    return out


def pack_dataset(dataset, seq_length: int, strategy: str = "bfd", map_kwargs: dict | None = None):
    """Pack tokenised rows into rows of at most ``seq_length`` tokens.

    ``bfd`` truncates over-long rows, ``bfd_split`` re-queues the overflow as new
    fragments, ``wrapped`` concatenates everything and cuts every ``seq_length``.
    ``bfd*`` add a ``seq_lengths`` column with the document boundaries."""
    if strategy == "bfd-requeue":
        strategy = "bfd_split"
    if strategy not in ("bfd", "bfd_split", "wrapped"):
        raise ValueError(f"Invalid packing strategy: {strategy}. Use 'bfd', 'bfd_split' or 'wrapped'.")
    fn = lambda batch: _pack_columns({k: list(v) for k, v in batch.items()}, seq_length, strategy)
    if Dataset is not None and isinstance(dataset, (Dataset, DatasetDict)):
        kw = dict(map_kwargs or {})
        fmt = dataset.format if isinstance(dataset, Dataset) else None
        ds = dataset.with_format(None) if isinstance(dataset, Dataset) else dataset
        cols = ds.column_names if isinstance(dataset, Dataset) else None
        ds = ds.map(fn, batched=True, batch_size=kw.pop("batch_size", None) or len(ds) if isinstance(dataset, Dataset) else 1000,
                    remove_columns=cols, **kw)
        if fmt is not None and fmt.get("type") is not None:
            columns = fmt.get("columns")
            if columns is not None and "seq_lengths" in ds.column_names and "seq_lengths" not in columns:
                columns = list(columns) + ["seq_lengths"]
            ds = ds.with_format(fmt["type"], columns=columns, **(fmt.get("format_kwargs") or {}))
        return ds
    if Dataset is not None and isinstance(dataset, IterableDataset):
        return dataset.map(fn, batched=True, remove_columns=get_dataset_column_names(dataset))
    rows = list(dataset)
    if not rows:
        return rows
    res = _pack_columns({k: [r[k] for r in rows] for k in rows[0]}, seq_length, strategy)
    n = len(next(iter(res.values())))
    return [{k: v[i] for k, v in res.items()} for i in range(n)]


def truncate_dataset(dataset, max_length: int, map_kwargs: dict | None = None):
    def trunc(batch):
        return {k: ([x[:max_length] if isinstance(x, (list, tuple)) else x for x in v]) for k, v in batch.items()}
    return _map(dataset, trunc, batched=True, **(map_kwargs or {}))
