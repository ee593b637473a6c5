"""Chat-template helpers (names and results of trl/chat_template_utils.py).

``has_generation_markers`` :37, ``clone_chat_template`` :45, ``add_response_schema`` :593,
``supports_tool_calling`` :686, ``is_chat_template_prefix_preserving`` :752,
``is_chat_template_stop_token_trained`` :813, ``get_training_chat_template`` :947,
``parse_response`` :1143.
"""
from __future__ import annotations

import json
import os
import re
from typing import Any

_TEMPLATE_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "chat_templates")


def has_generation_markers(chat_template: str | None) -> bool:
    return bool(chat_template) and "{% generation %}" in chat_template.replace("{%-", "{%").replace("-%}", "%}")


def clone_chat_template(model, tokenizer, source_tokenizer_path, resize_to_multiple_of: int | None = 64):
    """Copy chat template, EOS and the special tokens it needs from another tokenizer, then grow the
    embeddings (to a multiple of 64 by default, padding the vocabulary with dummy tokens).
    Returns ``(model, tokenizer, added_token_ids)``."""
    from transformers import AutoTokenizer

    src = source_tokenizer_path if not isinstance(source_tokenizer_path, str) else AutoTokenizer.from_pretrained(source_tokenizer_path)
    tokenizer.chat_template = src.get_chat_template() if hasattr(src, "get_chat_template") else src.chat_template
    before = len(tokenizer)
    added = [t for t in src.added_tokens_decoder.values()] if hasattr(src, "added_tokens_decoder") else []
    if added:
        tokenizer.add_tokens(added)
    tokenizer.eos_token = src.eos_token
    if getattr(model, "config", None) is not None:
        model.config.eos_token_id = tokenizer.eos_token_id
    if getattr(model, "generation_config", None) is not None:
        model.generation_config.eos_token_id = tokenizer.eos_token_id
    n = len(tokenizer)
    if resize_to_multiple_of:
        target = (max(n, model.config.vocab_size) + resize_to_multiple_of - 1) // resize_to_multiple_of * resize_to_multiple_of
    else:
        target = max(n, model.config.vocab_size)
    model.resize_token_embeddings(target)
    if target > len(tokenizer):
        tokenizer.add_tokens([f"<extra_id_{i}>" for i in range(target - len(tokenizer))])
    return model, tokenizer, list(range(before, len(tokenizer)))


_FAMILY_MARKERS = [  # first match wins: more specific markers first
    ("<think>", "<|im_start|>", "qwen3_training.jinja"),
    ("You are Qwen, created by Alibaba Cloud", "<|im_start|>", "qwen2_5_training.jinja"),
    ("<|im_start|>", None, "chatml_training.jinja"),
    ("<|start_header_id|>", None, "llama3_training.jinja"),
    ("<start_of_turn>", "tool_code", "gemma3_training.jinja"),
    ("<start_of_turn>", None, "gemma_training.jinja"),
    ("[gMASK]", "<|assistant|>", "glm4moe_training.jinja"),
    ("<|START_OF_TURN_TOKEN|>", None, "cohere_training.jinja"),
    ("<|start|>", "<|message|>", "gptoss_training.jinja"),
    ("<|assistant|>", None, "phi3_training.jinja"),
    ("<｜Assistant｜>", None, "deepseekv3_training.jinja"),
    ("<end_of_utterance>", None, "idefics3_training.jinja"),
    ("[INST]", None, "mistral_training.jinja"),
    ("USER:", "ASSISTANT:", "llava_training.jinja"),
]


def get_training_chat_template(tokenizer) -> str | None:
    """A template that renders the family's chat format *and* is usable for training: assistant turns inside
    ``{% generation %}`` markers, prefix preserving, tool-call arguments as dicts or strings.  Returns ``None``
    when the tokenizer's own template already qualifies; raises for unknown families."""
    tpl = getattr(tokenizer, "chat_template", None) or ""
    if has_generation_markers(tpl) and is_chat_template_prefix_preserving(tokenizer):
        return None
    for a, b, fn in _FAMILY_MARKERS:
        if a in tpl and (b is None or b in tpl):
            with open(os.path.join(_TEMPLATE_DIR, fn), encoding="utf-8") as f:
                return f.read()
    raise ValueError("The tokenizer's chat template does not match a known family (ChatML/Qwen, Qwen3, Llama 3, Gemma, "
                     "GLM-4, Command-R, gpt-oss, Phi-3, DeepSeek-V3, Idefics3 / SmolVLM, Mistral [INST], LLaVA-1.5); pass a training template with {% generation %} markers explicitly.")


def _render(tok, messages, **kw):
    return tok.apply_chat_template(messages, tokenize=False, **kw)


def supports_tool_calling(processing_class) -> bool:
    """True when a user -> assistant(tool_calls) -> tool conversation renders and keeps the tool name, the
    argument key and value, and the tool result."""
    if getattr(processing_class, "chat_template", None) is None:
        return False
    name, key, val, content = "tool_name_3f9a", "tool_arg_key_7c21", "tool_arg_val_e05b", "tool_content_91dd"
    calls = [{"type": "function", "function": {"name": name, "arguments": {key: val}}}]
    msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "", "tool_calls": calls},
            {"role": "tool", "name": name, "content": content}]
    try:
        from jinja2.exceptions import TemplateError
    except Exception:  # pragma: no cover
        TemplateError = Exception
    try:
        out = _render(processing_class, msgs)
    except TemplateError:
        return False
    except TypeError:
        calls[0]["function"]["arguments"] = json.dumps({key: val})
        try:
            out = _render(processing_class, msgs)
        except TemplateError:
            return False
    return all(s in out for s in (name, key, val, content))


def is_chat_template_prefix_preserving(processing_class) -> bool:
    """Earlier messages render the same whatever follows (checked on a plain and a tool conversation)."""
    m1 = [{"role": "user", "content": "What color is the sky?"}, {"role": "assistant", "content": "It is blue."}]
    m2 = m1 + [{"role": "user", "content": "And at night?"}]
    try:
        a, b = _render(processing_class, m1), _render(processing_class, m2)
    except Exception:
        return False
    if not b.startswith(a):
        return False
    calls = [{"type": "function", "function": {"name": "f", "arguments": {"x": 1}}}]
    t1 = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "", "tool_calls": calls}]
    t2 = t1 + [{"role": "tool", "name": "f", "content": "1"}]
    try:
        a, b = _render(processing_class, t1), _render(processing_class, t2)
    except Exception:
        return True  # no tool support: the plain check decides
    return b.startswith(a)


def is_chat_template_stop_token_trained(processing_class) -> bool:
    """True when the assistant span marked by ``{% generation %}`` ends with the tokenizer's EOS token,
    i.e. assistant-only loss teaches the model to stop."""
    tok = processing_class
    if not has_generation_markers(getattr(tok, "chat_template", None)):
        return False
    msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"}]
    out = tok.apply_chat_template(msgs, tokenize=True, return_dict=True, return_assistant_tokens_mask=True)
    ids, mask = out["input_ids"], out["assistant_masks"]
    if ids and isinstance(ids[0], list):
        ids, mask = ids[0], mask[0]
    last = max((i for i, m in enumerate(mask) if m), default=None)
    return last is not None and ids[last] == tok.eos_token_id


_DEFAULT_SCHEMA = {
    "type": "object",
    "properties": {
        "role": {"const": "assistant"},
        "content": {"type": "string", "x-regex": r"^(.*?)(?:<tool_call>|$)"},
        "tool_calls": {
            "type": "array", "x-regex-iterator": r"<tool_call>\s*(.+?)\s*</tool_call>",
            "items": {"x-parser": "json", "x-parser-args": {"transform": "{type: 'function', function: @}"},
                      "type": "object"},
        },
    },
}


def add_response_schema(processing_class):
    """Attach a response schema describing how to parse the family's tool-call syntax back into a message."""
    tpl = getattr(processing_class, "chat_template", "") or ""
    if "<tool_call>" not in tpl and "tool_call" not in tpl:
        raise ValueError("Unrecognized chat template: no tool-call syntax to derive a response schema from.")
    processing_class.response_schema = _DEFAULT_SCHEMA
    return processing_class


_TOOL_CALL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.DOTALL)


def parse_response(processing_class, ids_or_text) -> dict[str, Any]:
    """Decode one completion into an assistant message.  ``<tool_call>{json}</tool_call>`` blocks become
    ``tool_calls``; malformed JSON falls back to plain text content."""
    text = ids_or_text if isinstance(ids_or_text, str) else processing_class.decode(ids_or_text, skip_special_tokens=False)
    for t in (getattr(processing_class, "eos_token", None), getattr(processing_class, "pad_token", None)):
        if t:
            text = text.replace(t, "")
    calls = []
    for m in _TOOL_CALL.finditer(text):
        try:
            obj = json.loads(m.group(1))
            if "name" not in obj:
                raise ValueError
            calls.append({"type": "function", "function": {"name": obj["name"], "arguments": obj.get("arguments", {})}})
        except (json.JSONDecodeError, ValueError):
            return {"role": "assistant", "content": text}
    msg: dict[str, Any] = {"role": "assistant", "content": _TOOL_CALL.sub("", text).strip() if calls else text}
    think = re.match(r"\s*<think>(.*?)</think>\s*(.*)$", msg["content"], re.DOTALL)
    if think:
        msg["reasoning_content"], msg["content"] = think.group(1).strip(), think.group(2)
    if calls:
        msg["tool_calls"] = calls
    return msg
