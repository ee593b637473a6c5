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


# Family registry.  A tokenizer's own template is matched on the special tokens / phrases it contains (``all_of``
# present, ``none_of`` absent); the first match wins, so more specific entries come first.  ``calls`` names the
# tool-call syntax the family's completions use (see ``_PARSERS``).
_FAMILIES = [
    # name, all_of, none_of, training template, tool-call syntax
    ("nemotron_3_ultra", ("<|im_start|>", "<function=", "<name>", "ultra"), (), "nemotron_3_ultra_training.jinja", "xml"),
    ("nemotron_3_super", ("<|im_start|>", "<function=", "<name>", "super"), (), "nemotron_3_super_training.jinja", "xml"),
    ("nemotron_3_nano", ("<|im_start|>", "<function=", "<name>"), (), "nemotron_3_nano_training.jinja", "xml"),
    ("qwen3_6", ("<|im_start|>", "<function=", "preserve_thinking"), (), "qwen3_6_training.jinja", "xml"),
    ("qwen3_5_think", ("<|im_start|>", "<function=", "enable_thinking"), (), "qwen3_5_think_training.jinja", "xml"),
    ("qwen3_5_nothink", ("<|im_start|>", "<function="), (), "qwen3_5_nothink_training.jinja", "xml"),
    ("qwen2_5_vl", ("<|im_start|>", "<|vision_start|>", "You are a helpful assistant"), (), "qwen2_5_vl_training.jinja", "json"),
    ("qwen3_vl", ("<|im_start|>", "<|vision_start|>"), (), "qwen3_vl_training.jinja", "json"),
    ("qwen3", ("<think>", "<|im_start|>"), (), "qwen3_training.jinja", "json"),
    ("qwen2_5", ("You are Qwen, created by Alibaba Cloud", "<|im_start|>"), (), "qwen2_5_training.jinja", "json"),
    ("lfm2_2_5", ("<|im_start|>", "<|tool_list_start|>", "keep_past_thinking"), (), "lfm2_2_5_training.jinja", "pythonic"),
    ("lfm2", ("<|im_start|>", "<|tool_list_start|>"), (), "lfm2_training.jinja", "pythonic"),
    ("qwen3_instruct_2507", ("<|im_start|>", "<tool_call>"), ("<think>",), "qwen3_instruct_2507_training.jinja", "json"),
    ("chatml", ("<|im_start|>",), (), "chatml_training.jinja", "json"),
    ("llama3_2", ("<|start_header_id|>", "Cutting Knowledge Date", "strftime_now"), (), "llama3_2_training.jinja", "llama"),
    ("llama3_1", ("<|start_header_id|>", "Cutting Knowledge Date"), (), "llama3_1_training.jinja", "llama"),
    ("llama3", ("<|start_header_id|>",), (), "llama3_training.jinja", "llama"),
    ("diffusion_gemma", ("<|turn>",), (), "diffusion_gemma_training.jinja", "gemma_call"),
    ("gemma3", ("<start_of_turn>", "tool_code"), (), "gemma3_training.jinja", "tool_code"),
    ("gemma", ("<start_of_turn>",), (), "gemma_training.jinja", "json"),
    ("glm4moe", ("[gMASK]", "<|assistant|>"), (), "glm4moe_training.jinja", "glm"),
    ("cohere2", ("<|START_OF_TURN_TOKEN|>", "<|START_RESPONSE|>"), (), "cohere2_training.jinja", "cohere_action"),
    ("cohere", ("<|START_OF_TURN_TOKEN|>",), (), "cohere_training.jinja", "cohere_json"),
    ("gptoss", ("<|start|>", "<|message|>"), (), "gptoss_training.jinja", "harmony"),
    ("phi3_5", ("<|assistant|>", "<|end|>", "eos_token"), (), "phi3_5_training.jinja", "llama"),
    ("phi3", ("<|assistant|>",), (), "phi3_training.jinja", "json"),
    ("deepseekv3", ("<｜Assistant｜>",), (), "deepseekv3_training.jinja", "json"),
    ("idefics3", ("<end_of_utterance>",), (), "idefics3_training.jinja", "json"),
    ("llava_next", ("[INST]", "<image>"), (), "llava_next_training.jinja", "json"),
    ("mistral", ("[INST]",), (), "mistral_training.jinja", "mistral"),
    ("llava", ("USER:", "ASSISTANT:"), (), "llava_training.jinja", "json"),
]


def detect_chat_family(processing_class_or_template) -> tuple[str, str, str] | None:
    """``(family, training template file, tool-call syntax)`` for a tokenizer (or a template string), or None."""
    tpl = processing_class_or_template if isinstance(processing_class_or_template, str) else (
        getattr(processing_class_or_template, "chat_template", None) or "")
    if isinstance(tpl, dict):  # named templates: the default one decides
        tpl = tpl.get("default", "") or next(iter(tpl.values()), "")
    for name, all_of, none_of, fn, calls in _FAMILIES:
        if all(m in tpl for m in all_of) and not any(m in tpl for m in none_of):
            return name, fn, calls
    return None


def list_chat_families() -> list[str]:
    return [f[0] for f in _FAMILIES]


def get_training_chat_template(tokenizer, family: str | None = None) -> str | None:
    """A template that renders the family's chat format *and* is usable for training: assistant turns inside
    ``{% generation %}`` markers, prefix preserving, tool-call arguments as dicts or strings.  Returns ``None``
    when the tokenizer's own template already qualifies; raises for unknown families.  ``family`` names an entry of
    :func:`list_chat_families` to bypass the detection (e.g. ``"nemotron_3_super"``)."""
    if family is not None:
        for name, _, _, fn, _ in _FAMILIES:
            if name == family:
                with open(os.path.join(_TEMPLATE_DIR, fn), encoding="utf-8") as f:
                    return f.read()
        raise ValueError(f"unknown chat family {family!r}; known: {', '.join(list_chat_families())}")
    tpl = getattr(tokenizer, "chat_template", None) or ""
    if has_generation_markers(tpl) and is_chat_template_prefix_preserving(tokenizer):
        return None
    hit = detect_chat_family(tokenizer)
    if hit is not None:
        with open(os.path.join(_TEMPLATE_DIR, hit[1]), encoding="utf-8") as f:
            return f.read()
    raise ValueError("The tokenizer's chat template does not match a known family (" + ", ".join(list_chat_families()) +
                     "); pass a training template with {% generation %} markers explicitly.")


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


# ---- response parsing --------------------------------------------------------------------------------------------------
# One parser per tool-call syntax.  Each takes the completion text (special end tokens already removed) and returns
# ``(content, tool_calls)`` or raises ValueError when a call block is malformed (the caller then keeps plain text).
def _call(name, arguments):
    return {"type": "function", "function": {"name": name, "arguments": arguments}}


def _loads_or_str(text: str):
    try:
        return json.loads(text)
    except (json.JSONDecodeError, ValueError):
        return text


_RE_JSON_CALL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.DOTALL)
_RE_XML_CALL = re.compile(r"<tool_call>\s*<function=([^>\n]+)>(.*?)</function>\s*</tool_call>", re.DOTALL)
_RE_XML_PARAM = re.compile(r"<parameter=([^>\n]+)>\n?(.*?)\n?</parameter>", re.DOTALL)
_RE_GLM_CALL = re.compile(r"<tool_call>\s*([^\n<]+)\s*(.*?)</tool_call>", re.DOTALL)
_RE_GLM_ARG = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.DOTALL)
_RE_HARMONY_CALL = re.compile(r"to=functions\.([\w.\-]+).*?<\|message\|>(.*?)(?:<\|call\|>|$)", re.DOTALL)
_RE_HARMONY_FINAL = re.compile(r"<\|channel\|>final<\|message\|>(.*?)(?:<\|return\|>|<\|end\|>|$)", re.DOTALL)
_RE_HARMONY_THINK = re.compile(r"<\|channel\|>analysis<\|message\|>(.*?)(?:<\|end\|>|$)", re.DOTALL)
_RE_PY_BLOCK = re.compile(r"<\|tool_call_start\|>\s*\[(.*?)\]\s*<\|tool_call_end\|>", re.DOTALL)
_RE_ACTION = re.compile(r"<\|START_ACTION\|>(.*?)<\|END_ACTION\|>", re.DOTALL)
_RE_GEMMA_CALL = re.compile(r"<\|tool_call>call:([\w.\-]+)\{(.*?)\}<tool_call\|>", re.DOTALL)


def _parse_json_calls(text):
    calls = []
    for m in _RE_JSON_CALL.finditer(text):
        obj = json.loads(m.group(1))
        if "name" not in obj:
            raise ValueError("tool call without a name")
        calls.append(_call(obj["name"], obj.get("arguments", obj.get("parameters", {}))))
    return (_RE_JSON_CALL.sub("", text).strip() if calls else text), calls


def _parse_xml_calls(text):
    calls = []
    for m in _RE_XML_CALL.finditer(text):
        args = {k.strip(): _loads_or_str(v) for k, v in _RE_XML_PARAM.findall(m.group(2))}
        calls.append(_call(m.group(1).strip(), args))
    if "<tool_call>" in text and not calls:
        raise ValueError("malformed <function=...> block")
    return (_RE_XML_CALL.sub("", text).strip() if calls else text), calls


_RE_HEADER = re.compile(r"^\s*(?:<\|start_header_id\|>assistant<\|end_header_id\|>|<\|assistant\|>)\s*")


def _parse_llama_call(text):
    """The whole turn is one JSON object {"name": ..., "parameters" | "arguments": ...} (Llama 3.x, Phi)."""
    body = _RE_HEADER.sub("", text).strip()
    if body.startswith("<|python_tag|>"):
        body = body[len("<|python_tag|>"):]
    if not (body.startswith("{") and body.endswith("}")):
        return text, []
    obj = json.loads(body)
    if "name" not in obj:
        return text, []
    return "", [_call(obj["name"], obj.get("parameters", obj.get("arguments", {})))]


def _parse_glm_calls(text):
    calls = []
    for m in _RE_GLM_CALL.finditer(text):
        calls.append(_call(m.group(1).strip(), {k.strip(): _loads_or_str(v.strip()) for k, v in _RE_GLM_ARG.findall(m.group(2))}))
    return (_RE_GLM_CALL.sub("", text).strip() if calls else text), calls


def _parse_harmony(text):
    calls = [_call(n, _loads_or_str(b.strip())) for n, b in _RE_HARMONY_CALL.findall(text)]
    final = _RE_HARMONY_FINAL.search(text)
    content = final.group(1) if final else ("" if calls else text)
    return content, calls


def _parse_pythonic(text):
    import ast

    calls = []
    for m in _RE_PY_BLOCK.finditer(text):
        tree = ast.parse("[" + m.group(1) + "]", mode="eval")
        for node in tree.body.elts:
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Name)):
                raise ValueError("not a function call")
            calls.append(_call(node.func.id, {kw.arg: ast.literal_eval(kw.value) for kw in node.keywords}))
    return (_RE_PY_BLOCK.sub("", text).strip() if calls else text), calls


_RE_TOOL_CODE = re.compile(r"```tool_code\s*(.*?)\s*```", re.DOTALL)
_RE_COHERE_JSON = re.compile(r"Action:\s*```json\s*(.*?)\s*```", re.DOTALL)


def _parse_tool_code(text):
    import ast

    calls = []
    for m in _RE_TOOL_CODE.finditer(text):
        node = ast.parse(m.group(1).strip(), mode="eval").body
        if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Name)):
            raise ValueError("not a function call")
        calls.append(_call(node.func.id, {kw.arg: ast.literal_eval(kw.value) for kw in node.keywords}))
    return (_RE_TOOL_CODE.sub("", text).strip() if calls else text), calls


def _parse_cohere_json(text):
    calls = []
    for m in _RE_COHERE_JSON.finditer(text):
        for item in json.loads(m.group(1)):
            calls.append(_call(item["tool_name"], item.get("parameters", {})))
    return (_RE_COHERE_JSON.sub("", text).strip() if calls else text), calls


def _parse_cohere_action(text):
    calls = []
    for m in _RE_ACTION.finditer(text):
        for item in json.loads(m.group(1)):
            calls.append(_call(item["tool_name"], item.get("parameters", {})))
    content = re.sub(r"<\|START_RESPONSE\|>|<\|END_RESPONSE\|>", "", _RE_ACTION.sub("", text))
    content = re.sub(r"<\|START_THINKING\|>.*?<\|END_THINKING\|>", "", content, flags=re.DOTALL)
    return content.strip() if calls else content, calls


def _parse_gemma_calls(text):
    def value(tok):
        tok = tok.strip()
        if tok.startswith('<|"|>') and tok.endswith('<|"|>'):
            return tok[5:-5]
        return _loads_or_str(tok)

    calls = []
    for m in _RE_GEMMA_CALL.finditer(text):
        args, depth, key, cur = {}, 0, None, ""
        for part in re.split(r'(<\|"\|>.*?<\|"\|>|[:,{}\[\]])', m.group(2)):
            if part in ("{", "["):
                depth += 1
            elif part in ("}", "]"):
                depth -= 1
            if depth == 0 and part == ":" and key is None:
                key, cur = cur.strip(), ""
            elif depth == 0 and part == ",":
                args[key], key, cur = value(cur), None, ""
            else:
                cur += part
        if key is not None:
            args[key] = value(cur)
        calls.append(_call(m.group(1), args))
    return (_RE_GEMMA_CALL.sub("", text).strip() if calls else text), calls


def _parse_mistral_calls(text):
    if "[TOOL_CALLS]" not in text:
        return text, []
    head, _, tail = text.partition("[TOOL_CALLS]")
    items = json.loads(tail.strip())
    return head.strip(), [_call(i["name"], i.get("arguments", {})) for i in items]


_PARSERS = {"json": _parse_json_calls, "xml": _parse_xml_calls, "llama": _parse_llama_call, "glm": _parse_glm_calls,
            "harmony": _parse_harmony, "pythonic": _parse_pythonic, "cohere_action": _parse_cohere_action,
            "gemma_call": _parse_gemma_calls, "mistral": _parse_mistral_calls, "tool_code": _parse_tool_code,
            "cohere_json": _parse_cohere_json}

# Declarative schemas (transformers' response-schema vocabulary) for the syntaxes a regex schema can express.
_SCHEMAS = {
    "json": {
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
    },
    "xml": {
        "type": "object",
        "properties": {
            "role": {"const": "assistant"},
            "reasoning_content": {"type": "string", "x-regex": r"<think>\s*(.*?)\s*</think>"},
            "content": {"type": "string", "x-regex": r"(?:</think>\s*)?(.*?)(?:<tool_call>|$)"},
            "tool_calls": {
                "type": "array", "x-regex-iterator": r"<tool_call>\s*(<function=.+?</function>)\s*</tool_call>",
                "items": {"type": "object", "properties": {
                    "type": {"const": "function"},
                    "function": {"type": "object", "properties": {
                        "name": {"type": "string", "x-regex": r"<function=([^>\n]+)>"},
                        "arguments": {"type": "object", "x-regex-key-value": r"<parameter=(?P<key>[^>\n]+)>\n?(?P<value>.*?)\n?</parameter>",
                                      "additionalProperties": {"x-parser": "json", "x-parser-args": {"allow_non_json": True}}},
                    }},
                }},
            },
        },
    },
}


def add_response_schema(processing_class, family: str | None = None):
    """Records on the tokenizer how its family writes tool calls, so that :func:`parse_response` (and transformers'
    own ``parse_response`` for the syntaxes a regex schema can express) turns a completion back into a message.
    Sets ``response_family`` / ``response_syntax`` always and ``response_schema`` where a declarative schema exists.
    For a processor the inner tokenizer gets the attributes too (trl/chat_template_utils.py:593-686)."""
    hit = None
    if family is not None:
        hit = next(((n, fn, c) for n, _, _, fn, c in _FAMILIES if n == family), None)
    else:
        hit = detect_chat_family(processing_class)
    tpl = getattr(processing_class, "chat_template", "") or ""
    if hit is None or (hit[2] == "json" and family is None and "tool_call" not in str(tpl)):
        raise ValueError("Unrecognized chat template: no tool-call syntax to derive a response schema from.")
    targets = [processing_class]
    inner = getattr(processing_class, "tokenizer", None)
    if inner is not None:
        targets.append(inner)
    for t in targets:
        t.response_family, t.response_syntax = hit[0], hit[2]
        if hit[2] in _SCHEMAS:
            t.response_schema = _SCHEMAS[hit[2]]
    return processing_class


_RE_THINK = re.compile(r"\s*(?:<think>)?(.*?)</think>\s*(.*)$", re.DOTALL)


def parse_response(processing_class, ids_or_text) -> dict[str, Any]:
    """Decode one completion into an assistant message.  The tool-call syntax is the one recorded by
    :func:`add_response_schema`, else the one detected from the chat template, else ``<tool_call>{json}</tool_call>``.
    Reasoning between ``<think>`` tags (or the harmony analysis channel) becomes ``reasoning_content``.  A malformed
    call block falls back to plain text content (trl/chat_template_utils.py:1143-1210)."""
    text = ids_or_text if isinstance(ids_or_text, str) else processing_class.decode(ids_or_text, skip_special_tokens=False)
    for t in (getattr(processing_class, "eos_token", None), getattr(processing_class, "pad_token", None), "<|im_end|>",
              "<|eot_id|>", "<|END_OF_TURN_TOKEN|>", "<turn|>", "<|end|>"):
        if t and t != "<|end|>" or (t == "<|end|>" and "<|channel|>" not in text):
            text = text.replace(t, "")
    syntax = getattr(processing_class, "response_syntax", None)
    if syntax is None:
        hit = detect_chat_family(processing_class)
        syntax = hit[2] if hit else "json"
    try:
        content, calls = _PARSERS[syntax](text)
    except (json.JSONDecodeError, ValueError, KeyError, SyntaxError, TypeError):
        return {"role": "assistant", "content": text}
    msg: dict[str, Any] = {"role": "assistant", "content": content}
    if syntax == "harmony":
        think = _RE_HARMONY_THINK.search(text)
        if think:
            msg["reasoning_content"] = think.group(1).strip()
    else:
        think = _RE_THINK.match(msg["content"]) if "</think>" in msg["content"] else None
        if think:
            if think.group(1).strip():
                msg["reasoning_content"] = think.group(1).strip()
            msg["content"] = think.group(2)
    if calls:
        msg["tool_calls"] = calls
    return msg
