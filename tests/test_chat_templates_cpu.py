"""Every packaged training template: renders its family's format, marks assistant spans, is prefix preserving, and
its tool calls parse back (template -> text -> ``parse_response`` -> the same call).  The shapes of these checks
follow tests/test_chat_template_utils.py of the reference."""
import glob
import os

import pytest

from trl_b200.chat_template_utils import (_FAMILIES, add_response_schema, detect_chat_family, get_training_chat_template,
                                          has_generation_markers, list_chat_families, parse_response)
from trl_b200.testing import make_tiny_tokenizer

TOOLS = [{"type": "function", "function": {"name": "multiply", "description": "Multiply two numbers", "parameters": {
    "type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "string"}}, "required": ["a", "b"]}}}]
CALL = {"type": "function", "function": {"name": "multiply", "arguments": {"a": 3, "b": "x y"}}}
CONV = [{"role": "system", "content": "SYS"}, {"role": "user", "content": "beautiful idea"},
        {"role": "assistant", "content": "simple explain"}, {"role": "user", "content": "U2"},
        {"role": "assistant", "content": "", "tool_calls": [CALL]}, {"role": "tool", "name": "multiply", "content": "12"},
        {"role": "assistant", "content": "A3"}]
NO_TOOL_SYNTAX = {"gemma", "phi3", "idefics3", "llava", "llava_next", "deepseekv3"}  # families without a call syntax here


def _tok(family):
    tok = make_tiny_tokenizer()
    tok.chat_template = get_training_chat_template(tok, family=family)
    return tok


def test_every_template_file_belongs_to_a_family():
    here = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "trl_b200", "chat_templates")
    files = {os.path.basename(f) for f in glob.glob(os.path.join(here, "*.jinja"))}
    assert files == {f[3] for f in _FAMILIES}
    assert len(list_chat_families()) == len(set(list_chat_families())) >= 31


@pytest.mark.parametrize("family", [f[0] for f in _FAMILIES])
def test_training_template_marks_assistant_spans_and_preserves_prefixes(family):
    tok = _tok(family)
    assert has_generation_markers(tok.chat_template)
    plain = CONV[:3]
    a = tok.apply_chat_template(plain, tokenize=False)
    b = tok.apply_chat_template(CONV[:4], tokenize=False)
    assert b.startswith(a) and "beautiful idea" in a and "simple explain" in a
    gp = tok.apply_chat_template(CONV[:2], tokenize=False, add_generation_prompt=True)
    assert gp.startswith(tok.apply_chat_template(CONV[:2], tokenize=False))
    out = tok.apply_chat_template(plain, tokenize=True, return_dict=True, return_assistant_tokens_mask=True)
    ids, mask = out["input_ids"], out["assistant_masks"]
    if ids and isinstance(ids[0], list):
        ids, mask = ids[0], mask[0]
    assert 0 < sum(mask) < len(ids)  # some, not all, tokens belong to the assistant
    marked = tok.decode([t for t, m in zip(ids, mask) if m])
    assert "simple" in marked and "explain" in marked and "beautiful" not in marked and "idea" not in marked


@pytest.mark.parametrize("family", [f[0] for f in _FAMILIES if f[0] not in NO_TOOL_SYNTAX])
def test_tool_calls_render_and_parse_back(family):
    tok = _tok(family)
    kw = {"tools": TOOLS}
    full = tok.apply_chat_template(CONV, tokenize=False, **kw)
    assert "multiply" in full and "12" in full and "A3" in full
    assert full.startswith(tok.apply_chat_template(CONV[:5], tokenize=False, **kw))  # the tool result is a pure suffix
    # the text the model would have produced for the tool-call turn = rendering up to it minus the prompt before it
    before = tok.apply_chat_template(CONV[:4], tokenize=False, **kw)
    upto = tok.apply_chat_template(CONV[:5], tokenize=False, **kw)
    assert upto.startswith(before)
    completion = upto[len(before):]  # the assistant turn as rendered (its header included: the parsers skip it)
    add_response_schema(tok, family=family)
    msg = parse_response(tok, completion)
    assert msg["role"] == "assistant" and msg.get("tool_calls"), (family, completion, msg)
    fn = msg["tool_calls"][0]["function"]
    assert fn["name"] == "multiply" and fn["arguments"] == {"a": 3, "b": "x y"}, (family, completion, fn)


def test_family_detection_from_a_tokenizers_own_template():
    cases = {
        "<|im_start|> ... <think> ...": "qwen3",
        "<|im_start|>system\nYou are Qwen, created by Alibaba Cloud": "qwen2_5",
        "<|im_start|> <tool_call> no reasoning here": "qwen3_instruct_2507",
        "<|im_start|> <function=x> <parameter= enable_thinking": "qwen3_5_think",
        "<|im_start|> <function=x> <name>": "nemotron_3_nano",
        "<|im_start|><|vision_start|>": "qwen3_vl",
        "<|start_header_id|> Cutting Knowledge Date: December 2023 strftime_now": "llama3_2",
        "<|start_header_id|> Cutting Knowledge Date": "llama3_1",
        "<|start_header_id|>": "llama3",
        "<|START_OF_TURN_TOKEN|><|START_RESPONSE|>": "cohere2",
        "<|im_start|><|tool_list_start|>": "lfm2",
        "<|turn>model": "diffusion_gemma",
        "[INST] <image>": "llava_next",
        "<|assistant|> <|end|> eos_token": "phi3_5",
    }
    for tpl, want in cases.items():
        assert detect_chat_family(tpl)[0] == want, (tpl, detect_chat_family(tpl))
    assert detect_chat_family("nothing known") is None
    with pytest.raises(ValueError):
        get_training_chat_template(make_tiny_tokenizer(), family="no_such_family")


def test_malformed_calls_fall_back_to_plain_text():
    tok = _tok("qwen3_5_think")
    add_response_schema(tok, family="qwen3_5_think")
    bad = "<tool_call>\n<function=multiply\n</tool_call>"
    assert parse_response(tok, bad) == {"role": "assistant", "content": bad}
    tok2 = _tok("lfm2")
    add_response_schema(tok2, family="lfm2")
    bad2 = "<|tool_call_start|>[multiply(a=3,]<|tool_call_end|>"
    assert parse_response(tok2, bad2)["content"] == bad2


_TURNS = ("{%- for m in messages %}{%- if m.role == 'user' %}{{- '<|im_start|>user\\n' + m.content + '<|im_end|>\\n' }}"
          "{%- elif m.role == 'tool' %}{{- '<|im_start|>tool\\n' + m.content + '<|im_end|>\\n' }}"
          "{%- elif m.role == 'assistant' %}ASSISTANT{%- endif %}{%- endfor %}"
          "{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}{%- endif %}")
_CALLS = ("{%- if m.tool_calls %}{%- for c in m.tool_calls %}{%- if c.function %}{%- set c = c.function %}{%- endif %}"
          "{{- '<tool_call>' + c.name + '</tool_call>' }}{%- endfor %}{%- endif %}")


def test_prefix_preservation_and_stop_token_probes_on_handwritten_templates():
    """The behaviours of tests/test_chat_template_utils.py:394-596: a template whose earlier turns never change when a
    tool turn is appended is prefix-preserving, one that renders a think block only for the last assistant turn is not;
    the end-of-turn token counts as trained only when it lies inside the generation span; a template that raises reads
    as not trained."""
    from trl_b200.chat_template_utils import is_chat_template_prefix_preserving, is_chat_template_stop_token_trained
    from trl_b200.testing import make_tiny_tokenizer

    tok = make_tiny_tokenizer()
    plain = "{{- '<|im_start|>assistant\\n' + (m.content or '') }}" + _CALLS + "{{- '<|im_end|>\\n' }}"
    tok.chat_template = _TURNS.replace("ASSISTANT", plain)
    assert is_chat_template_prefix_preserving(tok) is True
    last_only = ("{%- if loop.last %}{{- '<|im_start|>assistant\\n<think>\\n\\n</think>\\n\\n' + (m.content or '') }}"
                 "{%- else %}{{- '<|im_start|>assistant\\n' + (m.content or '') }}{%- endif %}" + _CALLS + "{{- '<|im_end|>\\n' }}")
    tok.chat_template = _TURNS.replace("ASSISTANT", last_only)
    assert is_chat_template_prefix_preserving(tok) is False

    inside = "{{- '<|im_start|>assistant\\n' }}{%- generation %}{{- m.content + '<|im_end|>' }}{%- endgeneration %}{{- '\\n' }}"
    tok.chat_template = _TURNS.replace("ASSISTANT", inside)
    assert is_chat_template_stop_token_trained(tok) is True
    outside = "{{- '<|im_start|>assistant\\n' }}{%- generation %}{{- m.content }}{%- endgeneration %}{{- '<|im_end|>\\n' }}"
    tok.chat_template = _TURNS.replace("ASSISTANT", outside)
    assert is_chat_template_stop_token_trained(tok) is False
    tok.chat_template = "{{ raise_exception('probe rejected') }}"
    assert is_chat_template_stop_token_trained(tok) is False


@pytest.mark.parametrize("family", [f[0] for f in _FAMILIES if f[0] not in NO_TOOL_SYNTAX])
def test_parse_response_never_raises_on_a_truncated_tool_call_turn(family):
    """tests/test_chat_template_utils.py:1301-1330: a completion cut anywhere inside a tool call still parses to a
    message (as text when the call is incomplete)."""
    tok = _tok(family)
    before = tok.apply_chat_template(CONV[:4], tokenize=False, tools=TOOLS)
    upto = tok.apply_chat_template(CONV[:5], tokenize=False, tools=TOOLS)
    completion = upto[len(before):]
    add_response_schema(tok, family=family)
    for end in range(1, len(completion)):
        msg = parse_response(tok, completion[:end])
        assert msg["role"] == "assistant" and ("content" in msg or "tool_calls" in msg)


def test_json_tool_call_with_a_missing_brace_stays_text():
    tok = _tok("qwen3")
    add_response_schema(tok, family="qwen3")
    bad = '<tool_call>\n{"name": "multiply", "arguments": {"a": 3, "b": 4}\n</tool_call>'
    assert parse_response(tok, bad + "<|im_end|>") == {"role": "assistant", "content": bad}
