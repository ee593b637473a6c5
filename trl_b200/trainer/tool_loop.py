"""Multi-turn tool calling for GRPO (behaviour of trl/trainer/grpo_trainer.py:1933-2141).

After each generation the completion is parsed (``parse_response``); requested tools are executed
(sync or async callables, looked up by ``__name__``), their results are appended as ``tool`` messages,
and generation continues from the extended conversation until no tool is called, the iteration limit
is reached, or the completion budget is exhausted.  Tool-result tokens are part of the completion but
excluded from the loss through ``tool_mask`` (0 on tool tokens, 1 on model tokens).
"""
from __future__ import annotations

import asyncio
import json

from ..chat_template_utils import parse_response
from .utils import run_coroutine_sync


class ToolLoop:
    def __init__(self, trainer, tools, max_iterations=None):
        self.t = trainer
        self.tools = {getattr(f, "__name__", str(i)): f for i, f in enumerate(tools)}
        self.max_iterations = max_iterations

    def _call(self, call):
        fn = call.get("function", call)
        name, args = fn.get("name"), fn.get("arguments", {})
        if isinstance(args, str):
            try:
                args = json.loads(args)
            except json.JSONDecodeError:
                return name, f"Error: could not parse arguments {args!r}"
        tool = self.tools.get(name)
        if tool is None:
            return name, f"Error: unknown tool {name!r}"
        try:
            res = tool(**args)
            if asyncio.iscoroutine(res):
                res = run_coroutine_sync(res)
            return name, str(res)
        except Exception as e:  # noqa: BLE001 - the error text is fed back to the model
            return name, f"Error: {type(e).__name__}: {e}"

    def generate(self, prompts):
        t, tok = self.t, self.t.processing_class
        B = len(prompts)
        convs = [list(p) if isinstance(p, list) else [{"role": "user", "content": p}] for p in prompts]
        prompt_ids = t._tokenize_prompts(convs)
        comp_ids = [[] for _ in range(B)]
        comp_lp = [[] for _ in range(B)]
        mask = [[] for _ in range(B)]
        active = list(range(B))
        calls_made, failures, it = 0, 0, 0
        while active:
            ids_now = [prompt_ids[i] + comp_ids[i] for i in active]
            budget = [t.max_completion_length - len(comp_ids[i]) for i in active]
            _, outs, lps, _ = t._generate([ids for ids in ids_now])
            nxt = []
            for j, i in enumerate(active):
                new = outs[j][: max(0, budget[j])]
                comp_ids[i] += new
                comp_lp[i] += list(lps[j][: len(new)]) if lps and lps[j] else [0.0] * len(new)
                mask[i] += [1] * len(new)
                msg = parse_response(tok, new)
                convs[i].append(msg)
                if not msg.get("tool_calls") or len(comp_ids[i]) >= t.max_completion_length:
                    continue
                if self.max_iterations is not None and it >= self.max_iterations:
                    continue
                before = tok.apply_chat_template(convs[i], tools=list(self.tools.values()) or None, tokenize=False)
                for call in msg["tool_calls"]:
                    name, result = self._call(call)
                    calls_made += 1
                    failures += result.startswith("Error:")
                    convs[i].append({"role": "tool", "name": name, "content": result})
                after = tok.apply_chat_template(convs[i], tools=list(self.tools.values()) or None, tokenize=False,
                                                add_generation_prompt=True)
                suffix = after[len(before):] if after.startswith(before) else after
                s_ids = tok(text=suffix, add_special_tokens=False)["input_ids"]
                room = t.max_completion_length - len(comp_ids[i])
                s_ids = s_ids[:room]
                comp_ids[i] += s_ids
                comp_lp[i] += [0.0] * len(s_ids)
                mask[i] += [0] * len(s_ids)
                if len(comp_ids[i]) < t.max_completion_length:
                    nxt.append(i)
            active = nxt
            it += 1
        m = t._metrics["train" if t.model.training else "eval"]
        m["tools/call_frequency"].append(calls_made / max(1, B))
        m["tools/failure_frequency"].append(failures / max(1, calls_made))
        return prompt_ids, comp_ids, comp_lp, {"tool_mask": mask}
