"""Multi-turn rollouts with tool use: the policy's response is appended to the conversation, tool calls found in it
are executed and their results appended as ``tool`` messages, and generation continues until a turn without tool
calls or the turn limit (cosmos_rl/dispatcher/data/packer/multi_turn.py, rollout/vllm_rollout/vllm_rollout.py:768-955).

Tool calls use the ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` convention of the Qwen / Hermes chat
templates."""
from __future__ import annotations

import json
import re
from typing import Any, Callable, Dict, List, Optional, Tuple

Conversation = List[Dict[str, Any]]
# the body never crosses a closing tag, so a malformed block cannot swallow the well-formed one after it
_CALL = re.compile(r"<tool_call>\s*((?:(?!</tool_call>).)*?)\s*</tool_call>", re.DOTALL)


class ToolRegistry:
    _tools: Dict[str, Tuple[Callable, Dict[str, Any]]] = {}

    @classmethod
    def register(cls, name: Optional[str] = None, description: str = "", parameters: Optional[Dict[str, Any]] = None):
        def deco(fn):
            n = name or fn.__name__
            cls._tools[n] = (fn, {"type": "function", "function": {
                "name": n, "description": description or (fn.__doc__ or "").strip(),
                "parameters": parameters or {"type": "object", "properties": {}}}})
            return fn
        return deco

    @classmethod
    def schemas(cls) -> List[Dict[str, Any]]:
        """Tool descriptions in the form chat templates take (``tools=`` of ``apply_chat_template``)."""
        return [s for _, s in cls._tools.values()]

    @classmethod
    def call(cls, name: str, arguments: Dict[str, Any]) -> str:
        if name not in cls._tools:
            return json.dumps({"error": f"unknown tool {name!r}"})
        try:
            out = cls._tools[name][0](**arguments)
        except Exception as e:  # noqa: BLE001  (the model sees its own mistakes as tool output)
            return json.dumps({"error": f"{type(e).__name__}: {e}"})
        return out if isinstance(out, str) else json.dumps(out)

    @classmethod
    def clear(cls) -> None:
        cls._tools = {}


def parse_tool_calls(text: str) -> List[Dict[str, Any]]:
    calls = []
    for m in _CALL.finditer(text):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        if isinstance(obj, dict) and isinstance(obj.get("name"), str):
            args = obj.get("arguments", {})
            calls.append({"name": obj["name"], "arguments": args if isinstance(args, dict) else {}})
    return calls


def extend_conversation(conversation: Conversation, response: str, enable_tools: bool) -> Tuple[Conversation, bool]:
    """Append the assistant turn (and tool results). Returns (conversation, finished)."""
    conv = list(conversation) + [{"role": "assistant", "content": response}]
    calls = parse_tool_calls(response) if enable_tools else []
    if not calls:
        return conv, True
    for c in calls:
        conv.append({"role": "tool", "name": c["name"], "content": ToolRegistry.call(c["name"], c["arguments"])})
    return conv, False


def assistant_token_mask(tokenizer, conversation: Conversation, tools=None) -> Tuple[List[int], List[int]]:
    """Token ids of the whole conversation and a 0/1 mask of the tokens the policy produced (assistant turns,
    including their end-of-turn marker): the chat template is applied to growing prefixes, so the mask follows the
    template exactly whatever markers it inserts."""
    kw = {"tools": tools} if tools else {}
    full = tokenizer.apply_chat_template(conversation, tokenize=True, add_generation_prompt=False, **kw)
    mask = [0] * len(full)
    for i, msg in enumerate(conversation):
        if msg.get("role") != "assistant":
            continue
        start = len(tokenizer.apply_chat_template(conversation[:i], tokenize=True, add_generation_prompt=True, **kw))
        end = len(tokenizer.apply_chat_template(conversation[:i + 1], tokenize=True, add_generation_prompt=False, **kw))
        for t in range(start, min(end, len(full))):
            mask[t] = 1
    return list(full), mask
