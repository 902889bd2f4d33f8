"""Multi-turn rollouts with tool calls: parsing, tool execution, the assistant-token mask, and the generation loop of
the built-in backend driven by a scripted engine."""
import json

import torch

from cosmos_rl_b200.config import Config
from cosmos_rl_b200.data.multi_turn import ToolRegistry, assistant_token_mask, extend_conversation, parse_tool_calls
from cosmos_rl_b200.data.packer import DecoderOnlyLLMDataPacker
from cosmos_rl_b200.dispatcher.data.schema import RLPayload
from cosmos_rl_b200.parallel.dims import ParallelDims


class CharTokenizer:
    """One token per character, ``<|role|>`` ... ``<|end|>`` markers (as single ids) around every message."""
    eos_token_id, pad_token_id = 1, 0
    MARK = {"system": 2, "user": 3, "assistant": 4, "tool": 5, "end": 1}

    def encode(self, text, add_special_tokens=False):
        return [ord(c) + 10 for c in text]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(i - 10) for i in ids if i >= 10)

    def apply_chat_template(self, conv, tokenize=True, add_generation_prompt=False, tools=None, **kw):
        ids = []
        if tools:
            ids += [2] + self.encode(json.dumps([t["function"]["name"] for t in tools])) + [1]
        for m in conv:
            ids += [self.MARK[m["role"]]] + self.encode(m["content"]) + [1]
        if add_generation_prompt:
            ids += [4]
        return ids


def test_tool_calls_and_assistant_mask():
    ToolRegistry.clear()

    @ToolRegistry.register(description="add two integers")
    def add(a: int, b: int):
        return {"sum": a + b}

    text = 'Let me compute. <tool_call>{"name": "add", "arguments": {"a": 2, "b": 40}}</tool_call> <tool_call>{bad json}</tool_call>'
    assert parse_tool_calls(text) == [{"name": "add", "arguments": {"a": 2, "b": 40}}]
    conv, done = extend_conversation([{"role": "user", "content": "2+40?"}], text, enable_tools=True)
    assert not done and conv[-1] == {"role": "tool", "name": "add", "content": '{"sum": 42}'}
    conv, done = extend_conversation(conv, "It is 42.", enable_tools=True)
    assert done and [m["role"] for m in conv] == ["user", "assistant", "tool", "assistant"]
    assert json.loads(ToolRegistry.call("add", {"a": 1}))["error"].startswith("TypeError")
    assert "unknown tool" in ToolRegistry.call("nope", {})
    tok = CharTokenizer()
    ids, mask = assistant_token_mask(tok, conv)
    scored = tok.decode([i for i, m in zip(ids, mask) if m])
    assert scored == text + "It is 42." and sum(mask) == len(text) + len("It is 42.") + 2     # + two end markers
    cfg = Config.from_dict({"rollout": {"multi_turn_config": {"enable": True, "enable_tools": True}}})
    packer = DecoderOnlyLLMDataPacker()
    packer.setup(cfg, tok)
    pi = packer.get_policy_input(conv[:1], conv)
    assert len(pi.input_ids) == len(pi.logprob_masks) and sum(pi.logprob_masks) == sum(mask)
    first = pi.logprob_masks.index(1)
    assert pi.input_ids[first + 1] == ids[mask.index(1)]          # mask position i scores token i + 1


class _ScriptedEngine:
    """Stands in for the generation engine: answers from a script keyed by the turn number of the prompt."""

    def __init__(self, tok):
        self.tok, self.calls = tok, []

    def generate(self, prompts, sp):
        from cosmos_rl_b200.rollout.engine import Completion
        self.calls.append(len(prompts))
        out = []
        for p in prompts:
            turn = sum(1 for t in p if t == 4) - 1               # assistant markers before the generation prompt
            text = '<tool_call>{"name": "add", "arguments": {"a": 1, "b": 2}}</tool_call>' if turn == 0 else "3"
            ids = self.tok.encode(text)
            out.append([Completion(token_ids=ids, logprobs=[-0.1] * len(ids), finish_reason="stop")])
        return out


def test_multi_turn_generation_loop(tmp_path):
    from cosmos_rl_b200.rollout.b200_rollout import B200Rollout
    ToolRegistry.clear()

    @ToolRegistry.register()
    def add(a: int, b: int):
        return a + b

    cfg = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 256},
        "rollout": {"n_generation": 2, "max_response_length": 64,
                    "multi_turn_config": {"enable": True, "enable_tools": True, "max_assistant_turns": 3}},
        "train": {"output_dir": str(tmp_path), "train_policy": {"type": "grpo"}}})
    tok = CharTokenizer()
    ro = B200Rollout(cfg, ParallelDims(world_size=1, device=torch.device("cpu")), torch.device("cpu"), tokenizer=tok)
    ro.engine = _ScriptedEngine(tok)
    packer = DecoderOnlyLLMDataPacker()
    packer.setup(cfg, tok)
    payloads = [RLPayload(prompt=[{"role": "user", "content": "1+2?"}], prompt_idx=0),
                RLPayload(prompt="What is 1+2?", prompt_idx=1)]
    res = ro.rollout_generation(payloads, packer)
    assert ro.engine.calls == [4, 4]                              # all four paths advance together, two turns each
    for r in res:
        assert r.completions == ["3", "3"] and r.extra_info["assistant_turns"] == [2, 2]
        conv = r.completed_conversations[0]
        assert [m["role"] for m in conv] == ["user", "assistant", "tool", "assistant"] and conv[2]["content"] == "3"
