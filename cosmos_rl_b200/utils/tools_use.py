"""Tool use in the object form user scripts of the reference write against (cosmos_rl/utils/tools_use/: ``BaseTool``,
``ToolParser`` / ``HermesToolParser``, ``ToolAgent`` and the OpenAI function-calling schema models). The multi-turn
rollout of this package drives tools through ``data/multi_turn.py: ToolRegistry``; ``ToolAgent.mount`` puts object tools
into that registry, so both styles end up on the same path.

A tool is a subclass with a ``function``; its schema comes from the signature and the docstring unless one is given:

    class Add(BaseTool):
        def function(self, a: int, b: int) -> ToolResponse:
            '''Add two integers.'''
            return ToolResponse(text=str(a + b))

    agent = ToolAgent(HermesToolParser(), [Add("add")])
    agent.call_tools('<tool_call>{"name": "add", "arguments": {"a": 1, "b": 2}}</tool_call>')
"""
from __future__ import annotations

import inspect
import re
from abc import ABC, abstractmethod
from contextlib import contextmanager
from typing import Any, Dict, List, Optional, Tuple, get_type_hints

from pydantic import BaseModel, Field

from ..data.multi_turn import ToolRegistry, parse_tool_calls
from .logging import logger


# ---------------------------------------------------------------------------------------------------
# OpenAI function-calling schema
# ---------------------------------------------------------------------------------------------------
class OpenAIFunctionPropertySchema(BaseModel):
    type: str
    description: Optional[str] = None
    enum: Optional[List[Any]] = None


class OpenAIFunctionParametersSchema(BaseModel):
    type: str = "object"
    properties: Dict[str, OpenAIFunctionPropertySchema] = Field(default_factory=dict)
    required: List[str] = Field(default_factory=list)


class OpenAIFunctionSchema(BaseModel):
    name: str
    description: str = ""
    parameters: OpenAIFunctionParametersSchema = Field(default_factory=OpenAIFunctionParametersSchema)
    strict: bool = False


class OpenAIFunctionToolSchema(BaseModel):
    type: str = "function"
    function: OpenAIFunctionSchema


class OpenAIFunctionParsedSchema(BaseModel):
    """A call as the model wrote it: the arguments still a JSON string."""
    name: str
    arguments: str


class OpenAIFunctionCallSchema(BaseModel):
    name: str
    arguments: Dict[str, Any] = Field(default_factory=dict)


class OpenAIFunctionToolCall(BaseModel):
    id: str
    type: str = "function"
    function: OpenAIFunctionCallSchema


class ToolResponse(BaseModel):
    text: Optional[str] = None
    image: Optional[Any] = None
    video: Optional[Any] = None

    def is_empty(self) -> bool:
        return self.text is None and self.image is None and self.video is None


_JSON_TYPES = {int: "integer", float: "number", str: "string", bool: "boolean", list: "array", dict: "object"}


def schema_from_function(fn, name: str) -> OpenAIFunctionToolSchema:
    """Schema of a callable from its annotations; the first docstring paragraph is the description, lines of the
    form ``arg: text`` (after an ``Args:`` heading or anywhere) describe parameters."""
    doc = inspect.getdoc(fn) or ""
    hints = get_type_hints(fn) if callable(fn) else {}
    arg_doc = {m.group(1): m.group(2).strip() for m in re.finditer(r"^\s*(\w+)\s*(?:\([^)]*\))?:\s*(.+)$", doc, re.MULTILINE)}
    props, required = {}, []
    for pname, p in inspect.signature(fn).parameters.items():
        if pname == "self" or p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
            continue
        t = hints.get(pname, str)
        origin = getattr(t, "__origin__", t)
        props[pname] = OpenAIFunctionPropertySchema(type=_JSON_TYPES.get(origin, "string"), description=arg_doc.get(pname))
        if p.default is inspect.Parameter.empty:
            required.append(pname)
    return OpenAIFunctionToolSchema(function=OpenAIFunctionSchema(
        name=name, description=doc.split("\n\n")[0].strip(),
        parameters=OpenAIFunctionParametersSchema(properties=props, required=required)))


# ---------------------------------------------------------------------------------------------------
class BaseTool(ABC):
    def __init__(self, name: str, schema: Optional[OpenAIFunctionToolSchema] = None):
        self.name = name
        self._schema = schema

    def __call__(self, *args, **kwargs) -> Any:
        return self.function(*args, **kwargs)

    @contextmanager
    def tool_context(self, ground_truth: Optional[str] = None):
        """Entered around every call; override to give the tool what it may check against (the reference answer of the
        sample), or to acquire and release a resource."""
        yield self

    @property
    def tool_schema(self) -> OpenAIFunctionToolSchema:
        if self._schema is None:
            self._schema = schema_from_function(self.function, self.name)
        return self._schema

    @abstractmethod
    def function(self, *args, **kwargs) -> ToolResponse:
        raise NotImplementedError


class ToolParser(ABC):
    @abstractmethod
    def extract_tool_calls(self, text: str) -> Tuple[str, List[OpenAIFunctionCallSchema]]:
        """(the text without the call blocks, the calls found in it)."""
        raise NotImplementedError


class HermesToolParser(ToolParser):
    """``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` blocks (the Qwen / Hermes chat templates)."""
    tool_call_start_token = "<tool_call>"
    tool_call_end_token = "</tool_call>"
    _block = re.compile(r"<tool_call>.*?</tool_call>", re.DOTALL)

    def extract_tool_calls(self, text: str) -> Tuple[str, List[OpenAIFunctionCallSchema]]:
        calls = [OpenAIFunctionCallSchema(**c) for c in parse_tool_calls(text)]      # malformed blocks are skipped
        return (self._block.sub("", text) if calls or self.tool_call_start_token in text else text), calls


class ToolAgent:
    def __init__(self, tool_parser: ToolParser, tools: List[BaseTool]):
        self.tool_parser = tool_parser
        self.tools: Dict[str, BaseTool] = {t.name: t for t in tools}

    def call_tools(self, text: str, ground_truth: Optional[str] = None) -> Optional[List[ToolResponse]]:
        """Run every call found in ``text``; None when there is none. A call that fails (unknown tool, bad arguments,
        an exception in the tool) yields a response that says so: the model sees its own mistakes."""
        _, calls = self.tool_parser.extract_tool_calls(text)
        if not calls:
            return None
        out: List[ToolResponse] = []
        for c in calls:
            tool = self.tools.get(c.name)
            if tool is None:
                out.append(ToolResponse(text=f"error: unknown tool {c.name!r}"))
                continue
            try:
                with tool.tool_context(ground_truth):
                    r = tool(**c.arguments)
                out.append(r if isinstance(r, ToolResponse) else ToolResponse(text=str(r)))
            except Exception as e:  # noqa: BLE001
                logger.warning("[ToolAgent] tool %s failed: %s", c.name, e)
                out.append(ToolResponse(text=f"error: {type(e).__name__}: {e}"))
        return out

    def tool_schemas(self) -> List[Dict[str, Any]]:
        return [t.tool_schema.model_dump(exclude_none=True) for t in self.tools.values()]

    def mount(self) -> None:
        """Register the tools with the multi-turn rollout's registry (``rollout.multi_turn_config.enable_tools``)."""
        for t in self.tools.values():
            schema = t.tool_schema.model_dump(exclude_none=True)["function"]

            def run(_tool=t, **kw):
                with _tool.tool_context(None):
                    r = _tool(**kw)
                return r.text if isinstance(r, ToolResponse) else r
            ToolRegistry.register(t.name, schema.get("description", ""), schema.get("parameters"))(run)
