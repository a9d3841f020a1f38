"""Anthropic-Messages-compatible request validation and response assembly.

Request models forbid unknown fields (HTTP 400 ``unknown_field``), sampling controls are range
checked, conversation shape / tool / thinking rules are enforced before any work is queued, and
one ``ResponseAssembler`` state machine produces both projections of a reply: the SSE event
sequence and the final JSON message.

Behavioural parity: naivert/serve/messages_api.py (request models :58-100, feature checks
:165-199, tools :231-288, thinking :291-321, sampling :464-492, ``validate_request`` :515-545,
usage :564-573, ``ResponseAssembler`` :583-752) and docs/messages_http.md.
"""
from __future__ import annotations

import json
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Literal, Mapping, Optional, Sequence, Tuple, Union

from pydantic import BaseModel, ConfigDict, ValidationError

from ..models.spec import SamplingParams
from .syntax import ToolCallParseError, coerce_arguments, parse_tool_call, render_tool_calls


class ApiError(Exception):
    """An error that maps to the API's JSON error shape."""

    def __init__(self, status: int, warning: str, message: str, kind: Optional[str] = None):
        super().__init__(message)
        self.status, self.warning, self.message = status, warning, message
        self.kind = kind or {400: "invalid_request_error", 404: "not_found_error", 503: "overloaded_error",
                             529: "overloaded_error"}.get(status, "api_error")

    def body(self) -> dict:
        return {"type": "error", "error": {"type": self.kind, "message": self.message, "warning_type": self.warning}}


# ----------------------------------------------------------------------------- request models
class _Strict(BaseModel):
    model_config = ConfigDict(extra="forbid")


class CacheControl(_Strict):
    type: str
    ttl: Optional[str] = None


class TextBlock(_Strict):
    type: Literal["text"]
    text: str
    cache_control: Optional[CacheControl] = None
    citations: Optional[Any] = None


class ThinkingBlock(_Strict):
    type: Literal["thinking"]
    thinking: str
    signature: Optional[str] = None


class ToolUseBlock(_Strict):
    type: Literal["tool_use"]
    id: str
    name: str
    input: Dict[str, Any]
    cache_control: Optional[CacheControl] = None
    caller: Optional[Any] = None


class ToolResultBlock(_Strict):
    type: Literal["tool_result"]
    tool_use_id: str
    content: Union[str, List[TextBlock], None] = None
    is_error: Optional[bool] = None
    cache_control: Optional[CacheControl] = None


Block = Union[TextBlock, ThinkingBlock, ToolUseBlock, ToolResultBlock]


class Message(_Strict):
    role: Literal["user", "assistant", "system"]
    content: Union[str, List[Block]]


class ToolDef(_Strict):
    name: str
    description: Optional[str] = None
    input_schema: Dict[str, Any]
    cache_control: Optional[CacheControl] = None
    type: Optional[str] = None
    strict: Optional[bool] = None


class ToolChoice(_Strict):
    type: str
    name: Optional[str] = None
    disable_parallel_tool_use: Optional[bool] = None


class Thinking(_Strict):
    type: str
    budget_tokens: Optional[int] = None
    display: Optional[str] = None


class Metadata(BaseModel):
    model_config = ConfigDict(extra="allow")
    user_id: Optional[str] = None


class CountTokensRequest(_Strict):
    model: str
    messages: List[Message]
    system: Union[str, List[TextBlock], None] = None
    thinking: Optional[Thinking] = None
    tools: Optional[List[ToolDef]] = None
    tool_choice: Optional[ToolChoice] = None
    metadata: Optional[Metadata] = None
    output_config: Optional[Dict[str, Any]] = None
    context_management: Optional[Dict[str, Any]] = None


class MessagesRequest(CountTokensRequest):
    max_tokens: int
    stream: bool = False
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    seed: Optional[int] = None
    stop_sequences: Optional[List[str]] = None
    repetition_penalty: Optional[float] = None
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    parsed_output: Optional[Any] = None
    service_tier: Optional[Any] = None
    container: Optional[Any] = None
    mcp_servers: Optional[Any] = None
    betas: Optional[Any] = None


def parse_request(raw: bytes, model_cls=MessagesRequest):
    try:
        return model_cls.model_validate_json(raw)
    except ValidationError as e:
        errs = e.errors()
        first = errs[0]
        loc = ".".join(str(x) for x in first["loc"])
        if any(x["type"] == "extra_forbidden" for x in errs):
            bad = next(x for x in errs if x["type"] == "extra_forbidden")
            raise ApiError(400, "unknown_field", f"unknown field {'.'.join(str(v) for v in bad['loc'])}")
        raise ApiError(400, "schema", f"{loc}: {first['msg']}")


# ----------------------------------------------------------------------------- validated task
@dataclass
class TaskParams:
    model: str
    messages: List[dict]                 # chat-template messages (role/content[/tool_calls])
    tools: Optional[List[dict]]
    tool_schemas: Dict[str, dict]
    thinking: bool
    max_tokens: int
    stream: bool
    sampling: SamplingParams
    stop_sequences: List[str]
    stop_inclusive: bool
    single_tool_call: bool
    session_id: Optional[str]
    ignored: List[str] = field(default_factory=list)
    token_progress: bool = False


@dataclass
class ServerDefaults:
    served_model: str = "naive-n0.5"
    temperature: float = 1.0
    top_p: float = 0.95
    seed: int = 1234
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    max_output_tokens: int = 524288


def _text_of(content) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    return "".join(b.text for b in content)


def _validate_tools(req, ignored: List[str]) -> Tuple[Optional[List[dict]], Dict[str, dict], bool]:
    tools = req.tools or []
    choice = req.tool_choice
    if choice is not None:
        if not tools:
            raise ApiError(400, "invalid_tool_choice", "tool_choice requires a non-empty tools array")
        if choice.type not in ("auto", "none"):
            raise ApiError(400, "forced_tool_choice_unsupported", f"tool_choice type {choice.type!r} is not supported")
    schemas: Dict[str, dict] = {}
    rendered = []
    for t in tools:
        if t.type not in (None, "custom"):
            raise ApiError(400, "server_tool_unsupported", f"tool type {t.type!r} is not supported")
        if t.strict:
            raise ApiError(400, "strict_tools_unsupported", "strict tool schemas are not supported")
        if t.name in schemas:
            raise ApiError(400, "invalid_tool_schema", f"duplicate tool name {t.name!r}")
        if t.input_schema.get("type") != "object":
            raise ApiError(400, "invalid_tool_schema", f"tool {t.name!r}: input_schema must be an object schema")
        for pname, ps in (t.input_schema.get("properties") or {}).items():
            if isinstance(ps, dict) and not any(k in ps for k in ("type", "anyOf", "oneOf", "enum")):
                if "untyped_tool_property" not in ignored:
                    ignored.append("untyped_tool_property")
        if t.cache_control is not None and "cache_control" not in ignored:
            ignored.append("cache_control")
        schemas[t.name] = t.input_schema
        rendered.append({"type": "function", "function": {"name": t.name, "description": t.description or "",
                                                          "parameters": t.input_schema}})
    if choice is not None and choice.type == "none":
        return None, {}, False
    single = bool(choice and choice.disable_parallel_tool_use)
    return (rendered or None), schemas, single


def _validate_thinking(th: Optional[Thinking], max_tokens: Optional[int], ignored: List[str]) -> bool:
    if th is None or th.type == "disabled":
        return False
    if th.display is not None:
        ignored.append("thinking.display")
    if th.type == "adaptive":
        ignored.append("thinking.adaptive")
        return True
    if th.type != "enabled":
        raise ApiError(400, "thinking_mode_unsupported", f"thinking type {th.type!r} is not supported")
    b = th.budget_tokens
    if not isinstance(b, int) or b < 1024 or (max_tokens is not None and b >= max_tokens):
        raise ApiError(400, "invalid_thinking_budget", "thinking.budget_tokens must satisfy 1024 <= budget < max_tokens")
    return True


def _build_messages(req, ignored: List[str]) -> List[dict]:
    """API messages -> chat-template messages; enforces the conversation shape."""
    out: List[dict] = []
    sys_text = _text_of(req.system) if req.system is not None else ""
    if isinstance(req.system, list) and any(b.cache_control for b in req.system) and "cache_control" not in ignored:
        ignored.append("cache_control")
    if sys_text:
        out.append({"role": "system", "content": sys_text})
    turns = [m for m in req.messages if m.role != "system"]
    if not turns or turns[0].role != "user" or turns[-1].role != "user":
        raise ApiError(400, "invalid_messages", "messages must start and end with a user turn")
    for a, b in zip(turns, turns[1:]):
        if a.role == b.role:
            raise ApiError(400, "invalid_messages", "user and assistant turns must alternate")
    pending_calls: Dict[str, str] = {}
    for m in req.messages:
        blocks = [TextBlock(type="text", text=m.content)] if isinstance(m.content, str) else m.content
        for b in blocks:
            if getattr(b, "cache_control", None) is not None and "cache_control" not in ignored:
                ignored.append("cache_control")
            if getattr(b, "citations", None) is not None or getattr(b, "caller", None) is not None:
                raise ApiError(400, "unsupported_feature", "citations / caller are not supported")
        if m.role == "system":
            if any(b.type != "text" for b in blocks):
                raise ApiError(400, "invalid_messages", "system messages accept text blocks only")
            out.append({"role": "system", "content": _text_of(blocks)})
        elif m.role == "user":
            results = [b for b in blocks if b.type == "tool_result"]
            for b in blocks:
                if b.type not in ("text", "tool_result"):
                    raise ApiError(400, "invalid_messages", f"user turns do not accept {b.type} blocks")
            for r in results:
                if r.tool_use_id not in pending_calls:
                    raise ApiError(400, "orphan_tool_result", f"tool_result {r.tool_use_id!r} has no matching tool_use")
                text = _text_of(r.content)
                out.append({"role": "tool", "content": ("[error] " + text) if r.is_error else text})
            text = "".join(b.text for b in blocks if b.type == "text")
            if text or not results:
                out.append({"role": "user", "content": text})
            pending_calls = {}
        else:
            calls, text, think = [], "", ""
            pending_calls = {}
            for b in blocks:
                if b.type == "text":
                    text += b.text
                elif b.type == "thinking":
                    if b.signature:
                        raise ApiError(400, "thinking_signature_unsupported", "non-empty thinking signatures are not supported")
                    think += b.thinking
                elif b.type == "tool_use":
                    calls.append({"name": b.name, "arguments": b.input})
                    pending_calls[b.id] = b.name
                else:
                    raise ApiError(400, "invalid_messages", f"assistant turns do not accept {b.type} blocks")
            msg = {"role": "assistant", "content": text}
            if think:
                msg["reasoning_content"] = think
            if calls:
                msg["tool_calls"] = calls
                msg["tool_calls_text"] = render_tool_calls(calls)
            out.append(msg)
    return out


def _rng(name, v, lo, hi, warn, lo_open=False):
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v != v or (v <= lo if lo_open else v < lo) or v > hi:
        br = "(" if lo_open else "["
        raise ApiError(400, warn, f"{name}={v} must be a number in {br}{lo}, {hi}]")


def validate_request(req, defaults: ServerDefaults, headers: Optional[Mapping[str, str]] = None,
                     count_only: bool = False) -> TaskParams:
    headers = {k.lower(): v for k, v in (headers or {}).items()}
    if req.model != defaults.served_model:
        raise ApiError(404, "unknown_model", f"model {req.model!r} is not served here (try {defaults.served_model!r})")
    ignored: List[str] = []
    if not count_only:
        for name in ("parsed_output", "service_tier", "container", "mcp_servers", "betas"):
            if getattr(req, name) is not None:
                raise ApiError(400, f"{name}_unsupported", f"{name} is not supported")
        if req.top_k is not None:
            raise ApiError(400, "top_k_unsupported", "top_k sampling is not supported")
        if isinstance(req.max_tokens, bool) or req.max_tokens < 1:
            raise ApiError(400, "schema", "max_tokens must be a positive integer")
        if req.max_tokens > defaults.max_output_tokens:
            raise ApiError(400, "max_tokens_exceeds_capture",
                           f"max_tokens={req.max_tokens} exceeds the server output limit {defaults.max_output_tokens}")
    if req.output_config is not None:
        if set(req.output_config) - {"effort"}:
            raise ApiError(400, "output_format_unsupported", "structured output formats are not supported")
        ignored.append("output_config.effort")
    if req.context_management is not None:
        if not isinstance(req.context_management.get("edits"), list):
            raise ApiError(400, "schema", "context_management.edits must be a list")
        ignored.append("context_management")
    max_tokens = None if count_only else req.max_tokens
    thinking = _validate_thinking(req.thinking, max_tokens, ignored)
    tools, schemas, single = _validate_tools(req, ignored)
    messages = _build_messages(req, ignored)
    if count_only:
        sp = SamplingParams()
        stops: List[str] = []
    else:
        t = defaults.temperature if req.temperature is None else req.temperature
        p = defaults.top_p if req.top_p is None else req.top_p
        seed = defaults.seed if req.seed is None else req.seed
        rp = defaults.repetition_penalty if req.repetition_penalty is None else req.repetition_penalty
        fp = defaults.frequency_penalty if req.frequency_penalty is None else req.frequency_penalty
        pp = defaults.presence_penalty if req.presence_penalty is None else req.presence_penalty
        _rng("temperature", t, 0, 5, "invalid_temperature", lo_open=True)
        _rng("top_p", p, 0, 1, "invalid_top_p", lo_open=True)
        if isinstance(seed, bool) or not isinstance(seed, int) or not 0 <= seed < 2 ** 63:
            raise ApiError(400, "invalid_seed", f"seed={seed} must be an integer in [0, 2^63 - 1]")
        _rng("repetition_penalty", rp, 0, 10, "invalid_repeat_penalty", lo_open=True)
        _rng("frequency_penalty", fp, -10, 10, "invalid_repeat_penalty")
        _rng("presence_penalty", pp, -10, 10, "invalid_repeat_penalty")
        stops = list(req.stop_sequences or [])
        if len(stops) > 8 or any((not isinstance(s, str)) or not s for s in stops):
            raise ApiError(400, "invalid_stop_sequences", "stop_sequences takes up to eight non-empty strings")
        sp = SamplingParams(temperature=float(t), top_p=float(p), seed=int(seed), repetition_penalty=float(rp),
                            frequency_penalty=float(fp), presence_penalty=float(pp))
    session = headers.get("x-session-id") or (req.metadata.user_id if req.metadata else None)
    if single:
        stops = stops + ["</tool_call>"]
    return TaskParams(model=req.model, messages=messages, tools=tools, tool_schemas=schemas, thinking=thinking,
                      max_tokens=0 if count_only else req.max_tokens, stream=False if count_only else req.stream,
                      sampling=sp, stop_sequences=stops, stop_inclusive=single, single_tool_call=single,
                      session_id=session, ignored=ignored, token_progress=headers.get("x-naivert-token-progress") == "1")


# ----------------------------------------------------------------------------- usage + assembly
def usage_dict(prompt_tokens: int, cached: int, output: int, thinking_tokens: Optional[int]) -> dict:
    u = {"input_tokens": 0, "cache_read_input_tokens": cached,
         "cache_creation_input_tokens": max(0, prompt_tokens - cached), "output_tokens": output}
    if thinking_tokens is not None:
        u["output_tokens_details"] = {"thinking_tokens": thinking_tokens}
    return u


class ResponseAssembler:
    """Consumes segments of the reply and yields SSE events; keeps the blocks for the JSON form.

    Event order: message_start, (content_block_start, content_block_delta*, content_block_stop)*,
    message_delta, message_stop."""

    def __init__(self, params: TaskParams, prompt_tokens: int = 0, cached_tokens: int = 0, queue_wait_ms: float = 0.0):
        self.p = params
        self.id = "msg_" + uuid.uuid4().hex[:24]
        self.blocks: List[dict] = []
        self.open_kind: Optional[str] = None
        self.prompt_tokens, self.cached_tokens, self.queue_wait_ms = prompt_tokens, cached_tokens, queue_wait_ms
        self.untyped = False
        self.saw_tool = False

    # -- SSE helpers
    @staticmethod
    def sse(event: str, data: dict) -> str:
        return f"event: {event}\ndata: {json.dumps(data, ensure_ascii=False, separators=(',', ':'))}\n\n"

    def start_event(self) -> str:
        msg = {"id": self.id, "type": "message", "role": "assistant", "model": self.p.model, "content": [],
               "stop_reason": None, "stop_sequence": None,
               "usage": usage_dict(self.prompt_tokens, self.cached_tokens, 0, 0 if self.p.thinking else None)}
        return self.sse("message_start", {"type": "message_start", "message": msg,
                                          "naivert": {"queue_wait_ms": round(self.queue_wait_ms, 3)}})

    def _close_open(self) -> List[str]:
        if self.open_kind is None:
            return []
        self.open_kind = None
        return [self.sse("content_block_stop", {"type": "content_block_stop", "index": len(self.blocks) - 1})]

    def _open(self, kind: str, block: dict) -> List[str]:
        out = self._close_open()
        self.blocks.append(block)
        self.open_kind = kind
        shown = {k: ("" if k in ("text", "thinking") else ({} if k == "input" else v)) for k, v in block.items()}
        out.append(self.sse("content_block_start", {"type": "content_block_start", "index": len(self.blocks) - 1,
                                                    "content_block": shown}))
        return out

    def feed(self, kind: str, text: str, closed: bool, generated_tokens: Optional[int] = None) -> List[str]:
        out: List[str] = []
        if kind in ("text", "thinking"):
            if text:
                if self.open_kind != kind:
                    out += self._open(kind, {"type": kind, kind: ""})
                self.blocks[-1][kind] += text
                delta = {"type": f"{kind}_delta", kind: text}
                ev = {"type": "content_block_delta", "index": len(self.blocks) - 1, "delta": delta}
                if self.p.token_progress and generated_tokens is not None:
                    ev["naivert"] = {"generated_tokens": generated_tokens}
                out.append(self.sse("content_block_delta", ev))
            if closed:
                out += self._close_open()
            return out
        # tool calls arrive whole
        if not closed:
            raise ToolCallParseError("the reply ended inside a <tool_call> block")
        name, raw = parse_tool_call(text)
        if name not in self.p.tool_schemas:
            raise ToolCallParseError(f"the model called an undeclared tool {name!r}")
        args, untyped = coerce_arguments(raw, self.p.tool_schemas[name])
        self.untyped |= bool(untyped)
        self.saw_tool = True
        block = {"type": "tool_use", "id": "toolu_" + uuid.uuid4().hex[:24], "name": name, "input": args}
        out += self._open("tool_use", block)
        out.append(self.sse("content_block_delta", {"type": "content_block_delta", "index": len(self.blocks) - 1,
                                                    "delta": {"type": "input_json_delta",
                                                              "partial_json": json.dumps(args, ensure_ascii=False)}}))
        out += self._close_open()
        return out

    def _trim(self) -> None:
        """Whitespace-only text blocks around tool calls carry no content."""
        self.blocks = [b for b in self.blocks if not (b["type"] == "text" and not b["text"].strip() and self.saw_tool)]

    def finish(self, stop_reason: str, stop_sequence: Optional[str], output_tokens: int,
               thinking_tokens: Optional[int], extension: Optional[dict] = None) -> List[str]:
        out = self._close_open()
        reason = {"eos": "end_turn", "output_limit": "max_tokens", "position_limit": "max_tokens",
                  "stop_sequence": "stop_sequence"}.get(stop_reason, stop_reason)
        if self.saw_tool and reason in ("end_turn", "stop_sequence") and (self.p.single_tool_call or reason == "end_turn"):
            reason, stop_sequence = "tool_use", None
        self.stop_reason, self.stop_sequence = reason, stop_sequence
        self.usage = usage_dict(self.prompt_tokens, self.cached_tokens, output_tokens,
                                thinking_tokens if self.p.thinking else None)
        self.extension = extension or {}
        out.append(self.sse("message_delta", {"type": "message_delta",
                                              "delta": {"stop_reason": reason, "stop_sequence": stop_sequence},
                                              "usage": self.usage, "naivert": self.extension}))
        out.append(self.sse("message_stop", {"type": "message_stop"}))
        return out

    def message(self) -> dict:
        self._trim()
        return {"id": self.id, "type": "message", "role": "assistant", "model": self.p.model, "content": self.blocks,
                "stop_reason": self.stop_reason, "stop_sequence": self.stop_sequence, "usage": self.usage,
                "naivert": self.extension}
