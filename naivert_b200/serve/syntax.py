"""Assistant-output syntax of the Naive-N chat template: splitting a generated character
stream into text / thinking / tool-call segments, parsing tool calls and coercing their raw
string arguments to the JSON types the tool's ``input_schema`` declares.

Wire format produced by the model::

    <think>...</think>                       (only at the very start of the reply)
    <tool_call>
    <function=NAME>
    <parameter=P>VALUE</parameter>
    </function>
    </tool_call>

Behavioural parity: naivert/serve/naive_n0p5_syntax.py (``SegmentStream`` :76,
``parse_tool_call`` :207, ``coerce_arguments`` :302, ``render_tool_calls`` :34).  The
implementation here is a small explicit state machine over a character buffer.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

THINK = ("<think>", "</think>")
TOOL = ("<tool_call>", "</tool_call>")


class ToolCallParseError(ValueError):
    """A generated tool call does not follow the template or violates its schema."""


@dataclass
class Segment:
    kind: str          # "text" | "thinking" | "tool_call"
    text: str          # newly available inner text (delimiters stripped)
    closed: bool       # the closing delimiter of this segment has been seen


def _held_tail(buf: str, markers: Iterable[str]) -> int:
    """Number of trailing characters that may still be the beginning of a marker."""
    hold = 0
    for m in markers:
        top = min(len(m) - 1, len(buf))
        for n in range(top, hold, -1):
            if buf.endswith(m[:n]):
                hold = n
                break
    return hold


class SegmentStream:
    """Incremental splitter.  ``feed(text)`` returns the segments (or segment parts) that
    became certain; text that could still turn into a delimiter is held back.  ``<think>`` is
    honoured only before any non-whitespace output; ``<tool_call>`` only if tools were declared."""

    def __init__(self, thinking: bool = True, tools: bool = True):
        self._buf = ""
        self._state = "text"
        self._may_think = thinking
        self._tools = tools
        self._done = False
        self._emitted_in_segment = False

    @property
    def kind(self) -> str:
        return self._state

    def feed(self, text: str) -> List[Segment]:
        if self._done:
            raise RuntimeError("stream already finished")
        self._buf += text
        return self._pump(final=False)

    def finish(self) -> List[Segment]:
        if self._done:
            return []
        self._done = True
        return self._pump(final=True)

    # ------------------------------------------------------------------
    def _openers(self) -> List[Tuple[str, str]]:
        out = []
        if self._may_think:
            out.append((THINK[0], "thinking"))
        if self._tools:
            out.append((TOOL[0], "tool_call"))
        return out

    def _pump(self, final: bool) -> List[Segment]:
        out: List[Segment] = []
        while True:
            if self._state == "text":
                openers = self._openers()
                hit = None
                for marker, kind in openers:
                    i = self._buf.find(marker)
                    if i >= 0 and (hit is None or i < hit[0]):
                        hit = (i, marker, kind)
                if hit is not None and hit[2] == "thinking" and self._buf[: hit[0]].strip():
                    # <think> after real text is ordinary text
                    self._may_think = False
                    continue
                if hit is not None:
                    before = self._buf[: hit[0]]
                    if before and (before.strip() or self._emitted_in_segment or hit[2] != "thinking"):
                        out.append(Segment("text", before, True))
                    elif before and hit[2] == "thinking":
                        pass                                  # leading whitespace before <think> is dropped
                    if before.strip():
                        self._may_think = False
                    self._buf = self._buf[hit[0] + len(hit[1]):]
                    self._state = hit[2]
                    self._emitted_in_segment = False
                    if hit[2] != "thinking":
                        self._may_think = False
                    continue
                hold = 0 if final else _held_tail(self._buf, [m for m, _ in openers])
                ready = self._buf[: len(self._buf) - hold]
                if self._may_think and not final and not ready.strip():
                    return out                                # only whitespace so far: <think> may still come
                if ready:
                    if ready.strip():
                        self._may_think = False
                    out.append(Segment("text", ready, False))
                    self._emitted_in_segment = True
                    self._buf = self._buf[len(ready):]
                if final and self._emitted_in_segment:
                    out.append(Segment("text", "", True))
                    self._emitted_in_segment = False
                return out
            closer = THINK[1] if self._state == "thinking" else TOOL[1]
            i = self._buf.find(closer)
            if i >= 0:
                out.append(Segment(self._state, self._buf[:i], True))
                self._buf = self._buf[i + len(closer):]
                self._state = "text"
                self._may_think = False
                self._emitted_in_segment = False
                continue
            if self._state == "tool_call" and not final:
                return out                                    # tool calls are delivered whole
            hold = 0 if final else _held_tail(self._buf, [closer])
            ready = self._buf[: len(self._buf) - hold]
            if ready or final:
                out.append(Segment(self._state, ready, False))
                self._buf = self._buf[len(ready):]
            return out


# ----------------------------------------------------------------------------- tool calls
_FUNC = re.compile(r"^\s*<function=([^>\n]+)>\n?(.*?)\n?</function>\s*$", re.S)
_PARAM = re.compile(r"<parameter=([^>\n]+)>\n?(.*?)\n?</parameter>", re.S)


def parse_tool_call(inner: str) -> Tuple[str, Dict[str, str]]:
    """Inner text of one ``<tool_call>`` block -> (function name, raw string arguments)."""
    m = _FUNC.match(inner)
    if not m:
        raise ToolCallParseError("tool call does not contain exactly one <function=...>...</function> block")
    name, body = m.group(1).strip(), m.group(2)
    args: Dict[str, str] = {}
    pos = 0
    for pm in _PARAM.finditer(body):
        if body[pos:pm.start()].strip():
            raise ToolCallParseError("unexpected text between parameters of a tool call")
        key = pm.group(1).strip()
        if key in args:
            raise ToolCallParseError(f"parameter {key!r} given twice")
        args[key] = pm.group(2)
        pos = pm.end()
    if body[pos:].strip():
        raise ToolCallParseError("unexpected trailing text inside a tool call")
    return name, args


def _schema_types(schema: Mapping[str, Any]) -> List[Mapping[str, Any]]:
    """Flatten type unions / anyOf / oneOf into candidate sub-schemas."""
    if not isinstance(schema, Mapping):
        return []
    out: List[Mapping[str, Any]] = []
    for key in ("anyOf", "oneOf"):
        for sub in schema.get(key, ()) or ():
            out.extend(_schema_types(sub))
    t = schema.get("type")
    if isinstance(t, list):
        out.extend({**schema, "type": x} for x in t)
    elif isinstance(t, str):
        out.append(schema)
    elif "enum" in schema and not out:
        out.append(schema)
    return out


def _coerce_one(raw: str, schema: Mapping[str, Any]) -> Any:
    t = schema.get("type")
    text = raw.strip()
    if "enum" in schema:
        for cand in schema["enum"]:
            if cand == raw or (not isinstance(cand, str) and json.dumps(cand) == text):
                return cand
        if t is None:
            raise ValueError("value is not one of the enum members")
    if t == "string":
        return raw
    if t == "integer":
        if re.fullmatch(r"[-+]?\d+", text):
            return int(text)
        raise ValueError("not an integer")
    if t == "number":
        v = float(text)
        return int(v) if re.fullmatch(r"[-+]?\d+", text) else v
    if t == "boolean":
        if text.lower() in ("true", "false"):
            return text.lower() == "true"
        raise ValueError("not a boolean")
    if t == "null":
        if text.lower() in ("null", "none", ""):
            return None
        raise ValueError("not null")
    if t in ("array", "object"):
        v = json.loads(text)
        if (t == "array") != isinstance(v, list) or (t == "object") != isinstance(v, dict):
            raise ValueError(f"not a JSON {t}")
        return v
    raise ValueError(f"unsupported schema type {t!r}")


def coerce_arguments(raw: Mapping[str, str], input_schema: Mapping[str, Any]) -> Tuple[Dict[str, Any], List[str]]:
    """Raw parameter strings -> typed arguments.  Returns (arguments, names of untyped properties)."""
    props = input_schema.get("properties", {}) or {}
    out: Dict[str, Any] = {}
    untyped: List[str] = []
    for key, value in raw.items():
        sch = props.get(key)
        cands = _schema_types(sch) if sch is not None else []
        if not cands:
            out[key] = value
            untyped.append(key)
            continue
        # prefer non-string interpretations so "3" becomes 3 under ["string", "integer"]... only when it parses
        ordered = sorted(cands, key=lambda s: s.get("type") == "string")
        err: Optional[Exception] = None
        for cand in ordered:
            try:
                out[key] = _coerce_one(value, cand)
                break
            except (ValueError, json.JSONDecodeError) as e:
                err = e
        else:
            raise ToolCallParseError(f"argument {key!r}={value!r} does not fit its schema: {err}")
    missing = [k for k in input_schema.get("required", ()) or () if k not in out]
    if missing:
        raise ToolCallParseError(f"tool call lacks required arguments {missing}")
    return out, untyped


def render_tool_calls(calls: Sequence[Mapping[str, Any]]) -> str:
    """Assistant-history tool calls rendered exactly the way the model writes them, so a replayed
    conversation reproduces the generated tokens and the cached prefix still matches."""
    blocks = []
    for call in calls:
        params = []
        for k, v in (call.get("arguments") or {}).items():
            text = v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)
            params.append(f"<parameter={k}>{text}</parameter>\n")
        blocks.append(f"{TOOL[0]}\n<function={call['name']}>\n{''.join(params)}</function>\n{TOOL[1]}")
    return "\n".join(blocks)
