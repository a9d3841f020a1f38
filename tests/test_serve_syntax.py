"""Segmentation of generated text, tool-call parsing and schema coercion."""
import pytest

from naivert_b200.serve.syntax import (SegmentStream, ToolCallParseError, coerce_arguments, parse_tool_call,
                                       render_tool_calls)


def _collect(chunks, **kw):
    s = SegmentStream(**kw)
    segs = []
    for c in chunks:
        segs += s.feed(c)
    segs += s.finish()
    merged = []
    for g in segs:
        if merged and merged[-1][0] == g.kind and not merged[-1][2]:
            merged[-1] = (g.kind, merged[-1][1] + g.text, g.closed)
        else:
            merged.append((g.kind, g.text, g.closed))
    return [m for m in merged if m[1] or m[0] != "text"]


def test_think_then_text_any_chunking():
    full = "<think>plan it</think>The answer."
    want = [("thinking", "plan it", True), ("text", "The answer.", True)]
    assert _collect([full]) == want
    assert _collect(list(full)) == want
    assert _collect([full[:3], full[3:9], full[9:]]) == want


def test_think_only_at_front_and_disabled():
    assert _collect(["hello <think>x</think>"]) == [("text", "hello <think>x</think>", True)]
    assert _collect(["<think>x</think>y"], thinking=False) == [("text", "<think>x</think>y", True)]


def test_tool_call_split_and_partial_tag_held_back():
    s = SegmentStream(thinking=False, tools=True)
    out = s.feed("Let me check <tool")
    assert [(g.kind, g.text) for g in out] == [("text", "Let me check ")]
    out = s.feed("_call>\n<function=f>\n</function>\n</tool_call>")
    assert [(g.kind, g.closed) for g in out][-1] == ("tool_call", True)
    assert s.finish() == [] or all(g.text == "" for g in s.finish())
    # without declared tools the tag is prose
    assert _collect(["a <tool_call> b"], tools=False) == [("text", "a <tool_call> b", True)]


def test_unclosed_blocks_reported_open():
    assert _collect(["<think>never ends"])[-1] == ("thinking", "never ends", False)
    assert _collect(["<tool_call>\n<function=f>"], thinking=False)[-1][2] is False


def test_parse_and_coerce():
    inner = "\n<function=get_weather>\n<parameter=city>Paris</parameter>\n<parameter=days>3</parameter>\n<parameter=opts>{\"a\": [1, 2]}</parameter>\n</function>\n"
    name, raw = parse_tool_call(inner)
    assert name == "get_weather" and raw == {"city": "Paris", "days": "3", "opts": '{"a": [1, 2]}'}
    schema = {"type": "object", "required": ["city"],
              "properties": {"city": {"type": "string"}, "days": {"type": ["integer", "null"]},
                             "opts": {"anyOf": [{"type": "object"}, {"type": "null"}]}}}
    args, untyped = coerce_arguments(raw, schema)
    assert args == {"city": "Paris", "days": 3, "opts": {"a": [1, 2]}} and untyped == []
    args, untyped = coerce_arguments({"city": "x", "extra": "1"}, schema)
    assert args["extra"] == "1" and untyped == ["extra"]
    with pytest.raises(ToolCallParseError):
        coerce_arguments({"days": "3"}, schema)                      # missing required
    with pytest.raises(ToolCallParseError):
        coerce_arguments({"city": "x", "days": "soon"}, schema)
    assert coerce_arguments({"b": "true", "e": "red"}, {"properties": {"b": {"type": "boolean"}, "e": {"enum": ["red", "blue"]}}})[0] == {"b": True, "e": "red"}


def test_malformed_calls_raise():
    for bad in ["no function", "<function=f>\n<parameter=a>1</parameter>\njunk\n</function>",
                "<function=f>\n<parameter=a>1</parameter>\n<parameter=a>2</parameter>\n</function>"]:
        with pytest.raises(ToolCallParseError):
            parse_tool_call(bad)


def test_render_round_trips():
    calls = [{"name": "f", "arguments": {"s": "a b", "n": 3, "flag": True}}, {"name": "g", "arguments": {}}]
    text = render_tool_calls(calls)
    segs = _collect([text], thinking=False)
    tools = [s for s in segs if s[0] == "tool_call"]
    assert len(tools) == 2
    name, raw = parse_tool_call(tools[0][1])
    assert name == "f" and raw == {"s": "a b", "n": "3", "flag": "true"}
