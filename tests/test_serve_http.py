"""HTTP surface against a fake engine (real uvicorn on loopback): JSON and SSE replies, event
order, validation errors, queue-full, cancel on disconnect, failures, tools, thinking, sessions."""
import json
import socket
import threading
import time

import httpx
import pytest

from naivert_b200.models.spec import SamplingParams
from naivert_b200.serve.chat import ByteTokenizer, ChatFormatter
from naivert_b200.serve.context import ServerContext
from naivert_b200.serve.http import build_app
from naivert_b200.serve.messages_api import ServerDefaults


class FakeConfig:
    capacity = 4096
    max_output_tokens = 4000
    eos_token_ids = (ByteTokenizer().eos_token_id,)


class FakeSession:
    def __init__(self, engine, reply_tokens, max_decode, cached):
        self.e, self.toks, self.max, self.i = engine, reply_tokens, max_decode, 0
        self.done, self.stop_reason, self.cached_tokens = False, None, cached
        self.cancelled = False

    def step(self, timeout):
        assert threading.get_ident() == self.e.owner, "engine used from a foreign thread"
        if self.e.fail_step:
            raise RuntimeError("injected step failure")
        if self.e.gate is not None:
            self.e.gate.wait(5)
        time.sleep(self.e.delay)
        out = self.toks[self.i:self.i + 3]
        self.i += len(out)
        if self.i >= min(len(self.toks), self.max):
            out = out[: max(0, len(out) - (self.i - min(len(self.toks), self.max)))]
            self.done = True
            self.stop_reason = "eos" if self.i >= len(self.toks) and self.max >= len(self.toks) else "output_limit"
        return out

    def cancel(self):
        self.cancelled = True
        self.e.cancels += 1

    def finish(self):
        return {"decode_tok_s_device": 1234.5, "segments": {"total": {"tokens": self.i, "rounds": 1}}}


class FakeEngine:
    config = FakeConfig()

    def __init__(self):
        self.tok = ByteTokenizer()
        self.reply = "Hello there."
        self.fail_open = self.fail_step = False
        self.delay, self.gate, self.cancels = 0.0, None, 0
        self.owner = None
        self.sessions = {}
        self.opened = []

    def align_prompt(self, tokens, session_id):
        return tokens

    def open_session(self, tokens, max_decode, session_id, sampling):
        self.owner = threading.get_ident()
        if self.fail_open:
            raise RuntimeError("injected open failure")
        assert isinstance(sampling, SamplingParams)
        prev = self.sessions.get(session_id, [])
        cached = 0
        for a, b in zip(prev, tokens):
            if a != b:
                break
            cached += 1
        self.sessions[session_id] = list(tokens)
        self.opened.append((session_id, len(tokens), max_decode, sampling))
        return FakeSession(self, self.tok.encode(self.reply) + [self.tok.eos_token_id], max_decode, cached)


@pytest.fixture()
def server(tmp_path_factory):
    import uvicorn
    eng = FakeEngine()
    eng.dump_path = str(tmp_path_factory.mktemp("dump") / "tokens.jsonl")
    app = build_app(lambda: ServerContext(eng, ChatFormatter(eng.tok)), ServerDefaults(served_model="naive-n0.5", max_output_tokens=4000),
                    queue_depth=2, dump_tokens=eng.dump_path)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    srv = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
    t = threading.Thread(target=srv.run, daemon=True)
    t.start()
    base = f"http://127.0.0.1:{port}"
    for _ in range(200):
        try:
            if httpx.get(base + "/health", timeout=1).status_code == 200:
                break
        except Exception:
            pass
        time.sleep(0.05)
    yield base, eng
    srv.should_exit = True
    t.join(5)


def _body(**kw):
    b = {"model": "naive-n0.5", "max_tokens": 64, "messages": [{"role": "user", "content": "hi"}]}
    b.update(kw)
    return b


def _events(text):
    out = []
    for block in text.split("\n\n"):
        ev = [l for l in block.splitlines() if l.startswith("event: ")]
        da = [l for l in block.splitlines() if l.startswith("data: ")]
        if ev and da:
            out.append((ev[0][7:], json.loads(da[0][6:])))
    return out


def test_json_reply_usage_and_models(server):
    base, eng = server
    r = httpx.post(base + "/v1/messages", json=_body(), headers={"x-session-id": "s1"})
    assert r.status_code == 200, r.text
    m = r.json()
    assert m["type"] == "message" and m["role"] == "assistant" and m["stop_reason"] == "end_turn"
    assert m["content"] == [{"type": "text", "text": "Hello there."}]
    u = m["usage"]
    assert u["input_tokens"] == 0 and u["cache_read_input_tokens"] == 0 and u["cache_creation_input_tokens"] > 0
    assert u["output_tokens"] == len("Hello there.") + 1 and "output_tokens_details" not in u
    assert m["naivert"]["timings"]["decode_tok_s_device"] == 1234.5 and m["naivert"]["timeline"]["spans"]
    r2 = httpx.post(base + "/v1/messages", json=_body(), headers={"x-session-id": "s1"})
    assert r2.json()["usage"]["cache_read_input_tokens"] > 0
    assert httpx.get(base + "/v1/models").json()["data"][0]["id"] == "naive-n0.5"
    h = httpx.get(base + "/health").json()
    assert h == {"status": "ok", "slot": "IDLE", "queued": 0}
    n = httpx.post(base + "/v1/messages/count_tokens", json={"model": "naive-n0.5", "messages": [{"role": "user", "content": "hi"}]}).json()
    assert n["input_tokens"] == eng.opened[0][1]


def test_token_dump_lines(server):
    base, eng = server
    r = httpx.post(base + "/v1/messages", json=_body(), timeout=30)
    assert r.status_code == 200
    deadline = time.time() + 5
    rows = []
    while time.time() < deadline and not rows:
        try:
            rows = [json.loads(l) for l in open(eng.dump_path)]
        except FileNotFoundError:
            time.sleep(0.05)
    assert rows and rows[-1]["output_tokens"] == r.json()["usage"]["output_tokens"] and isinstance(rows[-1]["tokens"], list)


def test_sse_event_order(server):
    base, eng = server
    with httpx.stream("POST", base + "/v1/messages", json=_body(stream=True), headers={"x-naivert-token-progress": "1"}) as r:
        assert r.headers["content-type"].startswith("text/event-stream")
        ev = _events("".join(r.iter_text()))
    names = [e[0] for e in ev]
    assert names[0] == "message_start" and names[-2:] == ["message_delta", "message_stop"]
    assert names[1] == "content_block_start" and "content_block_stop" in names
    text = "".join(e[1]["delta"]["text"] for e in ev if e[0] == "content_block_delta")
    assert text == "Hello there."
    assert all("generated_tokens" in e[1]["naivert"] for e in ev if e[0] == "content_block_delta")
    md = [e[1] for e in ev if e[0] == "message_delta"][0]
    assert md["delta"]["stop_reason"] == "end_turn" and md["usage"]["output_tokens"] > 0 and "timings" in md["naivert"]


@pytest.mark.parametrize("patch,code,warn", [
    ({"bogus": 1}, 400, "unknown_field"), ({"temperature": 0}, 400, "invalid_temperature"),
    ({"top_p": 1.5}, 400, "invalid_top_p"), ({"seed": -1}, 400, "invalid_seed"), ({"top_k": 5}, 400, "top_k_unsupported"),
    ({"model": "other"}, 404, "unknown_model"), ({"max_tokens": 99999}, 400, "max_tokens_exceeds_capture"),
    ({"stop_sequences": [""]}, 400, "invalid_stop_sequences"),
    ({"messages": [{"role": "assistant", "content": "x"}]}, 400, "invalid_messages"),
    ({"thinking": {"type": "enabled", "budget_tokens": 10}}, 400, "invalid_thinking_budget"),
    ({"tool_choice": {"type": "auto"}}, 400, "invalid_tool_choice"),
    ({"repetition_penalty": 0}, 400, "invalid_repeat_penalty"),
])
def test_validation_errors(server, patch, code, warn):
    base, _ = server
    r = httpx.post(base + "/v1/messages", json=_body(**patch))
    assert r.status_code == code, r.text
    assert r.json()["error"]["warning_type"] == warn and r.headers["x-naivert-warning"] == warn


def test_stop_sequence_max_tokens_and_top_p_clamp(server):
    base, eng = server
    r = httpx.post(base + "/v1/messages", json=_body(stop_sequences=["there"], top_p=1)).json()
    assert r["stop_reason"] == "stop_sequence" and r["stop_sequence"] == "there" and r["content"][0]["text"] == "Hello "
    assert eng.opened[-1][3].clamped_top_p() < 1.0
    r = httpx.post(base + "/v1/messages", json=_body(max_tokens=4)).json()
    assert r["stop_reason"] == "max_tokens" and r["usage"]["output_tokens"] <= 4


def test_thinking_and_tools(server):
    base, eng = server
    eng.reply = "pondering</think>\n\n<tool_call>\n<function=get_weather>\n<parameter=city>Paris</parameter>\n<parameter=days>2</parameter>\n</function>\n</tool_call>"
    tools = [{"name": "get_weather", "input_schema": {"type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}, "required": ["city"]}}]
    r = httpx.post(base + "/v1/messages", json=_body(max_tokens=2048, tools=tools, thinking={"type": "enabled", "budget_tokens": 1024}))
    m = r.json()
    assert r.status_code == 200, r.text
    kinds = [b["type"] for b in m["content"]]
    assert kinds == ["thinking", "tool_use"], m["content"]
    assert m["content"][0]["thinking"] == "pondering" and m["content"][1]["input"] == {"city": "Paris", "days": 2}
    assert m["stop_reason"] == "tool_use" and m["usage"]["output_tokens_details"]["thinking_tokens"] > 0
    # the tool result turn validates against the previous tool_use id
    hist = _body(max_tokens=64, tools=tools)
    hist["messages"] += [{"role": "assistant", "content": m["content"]},
                         {"role": "user", "content": [{"type": "tool_result", "tool_use_id": m["content"][1]["id"], "content": "18C"}]}]
    eng.reply = "It is 18C."
    assert httpx.post(base + "/v1/messages", json=hist).json()["content"][0]["text"] == "It is 18C."
    hist["messages"][-1]["content"][0]["tool_use_id"] = "toolu_nope"
    assert httpx.post(base + "/v1/messages", json=hist).json()["error"]["warning_type"] == "orphan_tool_result"
    eng.reply = "<tool_call>\n<function=get_weather>\n<parameter=days>x</parameter>\n</function>\n</tool_call>"
    bad = httpx.post(base + "/v1/messages", json=_body(tools=tools))
    assert bad.status_code == 500 and bad.json()["error"]["warning_type"] == "tool_call_parse_error"


def test_failures_and_recovery(server):
    base, eng = server
    eng.fail_open = True
    r = httpx.post(base + "/v1/messages", json=_body())
    assert r.status_code == 500 and r.json()["error"]["warning_type"] == "runtime_error"
    eng.fail_open, eng.fail_step = False, True
    with httpx.stream("POST", base + "/v1/messages", json=_body(stream=True)) as s:
        ev = _events("".join(s.iter_text()))
    assert ev[-1][0] == "error" and ev[-1][1]["error"]["warning_type"] == "runtime_error"
    eng.fail_step = False
    assert httpx.post(base + "/v1/messages", json=_body()).status_code == 200          # slot recovered (ERROR -> RESET -> IDLE)
    assert httpx.get(base + "/health").json()["slot"] == "IDLE"


def test_queue_full_and_disconnect_cancels(server):
    base, eng = server
    eng.gate = threading.Event()
    eng.reply = "x" * 600
    results = []

    def call():
        results.append(httpx.post(base + "/v1/messages", json=_body(max_tokens=700), timeout=30).status_code)

    threads = [threading.Thread(target=call) for _ in range(3)]     # 1 active + 2 queued
    for t in threads:
        t.start()
        time.sleep(0.15)
    assert httpx.post(base + "/v1/messages", json=_body()).status_code == 529
    assert httpx.get(base + "/health").json()["queued"] >= 1
    eng.gate.set()
    eng.gate = None
    for t in threads:
        t.join(30)
    assert results == [200, 200, 200]
    # a streaming client that goes away cancels the session
    eng.delay, before = 0.05, eng.cancels
    with httpx.stream("POST", base + "/v1/messages", json=_body(stream=True, max_tokens=700)) as s:
        for chunk in s.iter_text():
            if "content_block_delta" in chunk:
                break
    for _ in range(100):
        if eng.cancels > before:
            break
        time.sleep(0.05)
    assert eng.cancels > before
    eng.delay = 0.0
    eng.reply = "ok"
    assert httpx.post(base + "/v1/messages", json=_body()).json()["content"][0]["text"] == "ok"


def test_anthropic_sdk_round_trip(server):
    anthropic = pytest.importorskip("anthropic")
    base, eng = server
    eng.reply = "SDK says hi."
    with anthropic.Anthropic(base_url=base, api_key="unused", max_retries=0) as client:
        reply = client.messages.create(model="naive-n0.5", max_tokens=64, messages=[{"role": "user", "content": "hello"}],
                                       temperature=0.4, top_p=0.95, extra_body={"seed": 4}, extra_headers={"x-session-id": "sdk"})
        assert reply.content[0].text == "SDK says hi." and reply.stop_reason == "end_turn"
        assert reply.model_extra["naivert"]["timings"]["predicted_n"] > 0
        with client.messages.stream(model="naive-n0.5", max_tokens=64, messages=[{"role": "user", "content": "again"}]) as s:
            assert "".join(s.text_stream) == "SDK says hi."
    assert eng.opened[-2][3].seed == 4 and abs(eng.opened[-2][3].temperature - 0.4) < 1e-9


def test_studio_smoke_bench_compares_json_sse_and_proxy(server):
    """The Studio's smoke benchmark against the fake-engine server: JSON, SSE and SSE through the local proxy give the
    same text for the same seed; a wrong model name is reported as a failed mode."""
    import importlib.util
    import os
    base, eng = server
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def load(name):
        sp = importlib.util.spec_from_file_location(name, os.path.join(root, "apps", "studio", name + ".py"))
        m = importlib.util.module_from_spec(sp)
        sp.loader.exec_module(m)
        return m
    bench, proxy_mod = load("smoke_bench"), load("local_server")
    eng.reply = "<svg><circle r='3'/></svg>"
    proxy = proxy_mod.serve(base, port=0)
    threading.Thread(target=proxy.serve_forever, daemon=True).start()
    try:
        rep = bench.run(base, f"http://127.0.0.1:{proxy.server_address[1]}", max_tokens=256)
        assert rep["ok"] and rep["texts_identical"] and set(rep["modes"]) == {"json", "sse", "sse_via_proxy"}
        for r in rep["modes"].values():
            assert r["status"] == 200 and r["complete"] and r["stop_reason"] == "end_turn" and r["chars"] == len(eng.reply)
            assert r["device_tok_s"] == 1234.5 and r["output_tokens"] == len(eng.reply) + 1 and r["first_content_ms"] is not None
        bad = bench.run(base, model="no-such-model", max_tokens=16)
        assert not bad["ok"] and bad["modes"]["sse"]["status"] == 404
        assert bench.main(["--api", base, "--max-tokens", "64"]) == 0
    finally:
        proxy.shutdown()


def test_stream_ceiling_tool_counts_every_delta(capsys):
    """The host-path ceiling tool streams from an instant fake engine: all tokens arrive as deltas and the rate it
    reports is far above any device rate (the serving layer is not the bottleneck of a single stream)."""
    from naivert_b200.serve.tools import bench_serve_stream
    assert bench_serve_stream.main(["--tokens", "2000", "--per-step", "4"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["tokens"] == 2000 and rep["delta_events"] == 500 and rep["tokens_per_s"] > 5000
