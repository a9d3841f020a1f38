// node --test apps/studio/studio.test.js
import test from "node:test";
import assert from "node:assert/strict";
import { RequestQueue } from "./queue.js";
import { curvePoints, thin, summary } from "./curve.js";
import { renderMarkdown, escapeHtml } from "./markdown.js";
import { normalizeBase, buildRequest, assistantTurn } from "./core.js";

test("queue runs one item at a time in order", async () => {
  const seen = [];
  let release;
  const q = new RequestQueue((item) => new Promise((res) => { seen.push(item.prompt); release = res; }));
  q.push("a"); q.push("b"); q.push("c");
  assert.deepEqual(seen, ["a"]);
  assert.equal(q.snapshot().waiting.length, 2);
  assert.equal(q.remove(3), true);
  release(); await new Promise((r) => setTimeout(r, 0));
  assert.deepEqual(seen, ["a", "b"]);
  release(); await new Promise((r) => setTimeout(r, 0));
  assert.equal(q.snapshot().active, null);
});

test("curve geometry", () => {
  const { points, max } = curvePoints([[0, 10], [500, 20], [1000, 5]], 100, 50);
  assert.equal(max, 20);
  assert.deepEqual(points[0], [0, 50 - (10 / 20) * 46]);
  assert.equal(points[2][0], 100);
  assert.equal(thin([...Array(10).keys()].map((i) => [i, i]), 8).length, 8);
  assert.deepEqual(summary([[0, 2], [1, 4]]), { mean: 3, peak: 4 });
});

test("markdown escapes and renders", () => {
  assert.equal(escapeHtml("<a>"), "&lt;a&gt;");
  const html = renderMarkdown("# T\n\nsome **bold** and `x<y`\n\n- one\n- two\n\n```js\nlet a = 1 < 2;\n```");
  assert.ok(html.includes("<h1>T</h1>") && html.includes("<strong>bold</strong>") && html.includes("<code>x&lt;y</code>"));
  assert.ok(html.includes("<ul>") && html.includes("<li>two</li>") && html.includes('class="language-js"') && html.includes("1 &lt; 2"));
  assert.ok(!renderMarkdown("<script>alert(1)</script>").includes("<script>"));
});

test("request building", () => {
  assert.equal(normalizeBase("127.0.0.1:8080/v1/messages/"), "http://127.0.0.1:8080");
  const { body, headers } = buildRequest({ model: "m", maxTokens: 2048, temperature: 0.4, topP: 0.95, seed: 1, thinking: true, session: "s" }, [{ role: "user", content: "hi" }]);
  assert.equal(body.thinking.budget_tokens, 1024);
  assert.equal(headers["x-session-id"], "s");
  const turn = assistantTurn([{ type: "text", text: "ok" }, { type: "tool_use", text: '{"a":1}', block: { id: "t1", name: "f" } }]);
  assert.deepEqual(turn.content[1], { type: "tool_use", id: "t1", name: "f", input: { a: 1 } });
});

import { normalizeEndpoint, apiUrl, authHeaders, messagesOptions, saveAuth, loadAuth, clearAuth, parseQuickSetup } from "./endpoint.js";
import { checkConnection, explainStatus, HealthWatcher } from "./connection.js";

function memoryStorage() {
  const m = new Map();
  return { getItem: (k) => (m.has(k) ? m.get(k) : null), setItem: (k, v) => m.set(k, String(v)), removeItem: (k) => m.delete(k) };
}

test("endpoint is an origin; credentials never ride in the URL", () => {
  assert.equal(normalizeEndpoint(" http://10.0.0.5:8080/v1/messages "), "http://10.0.0.5:8080");
  assert.equal(normalizeEndpoint("api.example.com"), "http://api.example.com");
  assert.equal(normalizeEndpoint(""), "");
  assert.equal(apiUrl("https://h/", "/health"), "https://h/health");
  for (const bad of ["ftp://h", "http://u:p@h", "http://h/?a=1", "http://h/other", "http://h/#x"]) assert.throws(() => normalizeEndpoint(bad));
});

test("auth headers per kind; stored credentials are bound to one origin", () => {
  assert.deepEqual(authHeaders({ kind: "none" }), {});
  assert.deepEqual(authHeaders({ kind: "bearer", secret: "k" }), { authorization: "Bearer k" });
  assert.deepEqual(authHeaders({ kind: "api-key", secret: "k" }), { "x-api-key": "k" });
  assert.equal(authHeaders({ kind: "basic", user: "u", secret: "p" }).authorization, "Basic " + btoa("u:p"));
  assert.throws(() => authHeaders({ kind: "bearer", secret: "" }));
  assert.throws(() => authHeaders({ kind: "bearer", secret: "a\nb" }));
  const o = messagesOptions({ kind: "bearer", secret: "k", cookies: true }, "s1", { "x-naivert-token-progress": "1" });
  assert.equal(o.method, "POST");
  assert.equal(o.headers["x-session-id"], "s1");
  assert.equal(o.credentials, "include");
  const st = memoryStorage();
  assert.equal(saveAuth("http://a:1", { kind: "bearer", secret: "k" }, st), true);
  assert.deepEqual(loadAuth("http://a:1/v1/messages", st), { kind: "bearer", secret: "k", user: "", cookies: false });
  assert.deepEqual(loadAuth("http://b:1", st), { kind: "none" });
  clearAuth(st);
  assert.deepEqual(loadAuth("http://a:1", st), { kind: "none" });
});

test("quick setup line is parsed as data", () => {
  assert.deepEqual(parseQuickSetup("https://h KEY m1"), { endpoint: "https://h", auth: { kind: "bearer", secret: "KEY" }, model: "m1" });
  assert.deepEqual(parseQuickSetup("h:8080"), { endpoint: "http://h:8080", auth: { kind: "none" }, model: null });
  assert.throws(() => parseQuickSetup("a b c d"));
});

function sseResponse(events, status = 200) {
  const text = events.map((e) => `event: ${e}\ndata: {}\n\n`).join("");
  const bytes = new TextEncoder().encode(text);
  let sent = false;
  return { ok: status >= 200 && status < 300, status,
           body: { getReader: () => ({ read: async () => (sent ? { done: true } : (sent = true, { done: false, value: bytes })) }), cancel: async () => {} } };
}

test("connection check goes through the inference route", async () => {
  let seenUrl = null, seenAuth = null;
  const ok = await checkConnection({ endpoint: "http://h:1", model: "m", auth: { kind: "api-key", secret: "k" }, sessionId: "s",
    fetcher: async (url, opt) => { seenUrl = url; seenAuth = opt.headers["x-api-key"]; return sseResponse(["message_start", "content_block_start", "message_delta", "message_stop"]); } });
  assert.equal(ok.ok, true);
  assert.equal(seenUrl, "http://h:1/v1/messages");
  assert.equal(seenAuth, "k");
  const cut = await checkConnection({ endpoint: "http://h:1", model: "m", fetcher: async () => sseResponse(["message_start"]) });
  assert.equal(cut.ok, false);
  const denied = await checkConnection({ endpoint: "http://h:1", model: "m", fetcher: async () => sseResponse([], 401) });
  assert.match(denied.message, /HTTP 401: authentication rejected/);
  const cors = await checkConnection({ endpoint: "http://h:1", model: "m", fetcher: async () => { throw new TypeError("failed to fetch"); } });
  assert.match(cors.message, /CORS/);
  assert.match(explainStatus(529), /queue/);
});

test("health watcher reports changes only and backs off while unreachable", async () => {
  const answers = [() => { throw new TypeError("down"); }, () => { throw new TypeError("down"); },
                   () => ({ ok: true, json: async () => ({ status: "loading" }) }), () => ({ ok: true, json: async () => ({ status: "ok", slot: "IDLE" }) }),
                   () => ({ ok: true, json: async () => ({ status: "ok", slot: "IDLE" }) })];
  const seen = [];
  let calls = 0, lastUrl = null, lastHeaders = null;
  const w = new HealthWatcher(() => ({ endpoint: "http://h:1", auth: { kind: "bearer", secret: "k" } }), (state) => seen.push(state),
    { fetcher: async (url, opt) => { lastUrl = url; lastHeaders = opt.headers; return answers[calls++](); }, baseMs: 100, maxMs: 350 });
  await w.pollOnce(); assert.equal(w.delay, 200);
  await w.pollOnce(); assert.equal(w.delay, 350);
  await w.pollOnce(); assert.equal(w.delay, 100);
  await w.pollOnce(); await w.pollOnce();
  assert.deepEqual(seen, ["unreachable", "loading", "ok"]);
  assert.equal(lastUrl, "http://h:1/health");
  assert.equal(lastHeaders.authorization, "Bearer k");
});
