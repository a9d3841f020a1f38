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
