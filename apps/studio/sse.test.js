// node --test apps/studio/sse.test.js
import assert from "node:assert/strict";
import { test } from "node:test";
import { SseParser, Throughput } from "./sse.js";

test("parser reassembles events across chunk boundaries and skips keep-alives", () => {
  const p = new SseParser();
  const text = ': keepalive\n\nevent: message_start\ndata: {"a":1}\n\nevent: content_block_delta\ndata: {"delta":{"text":"hi"}}\n\n';
  let got = [];
  for (let i = 0; i < text.length; i += 7) got = got.concat(p.feed(text.slice(i, i + 7)));
  assert.deepEqual(got.map((e) => e.event), ["message_start", "content_block_delta"]);
  assert.equal(got[1].data.delta.text, "hi");
});

test("sliding-window throughput and peak", () => {
  const t = new Throughput(1000);
  let r = 0;
  for (let ms = 0; ms <= 3000; ms += 100) r = t.push(ms, ms * 2);      // 2000 tok/s
  assert.ok(Math.abs(r - 2000) < 1);
  assert.ok(Math.abs(t.peak - 2000) < 1);
});
