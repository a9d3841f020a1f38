import { SseParser, Throughput } from "./sse.js";

const $ = (id) => document.getElementById(id);
let controller = null;
const history = [];
const pending = [];

async function health() {
  try {
    const r = await fetch($("base").value + "/health");
    const j = await r.json();
    $("health").textContent = `health: ${j.status} slot=${j.slot} queued=${j.queued}`;
  } catch (e) { $("health").textContent = "health: unreachable"; }
}
setInterval(health, 2000); health();

function drawCurve(points) {
  const c = $("curve"), g = c.getContext("2d");
  g.clearRect(0, 0, c.width, c.height);
  if (points.length < 2) return;
  const max = Math.max(...points.map((p) => p[1]), 1), t0 = points[0][0], t1 = points[points.length - 1][0] || 1;
  g.beginPath();
  points.forEach(([t, v], i) => { const x = (t - t0) / (t1 - t0 || 1) * c.width, y = c.height - v / max * (c.height - 4); i ? g.lineTo(x, y) : g.moveTo(x, y); });
  g.strokeStyle = "#3b82f6"; g.stroke();
  g.fillText(`${max.toFixed(0)} tok/s`, 4, 10);
}

async function run(prompt) {
  const out = $("out");
  const span = (cls) => { const s = document.createElement("span"); s.className = cls; out.appendChild(s); return s; };
  out.appendChild(document.createTextNode(`\n> ${prompt}\n`));
  history.push({ role: "user", content: prompt });
  const body = { model: $("model").value, max_tokens: +$("max").value, temperature: +$("temp").value, top_p: +$("topp").value,
                 seed: +$("seed").value, stream: true, messages: history.slice() };
  if ($("think").checked) body.thinking = { type: "enabled", budget_tokens: 1024 };
  controller = new AbortController();
  const t0 = performance.now();
  const tp = new Throughput(1000), parser = new SseParser(), curve = [];
  const blocks = [];
  let current = null, firstContent = null;
  try {
    const r = await fetch($("base").value + "/v1/messages", { method: "POST", signal: controller.signal,
      headers: { "content-type": "application/json", "x-session-id": $("session").value, "x-naivert-token-progress": "1" }, body: JSON.stringify(body) });
    if (!r.ok) { out.appendChild(document.createTextNode(`[${r.status}] ${await r.text()}\n`)); history.pop(); return; }
    const reader = r.body.getReader(), dec = new TextDecoder();
    for (;;) {
      const { done, value } = await reader.read();
      if (done) break;
      for (const { event, data } of parser.feed(dec.decode(value, { stream: true }))) {
        if (event === "content_block_start") { current = { type: data.content_block.type, el: span(data.content_block.type === "thinking" ? "think" : data.content_block.type === "tool_use" ? "tool" : ""), text: "", block: data.content_block }; blocks.push(current); }
        else if (event === "content_block_delta") {
          const d = data.delta, piece = d.text ?? d.thinking ?? d.partial_json ?? "";
          if (firstContent === null) firstContent = performance.now() - t0;
          current.text += piece; current.el.textContent += piece;
          const n = data.naivert?.generated_tokens;
          if (n !== undefined) { const now = performance.now() - t0; curve.push([now, tp.push(now, n)]); drawCurve(curve); }
        } else if (event === "message_delta") {
          const tm = data.naivert?.timings || {};
          $("stats").textContent = `stop=${data.delta.stop_reason} out=${data.usage.output_tokens} cache_read=${data.usage.cache_read_input_tokens} ` +
            `device=${tm.decode_tok_s_device ?? "?"} tok/s peak1s=${tp.peak.toFixed(0)} tok/s first=${(firstContent ?? 0).toFixed(0)} ms total=${(performance.now() - t0).toFixed(0)} ms`;
        } else if (event === "error") { out.appendChild(document.createTextNode(`\n[error] ${data.error?.message}\n`)); }
      }
      out.scrollTop = out.scrollHeight;
    }
    history.push({ role: "assistant", content: blocks.map((b) => b.type === "thinking" ? { type: "thinking", thinking: b.text } : b.type === "tool_use" ? { ...b.block, input: JSON.parse(b.text || "{}") } : { type: "text", text: b.text }) });
  } catch (e) { out.appendChild(document.createTextNode(`\n[stopped] ${e.name}\n`)); history.pop(); }
  finally { controller = null; }
}

async function drain() {
  while (pending.length) {
    const p = pending[0];
    renderQueue();
    await run(p);
    pending.shift();
    renderQueue();
  }
}
function renderQueue() { $("queue").innerHTML = pending.map((p, i) => `<li>${i === 0 ? "▶" : "…"} ${p.slice(0, 40)}</li>`).join(""); }

$("send").onclick = () => { const p = $("prompt").value.trim(); if (!p) return; $("prompt").value = ""; pending.push(p); if (pending.length === 1) drain(); else renderQueue(); };
$("stop").onclick = () => controller?.abort();
