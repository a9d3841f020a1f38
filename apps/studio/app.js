import { SseParser, Throughput } from "./sse.js";
import { RequestQueue } from "./queue.js";
import { curvePoints, thin } from "./curve.js";
import { renderMarkdown } from "./markdown.js";
import { normalizeBase, buildRequest, assistantTurn, describeHealth, statsLine } from "./core.js";
import { clearAuth, loadAuth, messagesOptions, parseQuickSetup, saveAuth } from "./endpoint.js";
import { HealthWatcher, probeInference } from "./connection.js";

const $ = (id) => document.getElementById(id);
let controller = null;
const history = [];
const base = () => normalizeBase($("base").value);
const auth = () => ({ kind: $("authkind").value, user: $("authuser").value, secret: $("authsecret").value, cookies: $("authcookies").checked });
function showAuth(a) {
  $("authkind").value = a.kind || "none"; $("authuser").value = a.user || ""; $("authsecret").value = a.secret || ""; $("authcookies").checked = Boolean(a.cookies);
}
showAuth(loadAuth($("base").value));
$("base").onchange = () => showAuth(loadAuth($("base").value));
$("quick").onkeydown = (ev) => {
  if (ev.key !== "Enter") return;
  try {
    const q = parseQuickSetup($("quick").value);
    $("base").value = q.endpoint; showAuth(q.auth);
    if (q.model) $("model").value = q.model;
    $("quick").value = ""; $("conn").textContent = "applied; press Check connection";
  } catch (e) { $("conn").textContent = e.message; }
};
$("check").onclick = async () => {
  $("conn").textContent = "checking…";
  try {
    const r = await probeInference({ endpoint: $("base").value, model: $("model").value, auth: auth(), sessionId: $("session").value });
    $("conn").textContent = r.message;
    if (r.ok) saveAuth($("base").value, auth());
  } catch (e) { $("conn").textContent = e.message; }
};
$("forget").onclick = () => { clearAuth(); showAuth({ kind: "none" }); $("conn").textContent = "credentials forgotten"; };

const watcher = new HealthWatcher(() => ({ endpoint: $("base").value, auth: auth() }),
  (state, json) => { $("health").textContent = "health: " + (json ? describeHealth(json) : describeHealth(null)); });
watcher.start();

function drawCurve(points) {
  const c = $("curve"), g = c.getContext("2d");
  g.clearRect(0, 0, c.width, c.height);
  const { points: xy, max } = curvePoints(points, c.width, c.height);
  if (xy.length < 2) return;
  g.beginPath();
  xy.forEach(([x, y], i) => { i ? g.lineTo(x, y) : g.moveTo(x, y); });
  g.strokeStyle = "#3b82f6"; g.stroke();
  g.fillText(`${max.toFixed(0)} tok/s`, 4, 10);
}

async function run(prompt) {
  const out = $("out");
  const span = (cls) => { const s = document.createElement("span"); s.className = cls; out.appendChild(s); return s; };
  out.appendChild(document.createTextNode(`\n> ${prompt}\n`));
  history.push({ role: "user", content: prompt });
  const { body, headers } = buildRequest({ model: $("model").value, maxTokens: +$("max").value, temperature: +$("temp").value,
    topP: +$("topp").value, seed: +$("seed").value, thinking: $("think").checked, session: $("session").value }, history);
  controller = new AbortController();
  const t0 = performance.now();
  const tp = new Throughput(1000), parser = new SseParser();
  let curve = [];
  const blocks = [];
  let current = null, firstContent = null;
  try {
    const opts = messagesOptions(auth(), $("session").value, headers);
    const r = await fetch(base() + "/v1/messages", Object.assign(opts, { signal: controller.signal, body: JSON.stringify(body) }));
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
          current.text += piece;
          if (current.type === "text" && $("md").checked) current.el.innerHTML = renderMarkdown(current.text); else current.el.textContent += piece;
          const n = data.naivert?.generated_tokens;
          if (n !== undefined) { const now = performance.now() - t0; curve.push([now, tp.push(now, n)]); curve = thin(curve, 2000); drawCurve(curve); }
        } else if (event === "message_delta") {
          const tm = data.naivert?.timings || {};
          $("stats").textContent = statsLine(data, tm, { peak: tp.peak, firstMs: firstContent ?? 0, totalMs: performance.now() - t0 });
        } else if (event === "error") { out.appendChild(document.createTextNode(`\n[error] ${data.error?.message}\n`)); }
      }
      out.scrollTop = out.scrollHeight;
    }
    history.push(assistantTurn(blocks));
  } catch (e) { out.appendChild(document.createTextNode(`\n[stopped] ${e.name}\n`)); history.pop(); }
  finally { controller = null; }
}

const queue = new RequestQueue((item) => run(item.prompt));
queue.onChange(({ active, waiting }) => {
  $("queue").innerHTML = (active ? [`<li>▶ ${active.prompt.slice(0, 40)}</li>`] : []).concat(waiting.map((w) => `<li>… ${w.prompt.slice(0, 40)}</li>`)).join("");
});

$("send").onclick = () => { const p = $("prompt").value.trim(); if (!p) return; $("prompt").value = ""; queue.push(p); };
$("stop").onclick = () => controller?.abort();
