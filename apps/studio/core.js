// Connection and request helpers shared by the page and the tests (no DOM).
export function normalizeBase(url) {
  let u = (url || "").trim();
  if (!u) return "";
  if (!/^https?:\/\//i.test(u)) u = "http://" + u;
  return u.replace(/\/+$/, "").replace(/\/v1(\/messages)?$/, "");
}
export function buildRequest(form, history) {
  const body = { model: form.model, max_tokens: form.maxTokens, temperature: form.temperature, top_p: form.topP,
                 seed: form.seed, stream: true, messages: history.slice() };
  if (form.system) body.system = form.system;
  if (form.thinking) body.thinking = { type: "enabled", budget_tokens: Math.max(1024, Math.min(form.thinkingBudget || 1024, form.maxTokens - 1)) };
  if (form.stop && form.stop.length) body.stop_sequences = form.stop.slice(0, 8);
  const headers = { "content-type": "application/json", "x-naivert-token-progress": "1" };
  if (form.session) headers["x-session-id"] = form.session;
  return { body, headers };
}
// Fold the streamed blocks of one reply into the assistant turn that goes back into the history.
export function assistantTurn(blocks) {
  const content = [];
  for (const b of blocks) {
    if (b.type === "text" && b.text) content.push({ type: "text", text: b.text });
    else if (b.type === "thinking") content.push({ type: "thinking", thinking: b.text, signature: "" });
    else if (b.type === "tool_use") { let input = {}; try { input = JSON.parse(b.text || "{}"); } catch (e) { input = {}; } content.push({ type: "tool_use", id: b.block.id, name: b.block.name, input }); }
  }
  return { role: "assistant", content };
}
export function describeHealth(j) {
  if (!j) return "unreachable";
  return `${j.status}${j.slot ? " slot=" + j.slot : ""}${j.queued !== undefined ? " queued=" + j.queued : ""}`;
}
export function statsLine(delta, timings, extra) {
  const u = delta.usage || {};
  return [`stop=${delta.delta?.stop_reason ?? "?"}`, `out=${u.output_tokens ?? "?"}`, `cache_read=${u.cache_read_input_tokens ?? 0}`,
          `device=${timings?.decode_tok_s_device ?? "?"} tok/s`, `peak1s=${extra.peak.toFixed(0)} tok/s`,
          `first=${extra.firstMs.toFixed(0)} ms`, `total=${extra.totalMs.toFixed(0)} ms`].join(" ");
}
