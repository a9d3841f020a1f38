// Two ways of knowing whether the server is there.
//
// probeInference(): a one-token streamed request through /v1/messages.  Gateways in front of the server often expose
// neither /health nor /v1/models, so the inference route itself is what proves endpoint, credentials, model name and
// CORS at once.
//
// HealthWatcher: polls /health while the page is open; backs off (2 s -> 30 s) while the server is unreachable and
// reports only changes of state.
import { SseParser } from "./sse.js";
import { apiUrl, authHeaders, messagesOptions } from "./endpoint.js";

const STATUS_TEXT = new Map([
  [401, "authentication rejected: check the credentials"],
  [403, "authentication rejected: check the credentials"],
  [404, "unknown model or route: check the model name and the endpoint"],
  [429, "server reachable, its queue or rate limit is full"],
  [529, "server reachable, its queue or rate limit is full"],
  [503, "server reachable, still loading or shutting down"],
]);

export function explainStatus(status) {
  return STATUS_TEXT.get(status) || "request rejected: check the model and the gateway configuration";
}

async function eventNames(response) {
  const names = [];
  const parser = new SseParser(), utf8 = new TextDecoder();
  const reader = response.body.getReader();
  for (let chunk = await reader.read(); !chunk.done; chunk = await reader.read()) {
    for (const ev of parser.feed(utf8.decode(chunk.value, { stream: true }))) names.push(ev.event);
  }
  return names;
}

function streamIsComplete(names) {
  if (names.includes("error")) return false;
  return names.length >= 3 && names[0] === "message_start" && names[names.length - 1] === "message_stop" && names.includes("message_delta");
}

export async function probeInference(cfg) {
  const fetcher = cfg.fetcher || globalThis.fetch.bind(globalThis);
  const limitMs = cfg.timeoutMs === undefined ? 20000 : cfg.timeoutMs;
  const clock = cfg.now || (() => Date.now());
  const abort = new AbortController();
  const timer = setTimeout(() => abort.abort(), limitMs);
  const started = clock();
  const request = Object.assign(messagesOptions(cfg.auth, cfg.sessionId), {
    signal: abort.signal,
    body: JSON.stringify({ model: cfg.model, max_tokens: 1, stream: true, thinking: { type: "disabled" },
                           messages: [{ role: "user", content: "Reply OK." }] }),
  });
  try {
    const response = await fetcher(apiUrl(cfg.endpoint, "/v1/messages"), request);
    if (!response.ok) {
      if (response.body && response.body.cancel) { try { await response.body.cancel(); } catch (e) { /* already closed */ } }
      return { ok: false, message: `HTTP ${response.status}: ${explainStatus(response.status)}` };
    }
    if (!streamIsComplete(await eventNames(response))) return { ok: false, message: "the server answered, but the Messages stream did not complete" };
    return { ok: true, message: `connected, streaming verified in ${((clock() - started) / 1000).toFixed(2)} s` };
  } catch (e) {
    if (abort.signal.aborted) return { ok: false, message: `no answer within ${limitMs / 1000} s: the server may be queued or down` };
    if (e instanceof TypeError) return { ok: false, message: "the browser cannot reach the API: check CORS / OPTIONS on the gateway, HTTPS and the network" };
    return { ok: false, message: "the server answered with an invalid Messages stream" };
  } finally { clearTimeout(timer); }
}
export const checkConnection = probeInference;

export class HealthWatcher {
  // getTarget() -> { endpoint, auth }; onChange(state, json) is called when the state string changes.
  constructor(getTarget, onChange, opts = {}) {
    this.getTarget = getTarget; this.onChange = onChange;
    this.fetcher = opts.fetcher || ((...a) => globalThis.fetch(...a));
    this.baseMs = opts.baseMs || 2000; this.maxMs = opts.maxMs || 30000;
    this.delay = this.baseMs; this.state = null; this.timer = null; this.stopped = true;
    this.schedule = opts.schedule || ((fn, ms) => setTimeout(fn, ms));
  }
  async pollOnce() {
    let state = "unreachable", json = null;
    try {
      const { endpoint, auth } = this.getTarget();
      let headers = {};
      try { headers = authHeaders(auth); } catch (e) { headers = {}; }
      const r = await this.fetcher(apiUrl(endpoint, "/health"), { headers });
      json = await r.json();
      state = String(json.status || (r.ok ? "ok" : "error"));
    } catch (e) { state = "unreachable"; }
    this.delay = state === "unreachable" ? Math.min(this.maxMs, this.delay * 2) : this.baseMs;
    if (state !== this.state) { this.state = state; this.onChange(state, json); }
    return state;
  }
  start() {
    if (!this.stopped) return;
    this.stopped = false;
    const tick = async () => { if (this.stopped) return; await this.pollOnce(); if (!this.stopped) this.timer = this.schedule(tick, this.delay); };
    tick();
  }
  stop() { this.stopped = true; if (this.timer !== null && typeof clearTimeout === "function") clearTimeout(this.timer); this.timer = null; }
}
