// Connection check through the inference route itself: gateways in front of the server often expose neither
// /health nor /v1/models, so a one-token streamed request is what proves that the endpoint, the credentials, the
// model name and CORS are right.
import { SseParser } from "./sse.js";
import { apiUrl, messagesOptions } from "./endpoint.js";

export function explainStatus(status) {
  if (status === 401 || status === 403) return "authentication rejected: check the credentials";
  if (status === 404) return "unknown model or route: check the model name and the endpoint";
  if (status === 429 || status === 529) return "server reachable, its queue or rate limit is full";
  if (status === 503) return "server reachable, still loading or shutting down";
  return "request rejected: check the model and the gateway configuration";
}

export async function checkConnection({ endpoint, model, auth, sessionId, fetcher, timeoutMs = 20000, now = () => Date.now() }) {
  const doFetch = fetcher || globalThis.fetch.bind(globalThis);
  const controller = new AbortController();
  const timer = setTimeout(() => controller.abort(), timeoutMs);
  const t0 = now();
  try {
    const body = { model, max_tokens: 1, stream: true, thinking: { type: "disabled" }, messages: [{ role: "user", content: "Reply OK." }] };
    const r = await doFetch(apiUrl(endpoint, "/v1/messages"), Object.assign(messagesOptions(auth, sessionId), { signal: controller.signal, body: JSON.stringify(body) }));
    if (!r.ok) {
      if (r.body && r.body.cancel) { try { await r.body.cancel(); } catch (e) { /* already closed */ } }
      return { ok: false, message: `HTTP ${r.status}: ${explainStatus(r.status)}` };
    }
    const parser = new SseParser(), dec = new TextDecoder();
    const seen = [];
    const reader = r.body.getReader();
    for (;;) {
      const { done, value } = await reader.read();
      if (done) break;
      for (const { event } of parser.feed(dec.decode(value, { stream: true }))) seen.push(event);
    }
    const complete = seen[0] === "message_start" && seen.includes("message_delta") && seen[seen.length - 1] === "message_stop" && !seen.includes("error");
    if (!complete) return { ok: false, message: "the server answered, but the Messages stream did not complete" };
    return { ok: true, message: `connected, streaming verified in ${((now() - t0) / 1000).toFixed(2)} s` };
  } catch (e) {
    if (controller.signal.aborted) return { ok: false, message: `no answer within ${timeoutMs / 1000} s: the server may be queued or down` };
    if (e instanceof TypeError) return { ok: false, message: "the browser cannot reach the API: check CORS / OPTIONS on the gateway, HTTPS and the network" };
    return { ok: false, message: "the server answered with an invalid Messages stream" };
  } finally { clearTimeout(timer); }
}
