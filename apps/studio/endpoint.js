// Where the API lives and how requests authenticate (no DOM; storage is injectable for the tests).
// The base may be a bare origin or the full Messages URL; credentials are remembered for one origin only, so a
// key typed for one server is never sent to another.

const ALLOWED_PATHS = ["", "/", "/v1", "/v1/", "/v1/messages", "/v1/messages/"];
const STORE_KEY = "naivert-b200-studio-auth";
const AUTH_KINDS = ["none", "bearer", "api-key", "basic"];

export function normalizeEndpoint(value) {
  const raw = (value || "").trim();
  if (!raw) return "";
  let url;
  try { url = new URL(/^https?:\/\//i.test(raw) ? raw : "http://" + raw); } catch (e) { throw new Error("not a URL: " + raw); }
  if (url.protocol !== "http:" && url.protocol !== "https:") throw new Error("only http and https endpoints");
  if (url.username || url.password) throw new Error("put credentials in the auth fields, not in the URL");
  if (url.search || url.hash) throw new Error("endpoint without query or fragment");
  if (!ALLOWED_PATHS.includes(url.pathname)) throw new Error("endpoint is an origin or its /v1/messages URL");
  return url.origin;
}

export function apiUrl(endpoint, path) {
  return normalizeEndpoint(endpoint) + path;
}

export function checkAuth(auth) {
  const a = auth || { kind: "none" };
  if (!AUTH_KINDS.includes(a.kind || "none")) throw new Error("unknown auth kind " + a.kind);
  if (a.kind === "basic" && (!a.user || /:/.test(a.user))) throw new Error("basic auth needs a user name without ':'");
  if (a.kind && a.kind !== "none" && !a.secret) throw new Error("the secret is empty");
  if (/[\r\n]/.test((a.secret || "") + (a.user || ""))) throw new Error("line breaks in credentials");
  return a;
}

export function authHeaders(auth) {
  const a = checkAuth(auth);
  if (a.kind === "bearer") return { authorization: "Bearer " + a.secret };
  if (a.kind === "api-key") return { "x-api-key": a.secret };
  if (a.kind === "basic") return { authorization: "Basic " + btoa(unescape(encodeURIComponent(a.user + ":" + a.secret))) };
  return {};
}

// fetch() options of a Messages request: JSON body, optional session id, credentials.
export function messagesOptions(auth, sessionId, extraHeaders) {
  const headers = Object.assign({ "content-type": "application/json" }, authHeaders(auth), extraHeaders || {});
  if (sessionId) headers["x-session-id"] = sessionId;
  return { method: "POST", headers, credentials: auth && auth.cookies ? "include" : "same-origin" };
}

export function saveAuth(endpoint, auth, storage) {
  try {
    const origin = normalizeEndpoint(endpoint);
    if (!origin) return false;
    const a = checkAuth(auth);
    const clean = { kind: a.kind || "none", secret: a.kind && a.kind !== "none" ? a.secret : "", user: a.kind === "basic" ? a.user : "", cookies: Boolean(a.cookies) };
    (storage || globalThis.localStorage).setItem(STORE_KEY, JSON.stringify({ origin, auth: clean }));
    return true;
  } catch (e) { return false; }
}

export function loadAuth(endpoint, storage) {
  try {
    const saved = JSON.parse((storage || globalThis.localStorage).getItem(STORE_KEY));
    if (!saved || !endpoint || saved.origin !== normalizeEndpoint(endpoint)) return { kind: "none" };
    return checkAuth(saved.auth);
  } catch (e) { return { kind: "none" }; }
}

export function clearAuth(storage) {
  try { (storage || globalThis.localStorage).removeItem(STORE_KEY); return true; } catch (e) { return false; }
}

// "URL [KEY [MODEL]]" pasted in one line; parsed as data only.
export function parseQuickSetup(line) {
  const parts = (line || "").trim().split(/\s+/).filter(Boolean);
  if (parts.length < 1 || parts.length > 3) throw new Error("paste: URL [API_KEY [MODEL]]");
  const auth = parts[1] ? { kind: "bearer", secret: parts[1] } : { kind: "none" };
  return { endpoint: normalizeEndpoint(parts[0]), auth: checkAuth(auth), model: parts[2] || null };
}
