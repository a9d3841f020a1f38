// Incremental parser of a text/event-stream body: feed chunks, get {event, data} objects.
export class SseParser {
  constructor() { this.buf = ""; }
  feed(chunk) {
    this.buf += chunk;
    const out = [];
    let i;
    while ((i = this.buf.indexOf("\n\n")) >= 0) {
      const block = this.buf.slice(0, i);
      this.buf = this.buf.slice(i + 2);
      let event = "message", data = [];
      for (const line of block.split("\n")) {
        if (line.startsWith(":")) continue;                 // keep-alive comment
        if (line.startsWith("event: ")) event = line.slice(7);
        else if (line.startsWith("data: ")) data.push(line.slice(6));
      }
      if (data.length) { try { out.push({ event, data: JSON.parse(data.join("\n")) }); } catch (e) { out.push({ event: "parse_error", data: String(e) }); } }
    }
    return out;
  }
}

// Sliding-window throughput from cumulative token counts: push(t_ms, tokens) -> tokens/s over `windowMs`.
export class Throughput {
  constructor(windowMs = 1000) { this.w = windowMs; this.samples = []; this.peak = 0; }
  push(t, tokens) {
    this.samples.push([t, tokens]);
    while (this.samples.length > 2 && t - this.samples[1][0] >= this.w) this.samples.shift();
    const [t0, n0] = this.samples[0];
    const rate = t > t0 ? (tokens - n0) * 1000 / (t - t0) : 0;
    if (t - t0 >= this.w * 0.9) this.peak = Math.max(this.peak, rate);
    return rate;
  }
}
