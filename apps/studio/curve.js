// Throughput curve geometry: (time ms, tokens/s) samples -> points of a polyline inside a w x h box, newest at the
// right edge, scaled to the largest sample (at least `floor` tokens/s so an idle curve is flat, not noisy).
export function curvePoints(samples, w, h, floor = 1) {
  if (samples.length < 2) return { points: [], max: floor };
  const t0 = samples[0][0], t1 = samples[samples.length - 1][0];
  const span = Math.max(t1 - t0, 1e-9);
  let max = floor;
  for (const [, v] of samples) if (v > max) max = v;
  const points = samples.map(([t, v]) => [((t - t0) / span) * w, h - (v / max) * (h - 4)]);
  return { points, max };
}
// Keep at most `limit` samples by dropping every second one of the older half (the recent end stays dense).
export function thin(samples, limit) {
  if (samples.length <= limit) return samples;
  const half = samples.length >> 1;
  return samples.filter((_, i) => i >= half || i % 2 === 0);
}
export function summary(samples) {
  if (!samples.length) return { mean: 0, peak: 0 };
  let sum = 0, peak = 0;
  for (const [, v] of samples) { sum += v; if (v > peak) peak = v; }
  return { mean: sum / samples.length, peak };
}
