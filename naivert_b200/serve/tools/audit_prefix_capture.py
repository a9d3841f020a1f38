"""Audit a request capture for prompt-prefix continuity between consecutive turns.

    python -m naivert_b200.serve.tools.audit_prefix_capture --capture requests.jsonl \
        --pair RID_EARLIER:RID_LATER [--pair ...] --out report.json

The capture is JSON lines: request rows ``{"rid": ..., "body": "<Messages API request JSON>"}`` and response rows
``{"rid": ..., "response": true, "usage": {...}}``.  For each pair the report says whether the later request
extends the earlier one (same system prompt, same tools, earlier messages unchanged) after removing cache hints and
normalising plain-string content to text blocks - i.e. whether the server could have reused the parked prefix -
together with the later turn's usage counters.  Only hashes, counts and block types are written; never bodies.
Parity: tools/serve/audit_cc_prefix_capture.py of the reference.
"""
from __future__ import annotations

import argparse
import hashlib
import json
from pathlib import Path
from typing import Any, Dict, List, Optional


def canonical(value: Any) -> Any:
    """Drop ``cache_control`` keys and turn string content into a one-element text-block list."""
    if isinstance(value, dict):
        out = {k: canonical(v) for k, v in value.items() if k != "cache_control"}
        if isinstance(out.get("content"), str):
            out["content"] = [{"type": "text", "text": out["content"]}]
        return out
    if isinstance(value, list):
        return [canonical(v) for v in value]
    return value


def _digest(value: Any) -> str:
    return hashlib.sha256(json.dumps(canonical(value), sort_keys=True, ensure_ascii=False).encode()).hexdigest()[:16]


def compare_requests(earlier: Dict[str, Any], later: Dict[str, Any], usage: Optional[dict] = None) -> Dict[str, Any]:
    a, b = earlier.get("messages", []), later.get("messages", [])
    shared = len(a)
    first_diff = next((i for i in range(min(len(a), len(b))) if canonical(a[i]) != canonical(b[i])), None)
    if first_diff is None and len(b) < len(a):
        first_diff = len(b)
    added = b[shared:] if first_diff is None else []
    return {
        "earlier_messages": len(a), "later_messages": len(b),
        "messages_prefix_equal": first_diff is None,
        "first_changed_message": first_diff,
        "system_equal": canonical(earlier.get("system")) == canonical(later.get("system")),
        "tools_equal": canonical(earlier.get("tools")) == canonical(later.get("tools")),
        "system_digest": [_digest(earlier.get("system")), _digest(later.get("system"))],
        "tools_digest": [_digest(earlier.get("tools")), _digest(later.get("tools"))],
        "added_roles": [m.get("role") for m in added],
        "added_assistant_block_types": [[blk.get("type") for blk in m["content"]] for m in added
                                        if m.get("role") == "assistant" and isinstance(m.get("content"), list)],
        "later_usage": usage,
    }


def audit(capture: Path, pairs: List[List[str]]) -> Dict[str, Any]:
    wanted = {rid for p in pairs for rid in p}
    bodies: Dict[str, dict] = {}
    usages: Dict[str, Any] = {}
    h = hashlib.sha256()
    with capture.open("rb") as f:
        for line in f:
            h.update(line)
            if not line.strip():
                continue
            row = json.loads(line)
            rid = row.get("rid")
            if rid not in wanted:
                continue
            if row.get("response"):
                usages[rid] = row.get("usage")
            elif row.get("body"):
                bodies[rid] = json.loads(row["body"]) if isinstance(row["body"], str) else row["body"]
    report = {"capture_sha256": h.hexdigest(),
              "scope": "structure only (cache hints stripped, text blocks normalised); sampled token ids are not in a "
                       "capture, so equality here is necessary, not sufficient, for a prefix hit",
              "pairs": []}
    for old, new in pairs:
        missing = [r for r in (old, new) if r not in bodies]
        entry = {"earlier": old, "later": new}
        if missing:
            entry["error"] = f"request body not found for {missing}"
        else:
            entry.update(compare_requests(bodies[old], bodies[new], usages.get(new)))
        report["pairs"].append(entry)
    return report


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--capture", type=Path, required=True)
    ap.add_argument("--pair", action="append", required=True, help="earlier_request_id:later_request_id")
    ap.add_argument("--out", type=Path, required=True)
    a = ap.parse_args()
    pairs = [p.split(":", 1) for p in a.pair]
    report = audit(a.capture, pairs)
    a.out.parent.mkdir(parents=True, exist_ok=True)
    a.out.write_text(json.dumps(report, indent=2) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
