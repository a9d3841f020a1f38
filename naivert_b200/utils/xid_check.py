"""GPU fault check for test runs: compare two snapshots of the kernel log and fail on NVIDIA driver fault
lines (``NVRM: Xid``) that appeared in between.

A kernel that faults can leave the process alive (sticky context error seen only at the next call, or not at
all when the faulting work belonged to a child).  The driver logs every such event; a run that is clean by exit
code but added Xid lines is not clean.  Usage::

    python -m naivert_b200.utils.xid_check snapshot before.txt
    ... run the GPU tests ...
    python -m naivert_b200.utils.xid_check snapshot after.txt
    python -m naivert_b200.utils.xid_check compare before.txt after.txt     # exit 1 and the new lines on a fault

``snapshot`` reads ``dmesg`` (or the file named by ``--source``); where the kernel log is not readable it writes
an empty snapshot with a marker line and ``compare`` reports "unknown" (exit 0 unless ``--strict``).
Reference counterpart: tests/support/check_xid_delta.py.
"""
from __future__ import annotations

import argparse
import re
import subprocess
import sys
from typing import List, Optional

XID = re.compile(r"NVRM: Xid \(PCI:[0-9a-fA-F:.]+\): (\d+)")
UNREADABLE = "# kernel log unreadable"
_STAMP = re.compile(r"^\[\s*\d+\.\d+\]\s*")


def read_kernel_log(source: Optional[str] = None) -> Optional[str]:
    if source:
        try:
            return open(source, errors="replace").read()
        except OSError:
            return None
    try:
        p = subprocess.run(["dmesg"], capture_output=True, text=True, timeout=20)
    except (OSError, subprocess.TimeoutExpired):
        return None
    return p.stdout if p.returncode == 0 else None


def xid_lines(text: str) -> List[str]:
    return [ln for ln in text.splitlines() if XID.search(ln)]


def new_xid_lines(before: str, after: str) -> List[str]:
    """Fault lines of ``after`` that ``before`` does not have.  Lines are matched with their multiplicity (the
    same fault text can legitimately repeat), so a ring-buffer log that dropped old lines gives no false alarms."""
    left = {}
    for ln in xid_lines(before):
        left[ln] = left.get(ln, 0) + 1
    fresh = []
    for ln in xid_lines(after):
        if left.get(ln, 0) > 0:
            left[ln] -= 1
        else:
            fresh.append(ln)
    return fresh


def xid_codes(lines: List[str]) -> List[int]:
    return [int(XID.search(ln).group(1)) for ln in lines]


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("snapshot")
    s.add_argument("out")
    s.add_argument("--source", default=None, help="read this file instead of dmesg")
    c = sub.add_parser("compare")
    c.add_argument("before")
    c.add_argument("after")
    c.add_argument("--strict", action="store_true", help="an unreadable kernel log is a failure")
    a = ap.parse_args(argv)
    if a.cmd == "snapshot":
        text = read_kernel_log(a.source)
        with open(a.out, "w") as f:
            f.write(UNREADABLE + "\n" if text is None else "\n".join(xid_lines(text)) + "\n")
        return 0
    before, after = open(a.before).read(), open(a.after).read()
    if UNREADABLE in before or UNREADABLE in after:
        print("xid check: unknown (kernel log unreadable)")
        return 1 if a.strict else 0
    fresh = new_xid_lines(before, after)
    if fresh:
        print(f"xid check: {len(fresh)} new GPU fault line(s), codes {sorted(set(xid_codes(fresh)))}")
        for ln in fresh:
            print("  " + ln)
        return 1
    print("xid check: clean")
    return 0


if __name__ == "__main__":
    sys.exit(main())
