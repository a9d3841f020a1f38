"""Host view of the device control block and stop reasons (mirror of ``csrc/contract.h``).

``tests/test_utils.py::test_contract_header_matches_python`` parses the header and compares, so the two
cannot drift.  Parity: naivert/runtime/mtp_contract.py (``_DecodeControlLayout``), naivert/runtime/sequencer.py.
"""
from __future__ import annotations

import os
import re
from typing import Dict

CTRL_POS = 0
CTRL_COMMITTED = 1
CTRL_INGEST_POS = 2
CTRL_STOPPED = 4
CTRL_REASON = 5
CTRL_GENERATED = 6
CTRL_MAX_TOKENS = 7
CTRL_ROUND = 8
CTRL_CAPACITY = 9
CTRL_CURSOR = 10
CTRL_PROMPT_CTX = 11
CTRL_RELAUNCH_FAIL = 12
CTRL_PAUSED = 13
CTRL_WORDS = 16

STOP_REASONS = {0: None, 1: "eos", 2: "output_limit", 3: "position_limit", 4: "cancelled", 5: "device_wait_failed",
                6: "relaunch_failed"}


def parse_header(path: str = None) -> Dict[str, int]:
    """``NRT_*`` enumerators of ``csrc/contract.h``."""
    path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", "contract.h")
    text = open(path).read()
    return {m.group(1): int(m.group(2)) for m in re.finditer(r"\b(NRT_[A-Z0-9_]+)\s*=\s*(\d+)", text)}
