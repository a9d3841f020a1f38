"""Token bookkeeping of the serving slot: the cached token sequence and client stop strings.

Parity: naivert/serve/tokens.py (``ServerTokens`` :9, ``StopMatcher`` :107).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence


class ServerTokens:
    """The token sequence the engine currently holds state for (prompt + generated)."""

    def __init__(self, tokens: Iterable[int] = ()):
        self._t: List[int] = [int(x) for x in tokens]

    def __len__(self):
        return len(self._t)

    def __iter__(self):
        return iter(self._t)

    def __getitem__(self, i):
        return self._t[i]

    def as_list(self) -> List[int]:
        return list(self._t)

    def push_back(self, tok: int) -> None:
        self._t.append(int(tok))

    def extend(self, toks: Iterable[int]) -> None:
        self._t.extend(int(x) for x in toks)

    def clear(self) -> None:
        self._t.clear()

    def keep_first(self, n: int) -> None:
        if not 0 <= n <= len(self._t):
            raise ValueError(f"cannot keep {n} of {len(self._t)} tokens")
        del self._t[n:]

    def common_prefix(self, other: Sequence[int]) -> int:
        n = 0
        for a, b in zip(self._t, other):
            if a != b:
                break
            n += 1
        return n

    def validate(self, vocab: int) -> bool:
        return all(0 <= t < vocab for t in self._t)


@dataclass
class StopMatch:
    stop: str
    start: int           # character offset of the match in the full output text
    end: int

    def cut(self, inclusive: bool) -> int:
        return self.end if inclusive else self.start


class StopMatcher:
    """Finds the earliest client stop string in a growing output text and says how many
    trailing characters must be held back because they may still grow into one."""

    def __init__(self, stops: Sequence[str] = (), inclusive: bool = False):
        self.stops = [s for s in stops if s]
        self.inclusive = inclusive
        self.text = ""

    def reset(self) -> None:
        self.text = ""

    def feed(self, new_text: str) -> Optional[StopMatch]:
        before = len(self.text)
        self.text += new_text
        best: Optional[StopMatch] = None
        for s in self.stops:
            i = self.text.find(s, max(0, before - len(s) + 1))
            if i >= 0 and (best is None or i < best.start):
                best = StopMatch(s, i, i + len(s))
        return best

    def holdback(self) -> int:
        hold = 0
        for s in self.stops:
            for n in range(min(len(s) - 1, len(self.text)), hold, -1):
                if self.text.endswith(s[:n]):
                    hold = n
                    break
        return hold
