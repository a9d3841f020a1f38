"""The single generation slot as a small finite-state machine.

IDLE -> PROCESSING_PROMPT -> GENERATING -> DONE -> IDLE, with CANCELLED and ERROR side exits;
ERROR must be RESET (which invalidates the cached sequence) before the slot is IDLE again.
Parity: naivert/serve/slot.py (states :16-61, ``ServerSlot`` :68-182).
"""
from __future__ import annotations

from enum import Enum
from typing import Dict, Optional, Sequence, Tuple

from .tokens import ServerTokens


class SlotState(Enum):
    IDLE = "IDLE"
    PROCESSING_PROMPT = "PROCESSING_PROMPT"
    GENERATING = "GENERATING"
    DONE = "DONE"
    CANCELLED = "CANCELLED"
    ERROR = "ERROR"


class SlotEvent(Enum):
    START = "start"
    PROMPT_DONE = "prompt_done"
    FINISH = "finish"
    CANCEL = "cancel"
    FAIL = "fail"
    RELEASE = "release"
    RESET = "reset"


_T: Dict[Tuple[SlotState, SlotEvent], SlotState] = {
    (SlotState.IDLE, SlotEvent.START): SlotState.PROCESSING_PROMPT,
    (SlotState.PROCESSING_PROMPT, SlotEvent.PROMPT_DONE): SlotState.GENERATING,
    (SlotState.GENERATING, SlotEvent.FINISH): SlotState.DONE,
    (SlotState.PROCESSING_PROMPT, SlotEvent.CANCEL): SlotState.CANCELLED,
    (SlotState.GENERATING, SlotEvent.CANCEL): SlotState.CANCELLED,
    (SlotState.DONE, SlotEvent.RELEASE): SlotState.IDLE,
    (SlotState.CANCELLED, SlotEvent.RELEASE): SlotState.IDLE,
    (SlotState.ERROR, SlotEvent.RESET): SlotState.IDLE,
}
for _s in SlotState:
    if _s is not SlotState.ERROR:
        _T[(_s, SlotEvent.FAIL)] = SlotState.ERROR


class IllegalSlotTransition(RuntimeError):
    pass


class ServerSlot:
    def __init__(self):
        self.state = SlotState.IDLE
        self.cache_tokens = ServerTokens()        # sequence the engine holds KV for
        self.task_id: Optional[int] = None
        self.n_past = 0
        self.n_decoded = 0
        self.error: Optional[BaseException] = None

    def can(self, ev: SlotEvent) -> bool:
        return (self.state, ev) in _T

    def transition(self, ev: SlotEvent) -> SlotState:
        nxt = _T.get((self.state, ev))
        if nxt is None:
            raise IllegalSlotTransition(f"{ev.value} is not allowed in state {self.state.value}")
        self.state = nxt
        return nxt

    def start(self, task_id: int, prompt_tokens: Sequence[int]) -> int:
        """Begin a request; returns the number of cached tokens the prompt can reuse."""
        self.transition(SlotEvent.START)
        self.task_id, self.n_decoded = task_id, 0
        self.n_past = self.cache_tokens.common_prefix(prompt_tokens)
        return self.n_past

    def prompt_done(self, prompt_tokens: Sequence[int]) -> None:
        self.cache_tokens = ServerTokens(prompt_tokens)
        self.transition(SlotEvent.PROMPT_DONE)

    def add_tokens(self, toks: Sequence[int]) -> None:
        self.cache_tokens.extend(toks)
        self.n_decoded += len(toks)

    def finish(self) -> None:
        self.transition(SlotEvent.FINISH)

    def cancel(self) -> None:
        self.transition(SlotEvent.CANCEL)

    def release(self) -> None:
        self.transition(SlotEvent.RELEASE)
        self.task_id = None

    def fail(self, err: BaseException) -> None:
        self.error = err
        self.transition(SlotEvent.FAIL)

    def reset(self) -> None:
        self.transition(SlotEvent.RESET)
        self.cache_tokens.clear()
        self.task_id, self.n_past, self.n_decoded, self.error = None, 0, 0, None
