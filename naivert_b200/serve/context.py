"""Request execution on the inference worker thread: tokenise, open an engine session, pump
tokens through detokeniser -> stop matcher -> segment splitter, and report usage and timings.

The engine is a duck type (the seam the tests fake):

    engine.config            -> object with ``capacity``, ``max_output_tokens``, ``eos_token_ids``
    engine.align_prompt(tokens, session_id) -> tokens      (keeps sampled ids of a resumed session)
    engine.open_session(tokens, max_decode, session_id, sampling) -> session
    session.cached_tokens / session.prefill_info
    session.step(timeout_s) -> list[int] (possibly empty) ; session.done ; session.stop_reason
    session.cancel() ; session.finish() -> dict of device statistics

Parity: ``ServerContext.handle_completion`` (naivert/serve/context.py:108-321) and the result
types of naivert/serve/task.py.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional

from .chat import ChatFormatter, IncrementalDetokenizer
from .messages_api import ApiError, TaskParams
from .slot import ServerSlot, SlotState
from .syntax import SegmentStream
from .timeline import RequestTimeline
from .tokens import StopMatcher


@dataclass
class Opened:
    prompt_tokens: int
    cached_tokens: int
    ignored: List[str]


@dataclass
class Partial:
    kind: str
    text: str
    closed: bool
    generated_tokens: int


@dataclass
class Final:
    stop_reason: str
    stop_sequence: Optional[str]
    output_tokens: int
    thinking_tokens: int
    timings: Dict[str, Any]
    tokens: List[int] = field(default_factory=list)


class ServerContext:
    def __init__(self, engine: Any, formatter: ChatFormatter, step_timeout_s: float = 120.0):
        self.engine, self.formatter, self.step_timeout_s = engine, formatter, step_timeout_s
        self.slot = ServerSlot()
        self.owner = threading.get_ident()
        self._task_seq = 0

    # ------------------------------------------------------------------
    def count_tokens(self, p: TaskParams) -> int:
        return len(self.formatter.encode(p.messages, p.tools, p.thinking))

    def _check_owner(self) -> None:
        if threading.get_ident() != self.owner:
            raise RuntimeError("the serving context is used from a thread that does not own it")

    def handle_completion(self, p: TaskParams, timeline: Optional[RequestTimeline] = None,
                          cancelled: Optional[threading.Event] = None) -> Iterator[Any]:
        """Generator of Opened, Partial..., Final.  Raises ApiError for request-level refusals."""
        self._check_owner()
        tl = timeline or RequestTimeline()
        cancelled = cancelled or threading.Event()
        cfg = self.engine.config
        if self.slot.state is SlotState.ERROR:
            self.slot.reset()
        with tl.span("Worker", "format_tokenize"):
            tokens = self.formatter.encode(p.messages, p.tools, p.thinking)
            try:
                # engines that keep sampled ids of a parked history compare decoded text, not ids
                text = self.formatter.render(p.messages, p.tools, p.thinking)
                tokens = list(self.engine.align_prompt(tokens, p.session_id, text=text))
            except TypeError:
                tokens = list(self.engine.align_prompt(tokens, p.session_id))
        ignored = list(p.ignored)
        room = cfg.capacity - 16 - len(tokens)
        if room < 1:
            raise ApiError(400, "context_exceeded", f"prompt of {len(tokens)} tokens does not fit capacity {cfg.capacity}")
        max_decode = p.max_tokens
        if max_decode > room:
            max_decode = room
            ignored.append("max_tokens_clamped")
        self._task_seq += 1
        with tl.span("Worker", "cache_lookup"):
            self.slot.start(self._task_seq, tokens)
        session = None
        try:
            t_open = time.monotonic()
            with tl.span("Prefill", "open_session", prompt_tokens=len(tokens)):
                session = self.engine.open_session(tokens, max_decode, p.session_id, p.sampling)
            prefill_ms = (time.monotonic() - t_open) * 1e3
            cached = int(getattr(session, "cached_tokens", 0))
            self.slot.prompt_done(tokens)
            yield Opened(len(tokens), cached, ignored)

            detok = IncrementalDetokenizer(self.formatter.tok, skip_special_tokens=False)
            stops = StopMatcher(p.stop_sequences, inclusive=p.stop_inclusive)
            segs = SegmentStream(thinking=p.thinking, tools=bool(p.tool_schemas))
            if p.thinking:
                segs.feed("<think>")                        # the template already opened the block
            eos = set(getattr(cfg, "eos_token_ids", ()) or ())
            out_tokens: List[int] = []
            released = 0                                     # characters of stops.text already forwarded
            thinking_tokens = 0
            stop_reason, stop_seq = None, None
            t_dec = time.monotonic()
            while stop_reason is None:
                if cancelled.is_set():
                    session.cancel()
                    stop_reason = "cancelled"
                    break
                with tl.span("Token step", "step"):
                    new = session.step(self.step_timeout_s)
                piece = ""
                for t in new:
                    out_tokens.append(t)
                    if segs.kind == "thinking":
                        thinking_tokens += 1
                    if t in eos:
                        stop_reason = "eos"
                        break
                    piece += detok.add(t)
                self.slot.add_tokens(new)
                if piece:
                    hit = stops.feed(piece)
                    if hit is not None:
                        cut = hit.cut(p.stop_inclusive)
                        emit = stops.text[released:cut]
                        released = cut
                        stop_reason, stop_seq = "stop_sequence", hit.stop
                        session.cancel()
                    else:
                        upto = len(stops.text) - stops.holdback()
                        emit = stops.text[released:upto]
                        released = max(released, upto)
                    if emit:
                        for s in segs.feed(emit):
                            yield Partial(s.kind, s.text, s.closed, len(out_tokens))
                if stop_reason is None and session.done:
                    stop_reason = session.stop_reason or "eos"
            if stop_reason not in ("stop_sequence", "cancelled"):
                tail = detok.flush()
                if tail:
                    stops.feed(tail)
                rest = stops.text[released:]
                if rest:
                    for s in segs.feed(rest):
                        yield Partial(s.kind, s.text, s.closed, len(out_tokens))
            for s in segs.finish():
                yield Partial(s.kind, s.text, s.closed, len(out_tokens))
            decode_ms = (time.monotonic() - t_dec) * 1e3
            with tl.span("Worker", "finish"):
                stats = session.finish() or {}
            session = None
            if stop_reason == "cancelled":
                self.slot.cancel()
            else:
                self.slot.finish()
            self.slot.release()
            timings = {"prompt_n": len(tokens) - cached, "prompt_ms": round(prefill_ms, 3),
                       "n_prompt_tokens_cache": cached, "predicted_n": len(out_tokens),
                       "predicted_ms": round(decode_ms, 3)}
            timings.update(stats)
            if p.single_tool_call and stop_seq == "</tool_call>":
                stop_seq = None
            yield Final(stop_reason, stop_seq, len(out_tokens), thinking_tokens, timings, out_tokens)
        except BaseException as e:
            if session is not None:
                try:
                    session.cancel()
                    session.finish()
                except Exception:
                    pass
            if self.slot.state not in (SlotState.IDLE, SlotState.ERROR):
                self.slot.fail(e)
            raise
