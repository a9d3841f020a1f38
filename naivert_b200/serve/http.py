"""HTTP transport: FastAPI app with four routes, one inference worker thread that owns the
engine, a bounded request queue (HTTP 529 when full), SSE streaming with keep-alives and
disconnect -> cancel, and one structured log line per request.

    GET  /health                      readiness, slot state, queued requests
    GET  /v1/models                   served model id
    POST /v1/messages                 generate (JSON or text/event-stream)
    POST /v1/messages/count_tokens    formatted prompt length

Behavioural parity: naivert/serve/http.py (``Worker`` :69-265, ``CompletionResponse`` :324-549,
``build_app`` :552-645, ``run_app`` :648-671).
"""
from __future__ import annotations

import asyncio
import json
import logging
import queue
import signal
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, StreamingResponse

from .context import Final, Opened, Partial, ServerContext
from .messages_api import (ApiError, CountTokensRequest, MessagesRequest, ResponseAssembler, ServerDefaults, TaskParams,
                           parse_request, validate_request)
from .replay import AssistantReplay
from .syntax import ToolCallParseError
from .timeline import RequestTimeline

log = logging.getLogger("naivert_b200.serve")
KEEPALIVE_S = 5.0
SSE_BATCH_MAX = 32
_DONE = object()


@dataclass
class Job:
    params: TaskParams
    timeline: RequestTimeline
    enqueued: float
    out: "queue.Queue[Any]" = field(default_factory=lambda: queue.Queue())
    cancelled: threading.Event = field(default_factory=threading.Event)
    kind: str = "generate"            # or "count"


class Worker:
    """Single owner thread of the engine.  Status: loading -> ok -> shutting_down | error."""

    def __init__(self, ctx_factory: Callable[[], ServerContext], queue_depth: int = 8, dump_tokens: Optional[str] = None):
        self.ctx_factory = ctx_factory
        self.dump_tokens = dump_tokens               # JSONL path: one line of output token ids per finished request
        self.jobs: "queue.Queue[Optional[Job]]" = queue.Queue(maxsize=max(1, queue_depth))
        self.status = "loading"
        self.ctx: Optional[ServerContext] = None
        self.thread = threading.Thread(target=self.run, name="naivert-inference", daemon=True)
        self.error: Optional[str] = None

    def start(self) -> None:
        self.thread.start()

    def stop(self) -> None:
        self.status = "shutting_down" if self.status != "error" else self.status
        try:
            self.jobs.put_nowait(None)
        except queue.Full:
            pass

    def submit(self, job: Job) -> None:
        if self.status != "ok":
            raise ApiError(503, "loading" if self.status == "loading" else "shutting_down", f"server is {self.status}")
        try:
            self.jobs.put_nowait(job)
        except queue.Full:
            raise ApiError(529, "queue_full", "the request queue is full; retry later")

    def queued(self) -> int:
        return self.jobs.qsize()

    def slot_state(self) -> str:
        return self.ctx.slot.state.value if self.ctx is not None else "LOADING"

    # ------------------------------------------------------------------ worker thread
    def run(self) -> None:
        try:
            self.ctx = self.ctx_factory()
            self.ctx.owner = threading.get_ident()
            self.status = "ok"
        except BaseException as e:                         # noqa: BLE001 - reported through /health
            log.exception("engine start-up failed")
            self.status, self.error = "error", repr(e)
            return
        while True:
            job = self.jobs.get()
            if job is None:
                break
            if self.status == "shutting_down":
                # a real job was popped after shutdown began: its client still gets an answer
                job.out.put(ApiError(503, "shutting_down", "server is shutting_down"))
                job.out.put(_DONE)
                break
            try:
                self.complete(job)
            except ApiError as e:
                job.out.put(e)
            except ToolCallParseError as e:
                job.out.put(ApiError(500, "tool_call_parse_error", str(e)))
            except BaseException as e:                     # noqa: BLE001
                log.exception("request failed")
                job.out.put(ApiError(500, "runtime_error", f"{type(e).__name__}: {e}"))
                if getattr(e, "fatal", False):
                    self.status, self.error = "error", repr(e)
            finally:
                job.out.put(_DONE)
            if self.status == "error":
                break
        # drain whatever is still queued
        while True:
            try:
                j = self.jobs.get_nowait()
            except queue.Empty:
                break
            if j is not None:
                j.out.put(ApiError(503 if self.status == "shutting_down" else 500,
                                   "shutting_down" if self.status == "shutting_down" else "runtime_error",
                                   f"server is {self.status}"))
                j.out.put(_DONE)

    def complete(self, job: Job) -> None:
        tl, p = job.timeline, job.params
        wait_ms = (time.monotonic() - job.enqueued) * 1e3
        tl.record("Queue", "queue_wait", tl.now_ms() - wait_ms, wait_ms)
        if job.kind == "count":
            job.out.put({"input_tokens": self.ctx.count_tokens(p)})
            return
        job.out.put(("queue_wait_ms", wait_ms))
        t0 = time.monotonic()
        final: Optional[Final] = None
        opened: Optional[Opened] = None
        for item in self.ctx.handle_completion(p, tl, job.cancelled):
            if isinstance(item, Opened):
                opened = item
            elif isinstance(item, Final):
                final = item
            job.out.put(item)
        if final is not None and self.dump_tokens:
            try:
                with open(self.dump_tokens, "a") as f:
                    f.write(json.dumps({"t": time.time(), "stop_reason": final.stop_reason, "output_tokens": final.output_tokens,
                                        "tokens": list(final.tokens)}) + "\n")
            except OSError as e:
                log.warning("token dump failed: %s", e)
        if final is not None:
            seg = final.timings.get("segments", {}).get("total", {})
            log.info("request done prompt_n=%s cache=%s prefill_ms=%s predicted_n=%s stop=%s device_tok_s=%s wall_ms=%.1f",
                     final.timings.get("prompt_n"), final.timings.get("n_prompt_tokens_cache"),
                     final.timings.get("prompt_ms"), final.output_tokens, final.stop_reason,
                     final.timings.get("decode_tok_s_device", seg.get("device_tok_s")), (time.monotonic() - t0) * 1e3)


def _error_response(e: ApiError):
    return JSONResponse(e.body(), status_code=e.status, headers={"x-naivert-warning": e.warning})


def build_app(ctx_factory: Callable[[], ServerContext], defaults: Optional[ServerDefaults] = None, queue_depth: int = 8,
              cors_origin: Optional[str] = None, cors_credentials: bool = False, display_name: Optional[str] = None,
              dump_tokens: Optional[str] = None):
    from contextlib import asynccontextmanager

    defaults = defaults or ServerDefaults()
    worker = Worker(ctx_factory, queue_depth, dump_tokens=dump_tokens)
    replay = AssistantReplay()

    @asynccontextmanager
    async def lifespan(app):
        worker.start()
        yield
        worker.stop()

    app = FastAPI(lifespan=lifespan)
    app.state.worker = worker
    if cors_origin:
        from fastapi.middleware.cors import CORSMiddleware
        app.add_middleware(CORSMiddleware, allow_origins=[cors_origin], allow_credentials=cors_credentials,
                           allow_methods=["*"], allow_headers=["*"], expose_headers=["x-naivert-ignored", "x-naivert-warning"])

    @app.get("/health")
    async def health():
        body = {"status": worker.status, "slot": worker.slot_state(), "queued": worker.queued()}
        if worker.error:
            body["error"] = worker.error
        return JSONResponse(body, status_code=200 if worker.status == "ok" else 503)

    @app.get("/v1/models")
    async def models():
        m = {"id": defaults.served_model, "type": "model", "display_name": display_name or defaults.served_model}
        return {"data": [m], "has_more": False, "first_id": m["id"], "last_id": m["id"]}

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(request: Request):
        try:
            req = parse_request(await request.body(), CountTokensRequest)
            p = validate_request(req, defaults, request.headers, count_only=True)
            if worker.status != "ok":
                raise ApiError(503, "loading" if worker.status == "loading" else "shutting_down", f"server is {worker.status}")
            # tokenisation does not touch the engine: it runs here, outside the generation queue
            return {"input_tokens": worker.ctx.count_tokens(p)}
        except ApiError as e:
            return _error_response(e)

    @app.post("/v1/messages")
    async def messages(request: Request):
        tl = RequestTimeline()
        try:
            with tl.span("HTTP", "parse_validate"):
                req = parse_request(await request.body(), MessagesRequest)
                p = validate_request(req, defaults, request.headers)
                replay.restore(p)
            job = Job(p, tl, time.monotonic())
            with tl.span("HTTP", "wait_admission"):
                worker.submit(job)
        except ApiError as e:
            return _error_response(e)

        loop = asyncio.get_running_loop()

        async def next_item(timeout: float):
            try:
                return await loop.run_in_executor(None, lambda: job.out.get(timeout=timeout))
            except queue.Empty:
                return None

        if not p.stream:
            asm: Optional[ResponseAssembler] = None
            wait_ms = 0.0
            ignored: List[str] = []
            while True:
                if await request.is_disconnected():
                    job.cancelled.set()
                item = await next_item(1.0)
                if item is None:
                    continue
                if item is _DONE:
                    break
                if isinstance(item, ApiError):
                    return _error_response(item)
                if isinstance(item, tuple):
                    wait_ms = item[1]
                elif isinstance(item, Opened):
                    asm = ResponseAssembler(p, item.prompt_tokens, item.cached_tokens, wait_ms)
                    ignored = item.ignored
                elif isinstance(item, Partial):
                    try:
                        asm.feed(item.kind, item.text, item.closed, item.generated_tokens)
                    except ToolCallParseError as e:
                        job.cancelled.set()
                        return _error_response(ApiError(500, "tool_call_parse_error", str(e)))
                elif isinstance(item, Final):
                    ext = {"timings": {"queue_wait_ms": round(wait_ms, 3), **item.timings}, "timeline": tl.snapshot()}
                    asm.finish(item.stop_reason, item.stop_sequence, item.output_tokens, item.thinking_tokens, ext)
            if asm is None or not hasattr(asm, "usage"):
                return _error_response(ApiError(500, "runtime_error", "the request ended without a result"))
            if asm.untyped and "untyped_tool_property" not in ignored:
                ignored.append("untyped_tool_property")
            replay.remember(p, asm.blocks)
            headers = {"x-naivert-ignored": ",".join(ignored)} if ignored else {}
            return JSONResponse(asm.message(), headers=headers)

        async def sse():
            asm: Optional[ResponseAssembler] = None
            wait_ms = 0.0
            last_out = time.monotonic()
            try:
                while True:
                    if await request.is_disconnected():
                        job.cancelled.set()
                        return
                    item = await next_item(0.25)
                    if item is None:
                        if time.monotonic() - last_out >= KEEPALIVE_S:
                            last_out = time.monotonic()
                            yield ": keepalive\n\n" if asm is None else ResponseAssembler.sse("ping", {"type": "ping"})
                        continue
                    if item is _DONE:
                        return
                    if isinstance(item, ApiError):
                        yield ResponseAssembler.sse("error", item.body())
                        return
                    chunks: List[str] = []
                    batch = [item]
                    while len(batch) < SSE_BATCH_MAX:               # coalesce what is already waiting
                        try:
                            batch.append(job.out.get_nowait())
                        except queue.Empty:
                            break
                    ended = False
                    for it in batch:
                        if it is _DONE:
                            ended = True
                        elif isinstance(it, ApiError):
                            chunks.append(ResponseAssembler.sse("error", it.body()))
                            ended = True
                        elif isinstance(it, tuple):
                            wait_ms = it[1]
                        elif isinstance(it, Opened):
                            asm = ResponseAssembler(p, it.prompt_tokens, it.cached_tokens, wait_ms)
                            chunks.append(asm.start_event())
                        elif isinstance(it, Partial):
                            try:
                                chunks.extend(asm.feed(it.kind, it.text, it.closed, it.generated_tokens))
                            except ToolCallParseError as e:
                                job.cancelled.set()
                                chunks.append(ResponseAssembler.sse("error", ApiError(500, "tool_call_parse_error", str(e)).body()))
                                ended = True
                        elif isinstance(it, Final):
                            ext = {"timings": {"queue_wait_ms": round(wait_ms, 3), **it.timings}, "timeline": tl.snapshot()}
                            chunks.extend(asm.finish(it.stop_reason, it.stop_sequence, it.output_tokens, it.thinking_tokens, ext))
                            replay.remember(p, asm.blocks)
                        if ended:
                            break
                    if chunks:
                        last_out = time.monotonic()
                        yield "".join(chunks)
                    if ended:
                        return
            finally:
                if asm is None or not hasattr(asm, "usage"):
                    job.cancelled.set()

        headers = {"cache-control": "no-cache", "x-accel-buffering": "no"}
        if p.ignored:
            headers["x-naivert-ignored"] = ",".join(p.ignored)
        return StreamingResponse(sse(), media_type="text/event-stream", headers=headers)

    return app


def run_app(app, host: str = "127.0.0.1", port: int = 8080, log_level: str = "info") -> None:
    """Run under uvicorn; SIGTERM stops the worker before the server exits."""
    import uvicorn
    server = uvicorn.Server(uvicorn.Config(app, host=host, port=port, log_level=log_level))
    worker: Worker = app.state.worker

    def on_term(signum, frame):
        worker.stop()
        server.should_exit = True

    try:
        signal.signal(signal.SIGTERM, on_term)
    except ValueError:
        pass                                               # not the main thread
    server.run()
