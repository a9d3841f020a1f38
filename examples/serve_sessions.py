#!/usr/bin/env python3
"""Serve the Anthropic-Messages-compatible API from one node.

    python examples/serve_sessions.py --model naive-n0.5 --target /ckpt/target --draft /ckpt/draft
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/serve_sessions.py ...

Rank 0 runs the HTTP server; with more than one process the other ranks follow its engine calls.
Without checkpoints (``--random-init``) weights are drawn on device, which is what the smoke
tests and benchmarks use.  Flags mirror examples/serve_sessions.py:75-114 of the reference.
"""
from __future__ import annotations

import argparse
import logging
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--host", default=os.environ.get("NAIVERT_HOST", "127.0.0.1"))
    ap.add_argument("--port", type=int, default=int(os.environ.get("NAIVERT_PORT", "8080")))
    ap.add_argument("--cors-origin", default=None)
    ap.add_argument("--cors-credentials", action="store_true")
    ap.add_argument("--model", default="naive-n0.5", help="registry name of the architecture")
    ap.add_argument("--target", default=os.environ.get("NAIVERT_TARGET_CHECKPOINT"), help="target checkpoint directory or short name")
    ap.add_argument("--draft", "--checkpoint", dest="draft", default=os.environ.get("NAIVERT_DRAFT_CHECKPOINT"),
                    help="draft checkpoint directory or short name")
    ap.add_argument("--list-weights", action="store_true",
                    help="print the checkpoints found under NAIVERT_MODEL_ROOTS / NAIVERT_DRAFT_ROOTS and exit")
    ap.add_argument("--random-init", action="store_true", help="draw weights on device instead of loading checkpoints")
    ap.add_argument("--layers", type=int, default=0, help="truncate the model to its first N layers")
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--max-decode-tokens", type=int, default=524288)
    ap.add_argument("--capacity", type=int, default=1048576, help="KV positions per sequence")
    ap.add_argument("--output-capacity", type=int, default=None,
                    help="most tokens one request may generate; --max-decode-tokens is capped to it (the host ring "
                         "holds round records and is drained while the request runs, so it does not bound the output)")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--store-gb", type=float, default=8.0, help="parked-prefix budget per rank")
    ap.add_argument("--queue-depth", type=int, default=8)
    ap.add_argument("--resume-policy", choices=("cost", "replay", "native"), default="cost")
    ap.add_argument("--prefill", choices=("verify8", "native"), default="verify8",
                    help="native: long prompts are ingested in chunks (tensor-parallel attention, experts per --prefill-experts)")
    ap.add_argument("--prefill-chunk", type=int, default=4096, help="rows per native prefill chunk")
    ap.add_argument("--prefill-experts", choices=("tp", "ep"), default="tp",
                    help="ep: a second, expert-parallel copy of the experts (random-init only; doubles expert memory)")
    ap.add_argument("--prefill-warm-chunks", action="store_true", help="run every native chunk size once before serving")
    ap.add_argument("--draft-ingest", choices=("batched", "loop"), default="batched",
                    help="accepted for command-line compatibility: the draft's K/V of a prompt is written by whichever path "
                         "ingests the prompt (per chunk with --prefill native, per eight-row step with verify8); "
                         "'loop' with --prefill native only logs that the chunk path stays batched")
    ap.add_argument("--dump-tokens", default=None, help="append the output token ids of every request to this JSONL file")
    ap.add_argument("--thinking", action="store_true", help="enable thinking by default in the chat template")
    ap.add_argument("--log-level", default="info")
    return ap.parse_args(argv)


def main(argv=None) -> int:
    a = parse_args(argv)
    if a.list_weights:
        from naivert_b200.models.checkpoint import list_weights
        print(list_weights())
        return 0
    if a.output_capacity is not None:
        a.max_decode_tokens = min(a.max_decode_tokens, max(1, a.output_capacity))
    logging.basicConfig(level=a.log_level.upper(), format="%(asctime)s %(name)s %(levelname)s %(message)s")
    if a.draft_ingest == "loop" and a.prefill == "native":
        logging.getLogger("naivert_b200.serve").warning("--draft-ingest loop: the native chunk path writes the draft K/V per chunk")
    import torch
    import torch.distributed as dist

    from naivert_b200.models.checkpoint import resolve_checkpoint
    from naivert_b200.models.registry import resolve_model
    from naivert_b200.runtime.engine import Engine
    from naivert_b200.runtime.session_engine import SessionEngine
    from naivert_b200.runtime.tp_frontend import Commands, LeaderEngine, follower_loop
    from naivert_b200.serve.chat import ChatFormatter
    from naivert_b200.serve.context import ServerContext
    from naivert_b200.serve.http import build_app, run_app
    from naivert_b200.serve.messages_api import ServerDefaults

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = cpu_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
        cpu_group = dist.new_group(backend="gloo")
    spec = resolve_model(a.model)
    if a.layers:
        spec = spec.with_layers(a.layers)
    target = draft = None
    if not a.random_init:
        if not a.target or not a.draft:
            raise SystemExit("--target and --draft are required unless --random-init is given")
        target, draft = resolve_checkpoint(a.target), resolve_checkpoint(a.draft, "NAIVERT_DRAFT_ROOTS")

    def build_engine() -> SessionEngine:
        ep_w = None
        if a.prefill == "native" and a.prefill_experts == "ep" and world > 1:
            if not a.random_init:
                raise SystemExit("--prefill-experts ep needs --random-init (checkpoints are loaded in the tensor-parallel layout)")
            from naivert_b200.models.device_init import init_expert_rank_weights_device
            ep_w = init_expert_rank_weights_device(spec, rank, world, seed=a.seed, device=dev)
        eng = Engine.build(spec, rank=rank, tp=world, group=group, capacity=a.capacity, seed=a.seed, target_ckpt=target,
                           draft_ckpt=draft, device=dev, prefill_chunk=a.prefill_chunk if a.prefill == "native" else 0,
                           ep_weights=ep_w)
        if eng.prefill is not None and a.prefill_warm_chunks:
            with torch.cuda.stream(eng.round.stream):
                eng.prefill.warm_chunks()
        return SessionEngine(eng, store_gb=a.store_gb, max_output_tokens=a.max_decode_tokens, resume_policy=a.resume_policy)

    if rank != 0:
        follower_loop(build_engine(), Commands(cpu_group))
        return 0

    defaults = ServerDefaults(served_model=a.served_model_name or a.model, temperature=a.temperature, top_p=a.top_p, seed=a.seed,
                              repetition_penalty=a.repetition_penalty, frequency_penalty=a.frequency_penalty,
                              presence_penalty=a.presence_penalty, max_output_tokens=a.max_decode_tokens)

    def factory() -> ServerContext:
        torch.cuda.set_device(local)                      # the worker thread owns the device context
        se = build_engine()
        formatter = ChatFormatter.from_path(target, enable_thinking=a.thinking)

        class _Tok:                                        # decode / encode as the session engine's align_prompt wants them
            def decode(self, ids):
                return formatter.decode(ids)

            def encode(self, text):
                t = formatter.tok
                return list(t.encode(text)) if not hasattr(t, "apply_chat_template") else list(t.encode(text, add_special_tokens=False))

        se.tokenizer = _Tok()
        engine = LeaderEngine(se, Commands(cpu_group)) if world > 1 else se
        return ServerContext(engine, formatter)

    app = build_app(factory, defaults, queue_depth=a.queue_depth, cors_origin=a.cors_origin, cors_credentials=a.cors_credentials, dump_tokens=a.dump_tokens)
    run_app(app, a.host, a.port, a.log_level)
    return 0


if __name__ == "__main__":
    sys.exit(main())
