"""The tensor-parallel front end on CPU: two gloo ranks, fake engines.  Rank 0 (leader) mirrors every engine call to
rank 1 (follower); a follower that dies between requests surfaces on the leader as an error of its next command
(short process-group timeout), never as a hang.  No GPU is involved."""
import multiprocessing as mp
import os
import socket
import sys
import time
from datetime import timedelta

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _FakeSession:
    def __init__(self, log, tokens, max_decode):
        self.log, self.left, self.done = log, 3, False
        self.log.append(("open", tuple(tokens), max_decode))

    def step(self, timeout_s=120.0):
        self.left -= 1
        self.done = self.left == 0
        self.log.append(("step",))
        return [7]

    def cancel(self):
        self.log.append(("cancel",))

    def finish(self):
        self.log.append(("finish",))
        return {"tokens": 3}


class _FakeEngine:
    config = {"fake": True}

    def __init__(self, log):
        self.log = log

    def align_prompt(self, tokens, session_id, text=None):
        return list(tokens)

    def open_session(self, tokens, max_decode, session_id, sampling=None):
        return _FakeSession(self.log, tokens, max_decode)

    def close(self):
        self.log.append(("close",))


def _rank(rank, port, mode, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from naivert_b200.runtime.tp_frontend import Commands, LeaderEngine, follower_loop
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=2, timeout=timedelta(seconds=5))
    log = []
    ch = Commands(ack_timeout_s=3.0)
    try:
        if rank == 0:
            lead = LeaderEngine(_FakeEngine(log), ch)
            s = lead.open_session([1, 2, 3], 16, "S")
            while not s.done:
                s.step()
            s.finish()
            if mode == "follower_dies":
                time.sleep(1.0)                      # the follower has left by now
                t0 = time.monotonic()
                try:
                    lead.open_session([4, 5], 8, "S")
                    q.put((0, "no error"))
                except Exception as e:               # noqa: BLE001
                    q.put((0, "detected", round(time.monotonic() - t0, 1), type(e).__name__, str(e)))
                q.close()
                q.join_thread()                      # the record is on its way before the process leaves
                os._exit(0)
            lead.close()
            q.put((0, log))
        else:
            if mode == "follower_dies":
                # serve exactly one request, then leave without the close handshake (a crashed rank)
                eng = _FakeEngine(log)
                cmd = ch.recv()
                s = eng.open_session(cmd["tokens"], cmd["max_decode"], cmd["session_id"], cmd["sampling"])
                while not s.done:
                    s.step()
                assert ch.recv()["op"] == "finish"
                q.put((1, "left"))
                q.close()
                q.join_thread()
                os._exit(0)
            follower_loop(_FakeEngine(log), ch)
            q.put((1, log))
    finally:
        if mode != "follower_dies":
            dist.destroy_process_group()


def _run(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_rank, args=(r, port, mode, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = {}
    for _ in range(2):
        item = q.get(timeout=60)
        out[item[0]] = item[1:]
    for p in ps:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    return out


def test_follower_mirrors_the_leaders_calls():
    out = _run("normal")
    lead, follow = out[0][0], out[1][0]
    want = [("open", (1, 2, 3), 16), ("step",), ("step",), ("step",), ("finish",), ("close",)]
    assert lead == want and follow == want


def test_a_follower_that_left_is_an_error_not_a_hang():
    out = _run("follower_dies")
    assert out[1] == ("left",)
    assert out[0][0] == "detected" and out[0][1] < 20 and out[0][2] == "FollowerLost" and "[1]" in out[0][3], out[0]
