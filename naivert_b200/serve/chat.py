"""Chat formatting and incremental detokenisation.

``ChatFormatter`` renders API messages with the checkpoint's own chat template (a HF
tokenizer loaded from the target checkpoint directory) or, when no tokenizer is available
(random-init checkpoints, tests), with a built-in byte-level tokenizer and a fixed template
of the same shape.  ``IncrementalDetokenizer`` turns a token stream into text without ever
emitting half a UTF-8 character.

Parity: naivert/serve/chat.py (``ChatFormatter`` :25, ``IncrementalDetokenizer`` :73).
"""
from __future__ import annotations

import json
from typing import Any, List, Mapping, Optional, Sequence


class ByteTokenizer:
    """256 byte tokens + a few specials; ids fit any vocabulary >= 264."""

    SPECIALS = ["<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>", "<|pad|>", "<|eos|>"]

    def __init__(self):
        self.special_ids = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.id_special = {v: k for k, v in self.special_ids.items()}
        self.eos_token_id = self.special_ids["<|im_end|>"]

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            for s, sid in self.special_ids.items():
                if text.startswith(s, i):
                    out.append(sid)
                    i += len(s)
                    break
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def decode_bytes(self, tokens: Sequence[int], skip_special: bool = False) -> bytes:
        out = bytearray()
        for t in tokens:
            if t < 256:
                out.append(t)
            elif t in self.id_special:
                if not skip_special:
                    out.extend(self.id_special[t].encode())
            else:
                out.extend(b"?")           # ids outside the byte alphabet (random-weight models)
        return bytes(out)

    def decode(self, tokens: Sequence[int], skip_special_tokens: bool = False) -> str:
        return self.decode_bytes(tokens, skip_special_tokens).decode("utf-8", errors="replace")


def load_tokenizer(path: Optional[str]):
    if path:
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(path)
        except Exception:
            pass
    return ByteTokenizer()


class ChatFormatter:
    def __init__(self, tokenizer: Any, enable_thinking: bool = False):
        self.tok = tokenizer
        self.default_thinking = enable_thinking

    @classmethod
    def from_path(cls, path: Optional[str], enable_thinking: bool = False) -> "ChatFormatter":
        return cls(load_tokenizer(path), enable_thinking)

    @property
    def eos_token_id(self) -> int:
        return int(self.tok.eos_token_id)

    def render(self, messages: Sequence[Mapping[str, Any]], tools: Optional[Sequence[Mapping[str, Any]]] = None,
               thinking: Optional[bool] = None) -> str:
        thinking = self.default_thinking if thinking is None else thinking
        if hasattr(self.tok, "apply_chat_template") and getattr(self.tok, "chat_template", None):
            msgs = [{k: v for k, v in m.items() if k != "tool_calls_text"} for m in messages]
            return self.tok.apply_chat_template(msgs, tools=list(tools) if tools else None, tokenize=False,
                                                add_generation_prompt=True, enable_thinking=thinking)
        parts: List[str] = []
        if tools:
            parts.append("<|im_start|>system\n# Tools\n" + "\n".join(json.dumps(t, sort_keys=True) for t in tools) + "<|im_end|>\n")
        for m in messages:
            body = m.get("content") or ""
            if m["role"] == "assistant":
                if m.get("reasoning_content"):
                    body = f"<think>{m['reasoning_content']}</think>" + body
                if m.get("tool_calls_text"):
                    body = (body + "\n\n" if body.strip() else body) + m["tool_calls_text"]
            parts.append(f"<|im_start|>{m['role']}\n{body}<|im_end|>\n")
        parts.append("<|im_start|>assistant\n" + ("<think>" if thinking else ""))
        return "".join(parts)

    def encode(self, messages, tools=None, thinking=None) -> List[int]:
        text = self.render(messages, tools, thinking)
        if isinstance(self.tok, ByteTokenizer):
            return self.tok.encode(text)
        return list(self.tok.encode(text, add_special_tokens=False))

    def decode(self, tokens: Sequence[int], skip_special_tokens: bool = False) -> str:
        return self.tok.decode(list(tokens), skip_special_tokens=skip_special_tokens)


class IncrementalDetokenizer:
    """Feeds tokens one at a time and returns only text that can no longer change: the decode
    of a sliding window is compared with the previous decode and an incomplete trailing
    character (U+FFFD) is withheld until its bytes are complete."""

    def __init__(self, tokenizer: Any, skip_special_tokens: bool = False, window: int = 8):
        self.tok, self.skip, self.window = tokenizer, skip_special_tokens, window
        self.reset()

    def reset(self) -> None:
        self.tokens: List[int] = []
        self.prefix_off = 0        # start of the decode window
        self.read_off = 0          # tokens whose text has been emitted

    def _dec(self, toks: Sequence[int]) -> str:
        return self.tok.decode(list(toks), skip_special_tokens=self.skip)

    def add(self, token: int) -> str:
        self.tokens.append(int(token))
        prev = self._dec(self.tokens[self.prefix_off:self.read_off])
        cur = self._dec(self.tokens[self.prefix_off:])
        if len(cur) > len(prev) and not cur.endswith("�"):
            out = cur[len(prev):]
            self.prefix_off = max(self.prefix_off, self.read_off - self.window) if self.read_off > self.window else self.prefix_off
            self.read_off = len(self.tokens)
            return out
        return ""

    def add_all(self, tokens: Sequence[int]) -> str:
        return "".join(self.add(t) for t in tokens)

    def flush(self) -> str:
        prev = self._dec(self.tokens[self.prefix_off:self.read_off])
        cur = self._dec(self.tokens[self.prefix_off:])
        self.read_off = len(self.tokens)
        return cur[len(prev):]
