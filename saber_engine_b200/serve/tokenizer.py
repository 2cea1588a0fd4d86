"""Tokenizers: a byte codec that needs no files (every test and the synthetic packs use it), and a
thin wrapper over a Hugging Face tokenizer directory when a pack ships one.

Parity: the reference's tests run on a `ByteCodec` / `MinimalChatRenderer` pair so nothing needs a
real tokenizer (`crates/saber-serve/src/engine.rs:316-650`); production loads the checkpoint's
tokenizer and chat template (`crates/saber-model/src/tokenizer`, `template/mod.rs`).
"""
from __future__ import annotations

from typing import Optional


class ByteCodec:
    """ids 0..255 are bytes; specials follow."""
    SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>",
                "</tool_call>", "<|image_pad|>"]

    def __init__(self, vocab: int = 1024):
        self.vocab_size = max(vocab, 256 + len(self.SPECIALS))
        self.special_ids = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.id_to_special = {v: k for k, v in self.special_ids.items()}
        self.eos_token_id = self.special_ids["<|im_end|>"]

    def encode(self, text: str) -> list:
        out, i = [], 0
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

    def token_bytes(self, tid: int) -> bytes:
        if tid < 256:
            return bytes([tid])
        if tid in self.id_to_special:
            return self.id_to_special[tid].encode()
        return f"<|tok{tid}|>".encode()          # ids of a random-init model outside the byte range

    def decode(self, ids) -> str:
        return b"".join(self.token_bytes(t) for t in ids).decode("utf-8", errors="replace")


class HfTokenizer:
    def __init__(self, path: str):
        from transformers import AutoTokenizer
        self.tok = AutoTokenizer.from_pretrained(path, local_files_only=True)
        self.vocab_size = len(self.tok)
        self.eos_token_id = self.tok.eos_token_id
        self.chat_template = getattr(self.tok, "chat_template", None)

    def encode(self, text: str) -> list:
        return self.tok.encode(text, add_special_tokens=False)

    def token_bytes(self, tid: int) -> bytes:
        return self.tok.decode([tid]).encode("utf-8")

    def decode(self, ids) -> str:
        return self.tok.decode(list(ids))


class IncrementalDetok:
    """Emits text as tokens arrive without ever splitting a UTF-8 sequence
    (`crates/saber-serve/src/detok.rs:1-12`)."""

    def __init__(self, tokenizer, skip_ids=()):
        self.tok, self.skip = tokenizer, set(skip_ids)
        self._buf = b""

    def push(self, ids) -> str:
        for t in ids:
            if t not in self.skip:
                self._buf += self.tok.token_bytes(t)
        # longest prefix that decodes cleanly
        for cut in range(len(self._buf), max(-1, len(self._buf) - 4), -1):
            try:
                text = self._buf[:cut].decode("utf-8")
            except UnicodeDecodeError:
                continue
            self._buf = self._buf[cut:]
            return text
        return ""

    def flush(self) -> str:
        text, self._buf = self._buf.decode("utf-8", errors="replace"), b""
        return text


DEFAULT_CHAT_TEMPLATE = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n"
    "{% if m['content'] is string %}{{ m['content'] }}{% else %}"
    "{% for part in m['content'] %}{% if part['type'] == 'text' %}{{ part['text'] }}"
    "{% elif part['type'] in ('image', 'image_url') %}<|image_pad|>{% endif %}{% endfor %}{% endif %}"
    "<|im_end|>\n{% endfor %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% if enable_thinking is defined and not enable_thinking %}"
    "<think>\n\n</think>\n\n{% endif %}{% endif %}")


def render_chat(messages: list, template: Optional[str] = None, add_generation_prompt: bool = True,
                tools: Optional[list] = None, **kwargs) -> str:
    """Jinja chat template (`crates/saber-model/src/template/mod.rs`)."""
    import jinja2
    env = jinja2.Environment(trim_blocks=False, lstrip_blocks=False, undefined=jinja2.ChainableUndefined)
    env.globals["raise_exception"] = lambda msg: (_ for _ in ()).throw(ValueError(msg))
    return env.from_string(template or DEFAULT_CHAT_TEMPLATE).render(
        messages=messages, add_generation_prompt=add_generation_prompt, tools=tools, **kwargs)


def normalise_messages(messages) -> list:
    """Shape checks the reference applies before templating (`conversation.rs:1-20`)."""
    if not isinstance(messages, list) or not messages:
        raise ValueError("messages must be a non-empty list")
    out = []
    for i, m in enumerate(messages):
        if not isinstance(m, dict) or "role" not in m:
            raise ValueError(f"messages[{i}] needs a role")
        if m["role"] not in ("system", "user", "assistant", "tool", "developer"):
            raise ValueError(f"messages[{i}].role {m['role']!r} is not supported")
        c = m.get("content")
        if c is None and m["role"] == "assistant" and m.get("tool_calls"):
            c = ""
        if not isinstance(c, (str, list)):
            raise ValueError(f"messages[{i}].content must be a string or a list of parts")
        out.append({**m, "content": c})
    return out
