"""Executors that need no model: a device mock and a seeded-acceptance mock.

Parity: `crates/saber-engine/src/null.rs:1-15` (NullForward: "a mock of the device, not the model":
same shape ladders and slot bookkeeping, arithmetic faked as a function of the prefix) and
`crates/saber-sched/src/mock.rs:1-20` (RandomAcceptanceExecutor with a seeded acceptance draw and a
deliberately `leaky` negative control that commits a rejected draft).
"""
from __future__ import annotations

import hashlib
import random
import struct
from typing import Optional

from .buckets import DEFAULT_DECODE_BATCHES, DEFAULT_PREFILL_RUNGS
from .executor import SeqOut, SeqRun


def _next_token(prefix_digest: bytes, vocab: int) -> int:
    return struct.unpack("<I", hashlib.blake2b(prefix_digest, digest_size=4).digest())[0] % vocab


class NullExecutor:
    """The "model" is a hash chain over the token prefix, kept per state slot exactly where a real
    device would keep KV and recurrent state, so wrong slot / shift / position bookkeeping in the
    scheduler changes the generated ids."""

    def __init__(self, vocab: int = 1024, max_seqs: int = 8, n_kv_blocks: int = 4096, page_tokens: int = 16,
                 decode_widths=(1, 5, 8), decode_batches=DEFAULT_DECODE_BATCHES,
                 prefill_rungs=DEFAULT_PREFILL_RUNGS, draft_hit_rate: float = 0.7, seed: int = 0,
                 leaky: bool = False):
        self.vocab, self.max_seqs, self.n_kv_blocks, self.page_tokens = vocab, max_seqs, n_kv_blocks, page_tokens
        self.decode_widths, self.decode_batches, self.prefill_rungs = tuple(decode_widths), tuple(decode_batches), tuple(prefill_rungs)
        self.draft_hit_rate, self.leaky = draft_hit_rate, leaky
        self._rng = random.Random(seed)
        self._state = {}           # slot -> (digest, n_tokens) committed
        self._stash = {}           # slot -> list of digests after each row of the last decode step
        self.launch_log = []       # (kind, n_seqs, rows) per call: what a launch census would count
        self.kv_written = {}       # (block, offset) -> position, to catch writes into shared pages

    def reset_slot(self, slot: int) -> None:
        self._state[slot] = (b"", 0)
        self._stash.pop(slot, None)

    def _advance(self, digest: bytes, tok: int) -> bytes:
        return hashlib.blake2b(digest + struct.pack("<i", tok), digest_size=16).digest()

    def _write_kv(self, run: SeqRun) -> None:
        for r in range(len(run.tokens)):
            pos = run.pos0 + r
            self.kv_written[(run.blocks[pos // self.page_tokens], pos % self.page_tokens)] = pos

    def prefill(self, runs: list) -> list:
        self.launch_log.append(("prefill", len(runs), sum(len(r.tokens) for r in runs)))
        outs = []
        for run in runs:
            d, n = self._state[run.slot]
            assert n == run.pos0, f"slot {run.slot}: state holds {n} tokens but the chunk starts at {run.pos0}"
            for t in run.tokens:
                d = self._advance(d, t)
            self._state[run.slot] = (d, n + len(run.tokens))
            self._stash.pop(run.slot, None)
            self._write_kv(run)
            plps = None
            if getattr(run, "prompt_lp", None) is not None:      # a stand-in law: the successor at a fixed distance below the best
                succ = list(run.tokens[1:]) + [run.next_token]
                plps = [{"token_id": int(t), "logprob": -1.0 - (t % 7) * 0.125,
                         "top": [((t + i) % self.vocab, -1.0 - (t % 7) * 0.125 - i) for i in range(run.prompt_lp)]}
                        for t in succ if t >= 0]
            if run.last_chunk:
                tok = _next_token(d, self.vocab)
                outs.append(SeqOut([tok], self._propose(d, tok, max(self.decode_widths) - 1),
                                   seam=self._seam([tok]) if run.want_seam else None, prompt_lps=plps))
            else:
                outs.append(SeqOut([], prompt_lps=plps))
        return outs

    def _seam(self, picks: list, k: int = 8) -> dict:
        """A stand-in for the head's candidate rows: the pick at logit 0, its successors one unit apart."""
        import math
        vals = [-float(i) for i in range(k)]
        lse = math.log(sum(math.exp(v) for v in vals))
        return {"ids": [[(t + i) % self.vocab for i in range(k)] for t in picks],
                "vals": [list(vals) for _ in picks], "lse": [lse for _ in picks]}

    def _propose(self, digest: bytes, first: int, k: int) -> list:
        """Drafts for the tokens AFTER `first`: right with probability draft_hit_rate each."""
        out, d, t = [], digest, first
        for _ in range(k):
            d = self._advance(d, t)
            t = _next_token(d, self.vocab)
            guess = t if self._rng.random() < self.draft_hit_rate else (t + 1) % self.vocab
            out.append(guess)
            if guess != t:
                t = guess
        return out

    def decode(self, runs: list, width: int) -> list:
        self.launch_log.append(("decode", len(runs), len(runs) * width))
        outs = []
        for run in runs:
            d, n = self._state[run.slot]
            if run.shift:                                   # replay the rows accepted last step
                d = self._stash[run.slot][run.shift - 1]
                n += run.shift
                self._state[run.slot] = (d, n)
            assert n == run.pos0, f"slot {run.slot}: committed {n} tokens but the step starts at {run.pos0}"
            assert len(run.tokens) == width
            self._write_kv(run)
            digests, toks = [], []
            dd = d
            accepted = 0
            for r, t in enumerate(run.tokens):
                dd = self._advance(dd, t)
                digests.append(dd)
                target = _next_token(dd, self.vocab)
                toks.append(target)
                if r + 1 < width and run.tokens[r + 1] == target:
                    accepted += 1
                else:
                    break
            if self.leaky and accepted + 1 < width:
                toks.append(run.tokens[accepted + 1])       # negative control: commits a rejected draft
                digests.append(self._advance(digests[-1], run.tokens[accepted + 1]))
            # rows beyond the accepted prefix still ran on the device; their digests are stale but
            # the stash keeps one entry per row like the real kernels do
            while len(digests) < width:
                digests.append(b"stale")
            self._stash[run.slot] = digests
            outs.append(SeqOut(toks, self._propose(digests[len(toks) - 1], toks[-1], width - 1),
                               seam=self._seam(toks) if run.want_seam else None))
        return outs

    # ---- prefix-cache hooks
    def snapshot_state(self, slot: int):
        return self._state[slot]

    def restore_state(self, slot: int, snap) -> None:
        self._state[slot] = snap
        self._stash.pop(slot, None)

    def snapshot_bytes(self) -> int:
        return 1 << 20

    # ---- session parking hooks
    def export_session(self, slot: int, blocks: list, n_tokens: int):
        import pickle
        payload = pickle.dumps((self._state[slot], self._stash.get(slot)))
        return {"kind": "null-executor", "n_tokens": n_tokens}, payload

    def import_session(self, slot: int, blocks: list, header: dict, payload: bytes) -> None:
        import pickle
        state, stash = pickle.loads(payload)
        self._state[slot] = state
        if stash is None:
            self._stash.pop(slot, None)
        else:
            self._stash[slot] = stash

    def free_snapshot(self, snap) -> None:
        pass


def reference_generation(prompt: list, n: int, vocab: int) -> list:
    """What NullExecutor must produce for a prompt, computed without any scheduler."""
    d = b""
    for t in prompt:
        d = hashlib.blake2b(d + struct.pack("<i", t), digest_size=16).digest()
    out = []
    for _ in range(n):
        t = _next_token(d, vocab)
        out.append(t)
        d = hashlib.blake2b(d + struct.pack("<i", t), digest_size=16).digest()
    return out
