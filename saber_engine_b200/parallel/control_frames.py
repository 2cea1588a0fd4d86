"""Per-step control frames from the planning rank to its followers, in a FIXED byte layout (no
pickling), carried over one shared-memory line per follower.

A frame is a 32-byte header (magic, op, part / parts, call number, sequences, width, payload bytes)
and a payload of little-endian words: one fixed record per sequence followed by its variable tails
(token ids, NEW KV blocks, uniform numbers, rotary positions).  A sequence's block table crosses
the line only when it changes: the follower keeps every live sequence's table and the record says
"keep the first k blocks, append these", so a decode step that crosses no page boundary sends no
block at all, whatever the context length.  A payload larger than one line slot (a 2048-row prompt
chunk is 8 KiB of token ids) is cut into parts; the receiver takes them in order.

Parity: the reference's leader sends the step's control block through its shared-memory line and
the block table only on page-crossing steps (`crates/saber-engine/src/tp2.rs:1897`,
`crates/saber-hip/src/shmline.rs:1-50`).
"""
from __future__ import annotations

import struct
import time
from typing import Optional

from ..sched.executor import SeqRun

MAGIC = 0x53424346                    # "SBCF"
OPS = {"prefill": 1, "decode": 2, "reset_slot": 3, "snapshot_state": 4, "restore_state": 5, "free_snapshot": 6, "stop": 7,
       "export_session": 8, "import_session": 9}
OP_NAMES = {v: k for k, v in OPS.items()}
HEADER = struct.Struct("<IHHHHQIII")  # magic, op, part, parts, reserved, call number, nseq, width, payload bytes (whole call)
SEQ = struct.Struct("<qqqiiiiiiiifiiiiffff")
# seq_id, uid, block-table key (-1: none), pos0, slot, shift, step_no, flags, rope_delta, prompt_lp, next_token, temperature,
# n_tokens, blocks_keep, n_new_blocks, n_uniforms, sampling[4]
F_LAST_CHUNK, F_WANT_SEAM, F_SAMPLING, F_ROPE, F_PROMPT_LP = 1, 2, 4, 8, 16
PART_BYTES = 4096 - HEADER.size


def _prune(blocks: dict) -> None:
    """Both sides drop the oldest tables by the same rule (same frames, same insertion order), so a
    table the encoder still counts on is never missing on the decoder."""
    if len(blocks) > 1024:
        for k in list(blocks)[:len(blocks) - 512]:
            del blocks[k]


class FrameEncoder:
    """Leader side: turns executor calls into frame parts; remembers what block table each follower
    already holds (all followers hold the same one: every frame goes to all of them)."""

    def __init__(self):
        self._blocks: dict = {}           # seq_id -> blocks the followers hold
        self._n = 0

    def _seq(self, r: SeqRun) -> bytes:
        held = self._blocks.get(r.seq_id, [])
        keep = 0
        lim = min(len(held), len(r.blocks))
        while keep < lim and held[keep] == r.blocks[keep]:
            keep += 1
        new = list(r.blocks[keep:])
        self._blocks[r.seq_id] = list(r.blocks)
        flags = (F_LAST_CHUNK if r.last_chunk else 0) | (F_WANT_SEAM if r.want_seam else 0) | \
                (F_SAMPLING if r.sampling is not None else 0) | (F_ROPE if r.rope_pos is not None else 0) | \
                (F_PROMPT_LP if r.prompt_lp is not None else 0)
        samp = tuple(float(x) for x in r.sampling) if r.sampling is not None else (0.0, 0.0, 0.0, 0.0)
        uni = list(r.uniforms or [])
        bkey = r.blocks_key[1] if isinstance(r.blocks_key, tuple) and len(r.blocks_key) == 2 else -1
        out = [SEQ.pack(r.seq_id, r.uid, int(bkey), r.pos0, r.slot, r.shift, r.step_no, flags, r.rope_delta,
                        r.prompt_lp if r.prompt_lp is not None else -1, r.next_token, float(r.temperature),
                        len(r.tokens), keep, len(new), len(uni), *samp),
               struct.pack(f"<{len(r.tokens)}i", *r.tokens), struct.pack(f"<{len(new)}i", *new),
               struct.pack(f"<{len(uni)}f", *uni)]
        if r.rope_pos is not None:
            flat = [int(v) for row in (r.rope_pos.tolist() if hasattr(r.rope_pos, "tolist") else r.rope_pos) for v in row]
            out.append(struct.pack(f"<{len(flat)}i", *flat))
        return b"".join(out)

    def encode(self, name: str, *args) -> list:
        op = OPS[name]
        nseq = width = 0
        if name == "prefill":
            runs = args[0]
            nseq, payload = len(runs), b"".join(self._seq(r) for r in runs)
        elif name == "decode":
            runs, width = args
            nseq, payload = len(runs), b"".join(self._seq(r) for r in runs)
        elif name == "stop":
            payload = b""
        else:                              # small integer arguments
            payload = struct.pack(f"<{len(args)}q", *[int(a) for a in args])
        _prune(self._blocks)
        self._n += 1
        parts = max(1, (len(payload) + PART_BYTES - 1) // PART_BYTES)
        return [HEADER.pack(MAGIC, op, i, parts, 0, self._n, nseq, width, len(payload)) + payload[i * PART_BYTES:(i + 1) * PART_BYTES]
                for i in range(parts)]

    def forget(self, seq_id: int) -> None:
        self._blocks.pop(seq_id, None)


class FrameDecoder:
    """Follower side: rebuilds the call (name, args) from its parts and keeps the block tables."""

    def __init__(self):
        self._blocks: dict = {}
        self._parts: list = []
        self.expect = 1

    def _seq(self, buf: memoryview, off: int):
        (seq_id, uid, bkey, pos0, slot, shift, step_no, flags, rope_delta, prompt_lp, next_token, temperature,
         n_tok, keep, n_new, n_uni, s0, s1, s2, s3) = SEQ.unpack_from(buf, off)
        off += SEQ.size
        tokens = list(struct.unpack_from(f"<{n_tok}i", buf, off)); off += 4 * n_tok
        new = list(struct.unpack_from(f"<{n_new}i", buf, off)); off += 4 * n_new
        uni = list(struct.unpack_from(f"<{n_uni}f", buf, off)); off += 4 * n_uni
        blocks = self._blocks.get(seq_id, [])[:keep] + new
        self._blocks[seq_id] = blocks
        rope = None
        if flags & F_ROPE:
            flat = struct.unpack_from(f"<{3 * n_tok}i", buf, off); off += 12 * n_tok
            rope = [list(flat[i * n_tok:(i + 1) * n_tok]) for i in range(3)]
        run = SeqRun(seq_id, tokens, pos0, slot, shift, list(blocks), uid=uid, step_no=step_no, last_chunk=bool(flags & F_LAST_CHUNK),
                     temperature=temperature, want_seam=bool(flags & F_WANT_SEAM), rope_pos=rope, rope_delta=rope_delta,
                     prompt_lp=prompt_lp if flags & F_PROMPT_LP else None, next_token=next_token,
                     sampling=(s0, int(s1), s2, s3) if flags & F_SAMPLING else None, uniforms=uni or None,
                     blocks_key=(seq_id, bkey) if bkey >= 0 else None)
        return run, off

    def feed(self, frame: bytes):
        """One part in; (name, args) out when the call is complete, else None."""
        magic, op, part, parts, _, n, nseq, width, total = HEADER.unpack_from(frame, 0)
        if magic != MAGIC:
            raise ValueError("not a control frame")
        if n != self.expect or part != len(self._parts):
            raise ValueError(f"control frame out of order: call {n} part {part}, expected call {self.expect} part {len(self._parts)}")
        self._parts.append(frame[HEADER.size:])
        if len(self._parts) < parts:
            return None
        payload = b"".join(self._parts)
        self._parts = []
        self.expect += 1
        if len(payload) != total:
            raise ValueError(f"control frame payload is {len(payload)} bytes, header says {total}")
        name = OP_NAMES[op]
        buf = memoryview(payload)
        if name in ("prefill", "decode"):
            runs, off = [], 0
            for _ in range(nseq):
                run, off = self._seq(buf, off)
                runs.append(run)
            _prune(self._blocks)
            return (name, (runs,) if name == "prefill" else (runs, width))
        if name == "stop":
            return (name, ())
        return (name, tuple(struct.unpack(f"<{len(payload) // 8}q", payload)))

    def forget(self, seq_id: int) -> None:
        self._blocks.pop(seq_id, None)


class ShmChannel:
    """One shared-memory line per follower.  The leader posts every part to every line (a part waits,
    with a deadline, while a follower has not taken the frame that occupies the slot); a follower
    takes the parts of its own line in order."""

    def __init__(self, name: str, world: int, rank: int, create: Optional[bool] = None):
        from .shmline import ShmLine
        self.rank, self.world = rank, world
        create = (rank == 0) if create is None else create
        ranks = range(1, world) if rank == 0 else [rank]
        self.lines = {r: ShmLine(f"{name}-r{r}", create=create) for r in ranks}
        self._taken = 0

    def send(self, parts: list, deadline_s: float = 60.0) -> None:
        for r, line in self.lines.items():
            for part in parts:
                t0 = time.monotonic()
                while True:
                    try:
                        line.post(part)
                        break
                    except BlockingIOError:
                        if time.monotonic() - t0 > deadline_s:
                            raise TimeoutError(f"rank {r} has not taken a control frame for {deadline_s} s")
                        time.sleep(0)

    def recv(self, poll_s: float = 1.0, alive=None) -> bytes:
        """Next part of this follower's line.  `alive()` is asked between polls: a follower whose
        leader is gone stops waiting."""
        line = self.lines[self.rank]
        while True:
            try:
                got = line.take(self._taken, timeout_s=poll_s)
                self._taken += 1
                return got
            except TimeoutError:
                if alive is not None and not alive():
                    raise ConnectionError("the leader is gone")

    def close(self) -> None:
        for line in self.lines.values():
            line.close()
