"""The seam between the scheduler and whatever runs the model.

Parity: `crates/saber-sched/src/executor.rs:1-40` (trait StepExecutor: prefill chunks commit no
token except the last one, which commits exactly one; a decode step commits 1 + accepted tokens per
sequence) and the run descriptors the engine turns into index tables
(`crates/saber-exec/src/forward.rs:587-860`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Protocol


@dataclass
class SeqRun:
    """One sequence's share of a step, as the executor needs it."""
    seq_id: int
    tokens: list            # rows of this step
    pos0: int               # position of the first row
    slot: int               # recurrent-state slot
    shift: int              # rows of the previous decode step that were committed
    blocks: list            # physical KV blocks
    uid: int = 0
    step_no: int = 0
    last_chunk: bool = True      # prefill: does this chunk end the prompt?
    temperature: float = 0.0
    want_seam: bool = False
    rope_pos: Optional[object] = None   # int [3, rows]: rotary positions of a chunk of a prompt with images
    rope_delta: int = 0          # rotary position - index for rows after the prompt's images
    prompt_lp: Optional[int] = None   # prefill: log-probability of every next prompt token with this many alternatives
    next_token: int = -1         # the prompt token after this chunk (-1: the chunk ends the prompt)
    sampling: Optional[tuple] = None   # (temperature, top_k, top_p, min_p): the device may draw for this sequence
    uniforms: Optional[list] = None    # the uniform numbers of this step's head rows
    blocks_key: Optional[object] = None   # identity of `blocks`: an executor may keep the block table of an unchanged key on the device


@dataclass
class SeqOut:
    tokens: list                 # committed tokens (decode: accepted drafts + bonus; prefill: 1 or 0)
    drafts: list = field(default_factory=list)   # proposal for the next step
    seam: Optional[dict] = None  # top-k candidates + log-sum-exps for sampled rows
    prompt_lps: Optional[list] = None   # prefill: per row with a successor {token_id, logprob, top} of that successor
    logits_rows: Optional[object] = None


class StepExecutor(Protocol):
    max_seqs: int
    decode_batches: tuple
    decode_widths: tuple
    prefill_rungs: tuple
    page_tokens: int
    n_kv_blocks: int
    vocab: int

    def reset_slot(self, slot: int) -> None: ...
    def prefill(self, runs: list) -> list: ...
    def decode(self, runs: list, width: int) -> list: ...
    def snapshot_state(self, slot: int): ...
    def restore_state(self, slot: int, snap) -> None: ...
    def snapshot_bytes(self) -> int: ...
    def free_snapshot(self, snap) -> None: ...
