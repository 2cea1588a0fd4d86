"""The engine trait the HTTP plane talks to, and the events it gets back.

Parity: `crates/saber-serve/src/engine.rs:89-309` (trait Engine {submit, abort, stats, model},
EngineRequest, StepEvent: exactly one event per live sequence per engine step, which the server
turns into exactly one SSE chunk).
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Optional, Protocol


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0                 # 0 = off
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    max_tokens: int = 256
    stop_token_ids: tuple = ()
    ignore_eos: bool = False
    logprobs: Optional[int] = None
    prompt_logprobs: Optional[int] = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    def validate(self, vocab: int, max_ctx: int, prompt_len: int) -> list:
        problems = []
        if self.temperature < 0:
            problems.append("temperature must be >= 0")
        if not (0 < self.top_p <= 1):
            problems.append("top_p must be in (0, 1]")
        if self.top_k < 0:
            problems.append("top_k must be >= 0")
        if not (0 <= self.min_p <= 1):
            problems.append("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0:
            problems.append("repetition_penalty must be > 0")
        if self.max_tokens < 1:
            problems.append("max_tokens must be >= 1")
        if prompt_len + self.max_tokens > max_ctx:
            problems.append(f"prompt ({prompt_len}) + max_tokens ({self.max_tokens}) exceeds the context window ({max_ctx})")
        if self.logprobs is not None and not (0 <= self.logprobs <= 20):
            problems.append("logprobs must be in [0, 20]")
        if self.prompt_logprobs is not None and not (isinstance(self.prompt_logprobs, int) and 0 <= self.prompt_logprobs <= 20):
            problems.append("prompt_logprobs must be in [0, 20]")
        return problems


@dataclass
class EngineRequest:
    prompt_token_ids: list
    params: SamplingParams = field(default_factory=SamplingParams)
    request_id: Optional[str] = None
    eos_token_id: Optional[int] = None
    # prompts with images: {"rope_pos": int [3, N], "rope_delta": int, "release": callable | None};
    # image rows are token ids >= vocab (rows of the executor's image arena), so such a prompt is
    # neither looked up in nor added to the prefix caches
    mm: Optional[dict] = None


@dataclass
class StepEvent:
    seq_id: int
    new_token_ids: list
    finished: bool = False
    finish_reason: Optional[str] = None      # "stop" | "length" | "abort" | "error"
    error: Optional[str] = None
    prompt_tokens: int = 0
    cached_tokens: int = 0
    n_drafted: int = 0
    n_accepted: int = 0
    logprobs: Optional[list] = None
    prompt_logprobs: Optional[list] = None     # with the first token: {token_id, logprob, top} of prompt tokens 1..
    step_time_s: float = 0.0
    first_token: bool = False


class StepStream:
    """Thread-safe event stream of one request (the scheduler thread puts, the server gets)."""

    def __init__(self):
        self._q: "queue.Queue[StepEvent]" = queue.Queue()
        self._notify = None

    def set_notifier(self, fn) -> None:
        self._notify = fn

    def put(self, ev: StepEvent) -> None:
        self._q.put(ev)
        if self._notify:
            self._notify()

    def get(self, timeout: Optional[float] = None) -> StepEvent:
        return self._q.get(timeout=timeout)

    def get_nowait(self) -> Optional[StepEvent]:
        try:
            return self._q.get_nowait()
        except queue.Empty:
            return None


@dataclass
class Submission:
    seq_id: int
    events: StepStream
    submitted_at: float = field(default_factory=time.monotonic)


class EngineRefused(Exception):
    """The engine cannot take this request (queue full, prompt too long, fatal state)."""

    def __init__(self, reason: str, status: int = 503):
        super().__init__(reason)
        self.reason, self.status = reason, status


class Engine(Protocol):
    def submit(self, req: EngineRequest) -> Submission: ...
    def abort(self, seq_id: int) -> None: ...
    def stats(self) -> dict: ...
    def model(self) -> dict: ...
