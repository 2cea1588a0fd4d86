"""Continuous-batching scheduler: admission against the two allocators, prefix-cache reuse, chunked
prefill at planned rungs, speculative decode steps at a (batch, width) bucket, commit with stop
rules, one StepEvent per live sequence per step.

Parity: `crates/saber-sched/src/sched.rs:1452-1600` (three phases: prepare under the core lock,
execute without it, commit under it), `:1924` admit_waiting, `:4190` commit_half, `:4777`
commit_tokens; implements the serving plane's Engine trait (`:4911-4951` submit).
"""
from __future__ import annotations

import itertools
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..serve.engine_api import (EngineRefused, EngineRequest, SamplingParams, StepEvent, StepStream,
                                Submission)
from . import buckets as B
from .alloc import Arenas, GdnStateAllocator, OutOfBlocks, PagedKvAllocator
from .executor import SeqOut, SeqRun
from .prefix_cache import PrefixCache
from .width import WidthByBatch, WidthEma


@dataclass
class SchedulerConfig:
    max_seqs: int = 8
    max_ctx: int = 262144
    max_waiting: int = 256
    prefix_cache: bool = True
    prefix_cache_bytes: int = 6 << 30
    prefix_cache_min_tokens: int = 512
    prefix_cache_interval: int = 1024
    prefill_pack_seqs: int = 1           # sequences packed in one prefill step
    width_table: Optional[WidthByBatch] = None
    model_name: str = "saber"
    # mixed steps: while a prompt prefills, the decoding sequences still get a decode launch in the
    # same step, and the prompt's chunks are capped so that no stream waits for a whole prompt
    prefix_aware_admission: bool = True  # a request waits while a prefilling prompt is about to cache a prefix they share
    mixed_steps: bool = True
    mixed_chunk_rows: int = 512
    width_policy: str = "table"          # "table" (batch -> width) | "ema" (widest recent acceptance of the live sequences)
    lookup_drafts: bool = False          # sequences without model drafts propose by prompt lookup (n-gram continuation)
    park_victims: bool = False           # a waiting request that does not fit parks the decoding sequence with most tokens to go
    mem_valve: Optional[object] = None   # sched.mem_valve.MemValve: demote (drop cached prefixes) -> park -> refuse
    mem_valve_every: int = 64            # steps between polls


@dataclass
class Sequence:
    seq_id: int
    req: EngineRequest
    stream: StepStream
    prompt: list
    blocks: list = field(default_factory=list)
    slot: int = 0
    pos: int = 0                          # tokens whose KV / state are committed
    output: list = field(default_factory=list)
    drafts: list = field(default_factory=list)
    shift: int = 0
    step_no: int = 0
    chunks: deque = field(default_factory=deque)   # pending prefill chunks (pos, n)
    cut_points: set = field(default_factory=set)
    cached_tokens: int = 0
    finished: bool = False
    aborted: bool = False
    t_submit: float = field(default_factory=time.monotonic)
    t_first: Optional[float] = None
    t_admit: Optional[float] = None
    n_drafted: int = 0
    n_accepted: int = 0
    ema: Optional[object] = None          # WidthEma of this sequence (width_policy = "ema")
    blocks_key: Optional[tuple] = None    # changes whenever `blocks` is reassigned (admission, restore)
    hashes: Optional[list] = None         # block-chained hashes of the prompt (prefix-aware admission)
    prompt_lps: list = field(default_factory=list)   # log-probabilities of prompt tokens 1.., chunk by chunk

    @property
    def prefilling(self) -> bool:
        return bool(self.chunks)


class Scheduler:
    """Implements Engine over a StepExecutor. `step()` runs one engine step; `spawn_step_loop()`
    runs steps on a thread until `shutdown()`."""

    def __init__(self, executor, config: Optional[SchedulerConfig] = None, sampler=None):
        self.ex = executor
        self.cfg = config or SchedulerConfig(max_seqs=executor.max_seqs)
        self.cfg.max_seqs = min(self.cfg.max_seqs, executor.max_seqs)
        self.page = executor.page_tokens
        kv = PagedKvAllocator(executor.n_kv_blocks, self.page)
        self.arenas = Arenas(kv, GdnStateAllocator(self.cfg.max_seqs + 1))
        self.prefix = PrefixCache(kv, self.page, self.cfg.prefix_cache_bytes, self.cfg.prefix_cache_min_tokens,
                                  self.cfg.prefix_cache_interval, self.cfg.prefix_cache,
                                  free_snapshot=getattr(executor, "free_snapshot", None))
        self.width_table = self.cfg.width_table or WidthByBatch(
            {1: max(executor.decode_widths)}, tuple(sorted(executor.decode_widths)))
        self.sampler = sampler
        self.waiting: deque = deque()
        self.running: list = []
        self._ids = itertools.count(1)
        self._bkeys = itertools.count(1)
        self._lock = threading.Lock()
        # device work from outside the step loop (parking from a server thread) must not meet a step in
        # flight on the executor's stream (a bucket may be under capture there): both take this lock
        self._device_lock = threading.Lock()
        self._wake = threading.Condition(self._lock)
        self._stop = False
        self._thread: Optional[threading.Thread] = None
        self.fatal: Optional[str] = None
        self.counters = dict(steps=0, prefill_steps=0, decode_steps=0, prompt_tokens=0, generation_tokens=0,
                             drafts=0, draft_tokens=0, accepted_tokens=0, requests_finished=0,
                             requests_refused=0, requests_aborted=0, padding_slots=0,
                             sampled_steps=0, sampled_steps_device_agrees=0)
        self.accepted_per_pos = [0] * 16
        self.last_step_s = 0.0
        self.on_step = None                 # optional callback(timing dict) for metrics
        from ..utils.host_trace import HostTrace
        from .park import ParkTier
        self.trace = HostTrace(False)       # named host phases per step; off unless asked for
        self.park_tier = ParkTier()
        self.parked: dict = {}              # key -> Sequence whose device state lives in the park tier
        self.prompt_store = None            # optional sched.prompt_store.PromptStore (prefixes that survive restarts)
        self.valve_level = "ok"
        self.auto_parked: list = []         # keys parked by the scheduler itself (victims), restored when room appears
        self.counters.update(mixed_steps=0, deferred_for_prefix=0, victims_parked=0, victims_restored=0, lookup_drafts=0, valve_demotions=0)

    # ------------------------------------------------------------------------------ Engine trait
    def submit(self, req: EngineRequest) -> Submission:
        if self.fatal:
            raise EngineRefused(f"engine is down: {self.fatal}", 503)
        n = len(req.prompt_token_ids)
        if n == 0:
            raise EngineRefused("empty prompt", 400)
        problems = req.params.validate(self.ex.vocab, self.cfg.max_ctx, n)
        if req.params.prompt_logprobs is not None and not getattr(self.ex, "supports_prompt_logprobs", True):
            problems.append("prompt_logprobs is not available on this engine (vocabulary-sharded ranks)")
        vocab = self.ex.vocab
        top = vocab + (int(getattr(self.ex, "image_rows", 0)) if req.mm is not None else 0)
        bad = next((t for t in req.prompt_token_ids if not isinstance(t, int) or isinstance(t, bool) or t < 0 or t >= top), None)
        if bad is not None:
            problems.append(f"prompt token id {bad!r} is outside the vocabulary [0, {vocab})")
        if problems:
            raise EngineRefused("; ".join(problems), 400)
        if self.valve_level == "refuse":
            with self._lock:
                self.counters["requests_refused"] += 1
            raise EngineRefused("host memory is exhausted: no new requests for now", 503)
        with self._lock:
            if len(self.waiting) >= self.cfg.max_waiting:
                self.counters["requests_refused"] += 1
                raise EngineRefused("waiting queue is full", 503)
            seq = Sequence(next(self._ids), req, StepStream(), list(req.prompt_token_ids))
            self.waiting.append(seq)
            self._wake.notify_all()
        return Submission(seq.seq_id, seq.stream)

    def abort(self, seq_id: int) -> None:
        with self._lock:
            for s in itertools.chain(self.waiting, self.running):
                if s.seq_id == seq_id:
                    s.aborted = True
            self._wake.notify_all()

    def stats(self) -> dict:
        with self._lock:
            return dict(self.counters, running=len(self.running), waiting=len(self.waiting),
                        kv_free_blocks=self.arenas.kv.free_blocks, kv_total_blocks=self.arenas.kv.n_blocks,
                        gdn_free_slots=self.arenas.gdn.free_slots, prefix_entries=len(self.prefix),
                        prefix_hits=self.prefix.stats.hits, prefix_hit_tokens=self.prefix.stats.hit_tokens,
                        prefix_lookups=self.prefix.stats.lookups, last_step_s=self.last_step_s,
                        accepted_per_pos=list(self.accepted_per_pos), fatal=self.fatal)

    def model(self) -> dict:
        return {"id": self.cfg.model_name, "max_model_len": self.cfg.max_ctx, "vocab": self.ex.vocab}

    # ------------------------------------------------------------------------------ phase 1
    def _drain_aborted(self) -> None:
        for s in [s for s in self.waiting if s.aborted]:
            self.waiting.remove(s)
            self._finish(s, "abort")
        for s in [s for s in self.running if s.aborted]:
            self._finish(s, "abort")

    def _admit_waiting(self) -> None:
        while self.waiting and len(self.running) < self.cfg.max_seqs:
            s = self.waiting[0]
            # speculative rows write KV past the last committed token: keep one step of head-room
            total = len(s.prompt) + s.req.params.max_tokens + max(self.ex.decode_widths)
            # image rows are arena addresses, not content: no prefix sharing; prompt log-probabilities
            # need every prompt row to run
            mm = s.req.mm is not None or s.req.params.prompt_logprobs is not None
            if not mm and self.cfg.prefix_aware_admission and self.prefix.enabled:
                coming = self._coming_prefix(s)
                if coming > 0:
                    have = self.prefix.lookup(s.prompt, count=False)
                    if coming > (have.n_tokens if have else 0):
                        # a prompt that is prefilling right now shares a longer prefix with this one and
                        # will put it in the cache at a cut point ahead: admitting now would compute it twice
                        self.counters["deferred_for_prefix"] += 1
                        break
            hit = None if mm else self.prefix.lookup(s.prompt)
            shared = list(hit.blocks) if hit else []
            need = self.arenas.kv.blocks_for(total) - len(shared)
            if not self.arenas.can_admit(total, len(shared)):
                self.prefix.evict_for_blocks(need)          # cached pages yield to live requests
                hit = None if mm else self.prefix.lookup(s.prompt)   # the entry itself may have been evicted
                shared = list(hit.blocks) if hit else []
                if not self.arenas.can_admit(total, len(shared)) and self.cfg.park_victims and self._park_victim():
                    continue                                # a victim left the device: try this request again
                if not self.arenas.can_admit(total, len(shared)):
                    if not self.running:                    # can never fit
                        self.waiting.popleft()
                        self.counters["requests_refused"] += 1
                        self._emit(s, StepEvent(s.seq_id, [], True, "error",
                                                error="request does not fit the KV pool", prompt_tokens=len(s.prompt)))
                        continue
                    break
            self.waiting.popleft()
            s.blocks, s.slot = self.arenas.admit(total, shared)
            s.blocks_key = (s.seq_id, next(self._bkeys))
            s.t_admit = time.monotonic()
            start = 0
            stored = None
            if not hit and not mm and self.prompt_store is not None and self._can_park():
                stored = self.prompt_store.get(s.prompt)     # verified before anything reaches the device
            if hit:
                self.ex.restore_state(s.slot, hit.snapshot)
                start = hit.n_tokens
                s.cached_tokens = start
            elif stored is not None:
                self.ex.reset_slot(s.slot)
                from .park import ParkError
                try:
                    self.ex.import_session(s.slot, s.blocks, stored.header, stored.payload)
                    start = stored.header["n_tokens"]
                    s.cached_tokens = start
                except ParkError:            # e.g. an image other ranks no longer hold their shards of: a cold prefill
                    pass
            else:
                self.ex.reset_slot(s.slot)
            s.pos = start
            cuts = [] if mm else self.prefix.cut_points(len(s.prompt), start)
            s.cut_points = set(cuts)
            s.chunks = deque(B.cut_prompt(len(s.prompt), start, self.ex.prefill_rungs, cuts))
            self.running.append(s)

    def _coming_prefix(self, s: Sequence) -> int:
        """Tokens of `s`'s prompt that a currently prefilling sequence will have inserted into the
        prefix cache at one of its cut points still ahead of it (0: none)."""
        from .prefix_cache import chain_hashes
        if len(s.prompt) < self.prefix.min_tokens:
            return 0
        if s.hashes is None:
            s.hashes = chain_hashes(s.prompt[: len(s.prompt) - 1], self.page)
        best = 0
        for r in self.running:
            if not r.prefilling or r.req.mm is not None or not r.cut_points:
                continue
            if r.hashes is None:
                r.hashes = chain_hashes(r.prompt[: len(r.prompt) - 1], self.page)
            n, limit = 0, min(len(s.hashes), len(r.hashes))
            while n < limit and s.hashes[n] == r.hashes[n]:
                n += 1
            shared = n * self.page
            ahead = [c for c in r.cut_points if r.pos < c <= shared]
            if ahead:
                best = max(best, max(ahead))
        return best

    def _can_park(self) -> bool:
        return bool(getattr(self.ex, "supports_parking", hasattr(self.ex, "export_session")))

    def _park_victim(self) -> bool:
        """Parks the decoding sequence with the most tokens still to generate (called under both locks)."""
        if not self._can_park():
            return False
        cands = [x for x in self.running if not x.prefilling and not x.finished and x.output]
        if not cands:
            return False
        v = max(cands, key=lambda x: x.req.params.max_tokens - len(x.output))
        try:
            key = self._park_locked(v)
        except Exception as exc:           # the victim stays where it is; the waiting request keeps waiting
            import sys
            print(f"saber: parking a victim failed: {type(exc).__name__}: {exc}", file=sys.stderr, flush=True)
            self.counters["victim_park_failures"] = self.counters.get("victim_park_failures", 0) + 1
            return False
        self.auto_parked.append(key)
        self.counters["victims_parked"] += 1
        return True

    def _restore_victims(self) -> None:
        """Brings scheduler-parked sequences back when nobody waits and there is room again."""
        while self.auto_parked and not self.waiting and len(self.running) < self.cfg.max_seqs:
            key = self.auto_parked[0]
            s = self.parked.get(key)
            if s is None:
                self.auto_parked.pop(0)
                continue
            total = len(s.prompt) + s.req.params.max_tokens + max(self.ex.decode_widths)
            if not self.arenas.can_admit(total, 0):
                return
            self.auto_parked.pop(0)
            self._restore_locked(key)
            self.counters["victims_restored"] += 1

    def _poll_valve(self) -> None:
        v = self.cfg.mem_valve
        if v is None or self.counters["steps"] % max(1, self.cfg.mem_valve_every):
            return
        level = v.poll()
        self.valve_level = level
        if level in ("demote", "park", "refuse"):
            dropped = self.prefix.evict_for_blocks(1 << 30)      # cached prefixes (pages + host snapshots) go first
            self.counters["valve_demotions"] += int(bool(dropped) or 0)
        if level in ("park", "refuse") and len(self.running) > 1:
            self._park_victim()

    def _plan(self) -> list:
        """The step's phases, in launch order: ("prefill", [(seq, pos, n)]) and / or
        ("decode", seqs, width, batch).  With mixed steps a prefill chunk (capped) and the decode
        launch of the other sequences share the step; without, prefill goes first and alone."""
        phases = []
        pre = [s for s in self.running if s.prefilling]
        dec = [s for s in self.running if not s.finished and not s.prefilling]
        mixed = bool(pre and dec and self.cfg.mixed_steps)
        if pre:
            picks, rows = [], 0
            top = max(self.ex.prefill_rungs)
            cap = min(top, self.cfg.mixed_chunk_rows) if mixed else top
            for s in pre[: max(1, self.cfg.prefill_pack_seqs)]:
                pos, n = s.chunks[0]
                if n > cap:                       # a capped chunk: the rest stays at the head of the queue
                    s.chunks[0] = (pos + cap, n - cap)
                    s.chunks.appendleft((pos, cap))
                    n = cap
                if picks and rows + n > cap:
                    break
                picks.append((s, pos, n))
                rows += n
            phases.append(("prefill", picks))
            if not mixed:
                return phases
        if dec:
            batch = B.select_batch(len(dec), self.ex.decode_batches)
            if self.cfg.width_policy == "ema":
                captured = self.width_table.captured
                width = max(s.ema.width(captured) if s.ema is not None else max(captured) for s in dec)
            else:
                width = self.width_table.width_for(len(dec))
            phases.append(("decode", dec, width, batch))
        return phases

    def _launch(self, phase):
        if phase[0] == "prefill":
            runs = [SeqRun(s.seq_id, s.prompt[pos:pos + n], pos, s.slot, 0, s.blocks, uid=s.seq_id,
                           last_chunk=(pos + n == len(s.prompt)),
                           temperature=s.req.params.temperature, want_seam=self._wants_seam(s),
                           rope_pos=(None if s.req.mm is None else
                                     [list(ax[pos:pos + n]) for ax in s.req.mm["rope_pos"]]),
                           prompt_lp=s.req.params.prompt_logprobs,
                           next_token=(s.prompt[pos + n] if pos + n < len(s.prompt) else -1),
                           blocks_key=s.blocks_key,
                           **(self._device_draw(s, 1) if pos + n == len(s.prompt) else {}))
                    for s, pos, n in phase[1]]
            return self.ex.prefill(runs)
        _, dec, width, batch = phase
        runs = []
        for s in dec:
            drafts = s.drafts
            if self.cfg.lookup_drafts and width > 1 and not any(drafts):
                from ..runtime.lookup import lookup_draft
                drafts = lookup_draft(s.prompt + s.output, width - 1)
                self.counters["lookup_drafts"] += 1
            s.drafts = (list(drafts) + [0] * width)[: width - 1]
            runs.append(SeqRun(s.seq_id, [s.output[-1]] + s.drafts, s.pos, s.slot, s.shift, s.blocks,
                               uid=s.seq_id, step_no=s.step_no, temperature=s.req.params.temperature,
                               want_seam=self._wants_seam(s),
                               rope_delta=(0 if s.req.mm is None else int(s.req.mm.get("rope_delta", 0))),
                               blocks_key=s.blocks_key,
                               **self._device_draw(s, width)))
        return self.ex.decode(runs, width)

    # ------------------------------------------------------------------------------ the step
    def step(self) -> bool:
        """One engine step. Returns False when there was nothing to do.

        Plan, Launch and Accept all run under the device lock: parking and restoring from another
        thread (which take the same lock) can therefore never slip between a plan and its launch.
        Whatever goes wrong in any phase ends in the fatal law: every request learns the reason."""
        t0 = time.monotonic()
        try:
            with self._device_lock:
                with self.trace.phase("Plan"), self._lock:
                    self._drain_aborted()
                    self._poll_valve()
                    self._restore_victims()
                    self._admit_waiting()
                    phases = self._plan()
                if not phases:
                    return False
                for phase in phases:
                    with self.trace.phase("Launch"):
                        outs = self._launch(phase)
                    dt = time.monotonic() - t0
                    with self.trace.phase("Accept"), self._lock:
                        if phase[0] == "prefill":
                            self._commit_prefill(phase[1], outs, dt)
                        else:
                            self._commit_decode(phase[1], phase[2], phase[3], outs, dt)
                with self._lock:
                    self.counters["steps"] += 1
                    self.counters["mixed_steps"] += int(len(phases) > 1)
                    self.last_step_s = dt
        except Exception as exc:       # every request learns why (fatal law); the loop ends
            self.set_fatal(f"step failed: {exc!r}")
            raise
        self.trace.end_step()
        if self.on_step:
            for phase in phases:
                self.on_step({"kind": phase[0], "seconds": dt, "live": len(phase[1])})
        return True

    # ------------------------------------------------------------------------------ parking / warm prompts
    def park(self, seq_id: int) -> str:
        """Moves a decoding sequence off the device: its KV pages and state slot become one verified
        image in the park tier, its blocks and slot are released.  Returns the key to restore with."""
        if not self._can_park():
            raise EngineRefused("session parking is not available on this engine", 501)
        with self._device_lock, self._lock:
            s = next((x for x in self.running if x.seq_id == seq_id), None)
            if s is None or s.prefilling or s.finished:
                raise EngineRefused(f"sequence {seq_id} is not a decoding sequence", 409)
            try:
                return self._park_locked(s)
            except NotImplementedError as exc:
                raise EngineRefused(f"session parking is not available on this engine: {exc}", 501)

    def _park_locked(self, s: Sequence) -> str:
        from .park import ParkImage
        header, payload = self.ex.export_session(s.slot, s.blocks, s.pos)
        key = f"seq{s.seq_id}"
        header.update(seq_id=s.seq_id, pos=s.pos, shift=s.shift, step_no=s.step_no)
        self.park_tier.put(key, ParkImage.build(header, payload))
        self.running.remove(s)
        self.arenas.release(s.blocks, s.slot)
        s.blocks, s.slot = [], 0
        self.parked[key] = s
        return key

    def restore(self, key: str) -> int:
        """Brings a parked sequence back (fresh blocks and slot, bytes verified first)."""
        with self._device_lock, self._lock:
            s = self.parked.get(key)
            if s is None:
                raise EngineRefused(f"no parked session {key!r}", 404)
            total = len(s.prompt) + s.req.params.max_tokens + max(self.ex.decode_widths)
            if len(self.running) >= self.cfg.max_seqs or not self.arenas.can_admit(total, 0):
                raise EngineRefused("no room to restore the session now", 503)
            from .park import ParkError
            try:
                sid = self._restore_locked(key)
            except ParkError as exc:       # the image is gone or corrupt: the session is lost, say so once
                self.parked.pop(key, None)
                s.finished = True
                self._emit(s, StepEvent(s.seq_id, [], True, "error", error=f"parked session lost: {exc}",
                                        prompt_tokens=len(s.prompt)))
                raise EngineRefused(f"parked session {key!r} cannot be restored: {exc}", 410)
            except NotImplementedError as exc:
                raise EngineRefused(f"session parking is not available on this engine: {exc}", 501)
            if key in self.auto_parked:
                self.auto_parked.remove(key)
            return sid

    def _restore_locked(self, key: str) -> int:
        s = self.parked[key]
        total = len(s.prompt) + s.req.params.max_tokens + max(self.ex.decode_widths)
        img = self.park_tier.take(key)            # raises ParkError on a corrupt image: nothing reached the device
        s.blocks, s.slot = self.arenas.admit(total, [])
        s.blocks_key = (s.seq_id, next(self._bkeys))
        self.ex.import_session(s.slot, s.blocks, img.header, img.payload)
        del self.parked[key]
        self.running.append(s)
        self._wake.notify_all()
        return s.seq_id

    def warm(self, prompts: list) -> int:
        """Warm prompts: run each prompt once (one generated token) so that its pages and state
        snapshots are in the prefix cache before the first user request arrives."""
        subs = [self.submit(EngineRequest(list(p), SamplingParams(max_tokens=1, ignore_eos=True))) for p in prompts]
        self.run_until_idle()
        return len(subs)

    # ------------------------------------------------------------------------------ phase 3
    def _commit_prefill(self, picks, outs, dt) -> None:
        self.counters["prefill_steps"] += 1
        for (s, pos, n), out in zip(picks, outs):
            s.chunks.popleft()
            s.pos = pos + n
            if out.prompt_lps is not None:
                s.prompt_lps.extend(out.prompt_lps)
            self.counters["prompt_tokens"] += n
            if s.pos in s.cut_points:
                snap = self.ex.snapshot_state(s.slot)
                self.prefix.insert(s.prompt, s.pos, s.blocks, snap, self.ex.snapshot_bytes())
                st = self.prompt_store
                if st is not None and self._can_park() and not st.has(s.prompt, s.pos):
                    from .park import ParkImage
                    header, payload = self.ex.export_session(s.slot, s.blocks, s.pos)
                    header["n_tokens"] = s.pos
                    st.put(s.prompt, s.pos, ParkImage.build(header, payload))
            if s.pos == len(s.prompt):
                tok = self._choose(s, out, 0, out.tokens[0] if out.tokens else 0)
                s.drafts = list(out.drafts)
                s.shift = 0
                s.t_first = time.monotonic()
                self._append(s, [tok], dt, first=True, lps=self._logprobs(s, out, [tok], 0))

    def _commit_decode(self, dec, width, batch, outs, dt) -> None:
        self.counters["decode_steps"] += 1
        self.counters["padding_slots"] += batch - len(dec)
        for s, out in zip(dec, outs):
            toks = list(out.tokens)
            if not s.req.params.greedy and self.sampler is not None and out.seam is not None:
                toks = self._accept_sampled(s, out, width)
                # census: did the device's own draw (same candidates, same uniform numbers) commit the same tokens?
                self.counters["sampled_steps"] += 1
                self.counters["sampled_steps_device_agrees"] += int(list(out.tokens) == toks)
            n = len(toks)
            self.counters["drafts"] += 1
            self.counters["draft_tokens"] += width - 1
            self.counters["accepted_tokens"] += n - 1
            for k in range(min(n - 1, len(self.accepted_per_pos))):
                self.accepted_per_pos[k] += 1
            s.n_drafted += width - 1
            s.n_accepted += n - 1
            if self.cfg.width_policy == "ema":
                if s.ema is None:
                    s.ema = WidthEma()
                s.ema.update(n - 1)
            s.pos += n
            s.shift = n
            s.step_no += 1
            s.drafts = list(out.drafts)
            self._append(s, toks, dt, drafted=width - 1, accepted=n - 1, lps=self._logprobs(s, out, toks, 0))

    def _device_draw(self, s: Sequence, n_rows: int) -> dict:
        """Sampling parameters and the uniform numbers of this step's head rows, for executors that
        draw on the device (the host repeats the draw and stays authoritative)."""
        smp = self.sampler
        if s.req.params.greedy or smp is None or not hasattr(smp, "device_params"):
            return {}
        dp = smp.device_params(s.req.params)
        if dp is None:
            return {}
        return {"sampling": dp, "uniforms": smp.uniforms(s.req.params, s.seq_id, len(s.output), n_rows)}

    @staticmethod
    def _wants_seam(s: Sequence) -> bool:
        return (not s.req.params.greedy) or s.req.params.logprobs is not None

    @staticmethod
    def _logprobs(s: Sequence, out: SeqOut, toks: list, row0: int) -> Optional[list]:
        """Per committed token: its log-probability and the `logprobs` most likely alternatives, from
        the seam row that produced it (log-softmax at temperature 1 over the whole vocabulary: value
        minus the row's log-sum-exp).  A token outside the 64 candidates gets the floor of the seam."""
        n = s.req.params.logprobs
        if n is None or out.seam is None:
            return None
        res = []
        for j, t in enumerate(toks):
            r = row0 + j
            if r >= len(out.seam["ids"]):
                break
            ids, vals = out.seam["ids"][r], out.seam["vals"][r]
            lse = out.seam["lse"][r]
            lse = lse[0] if isinstance(lse, (list, tuple)) else lse
            lp = (vals[ids.index(t)] if t in ids else vals[-1]) - lse
            res.append({"token_id": int(t), "logprob": float(lp),
                        "top": [(int(i), float(v - lse)) for i, v in list(zip(ids, vals))[:n]]})
        return res

    def _choose(self, s: Sequence, out: SeqOut, row: int, greedy_tok: int) -> int:
        if s.req.params.greedy or self.sampler is None or out.seam is None:
            return greedy_tok
        return self.sampler.sample_row(out.seam, row, s.req.params, s.prompt, s.output, len(s.output), s.seq_id)

    def _accept_sampled(self, s: Sequence, out: SeqOut, width: int) -> list:
        """Sampled rows: the token at each output position is a function of (seed, position), so the
        longest draft prefix that matches what the sampler draws is accepted, exactly as in greedy
        verification (`crates/saber-exec/src/forward.rs:475`, `seeded_invariance.rs:1-20`)."""
        drafts = (s.drafts + [0] * width)[: width - 1]
        toks, hist = [], list(s.output)
        for r in range(width):
            t = self.sampler.sample_row(out.seam, r, s.req.params, s.prompt, hist, len(hist), s.seq_id)
            toks.append(t)
            hist.append(t)
            if r >= width - 1 or drafts[r] != t:
                break
        return toks

    def _append(self, s: Sequence, toks: list, dt: float, first: bool = False, drafted: int = 0,
                accepted: int = 0, lps: Optional[list] = None) -> None:
        p = s.req.params
        kept, reason = [], None
        for t in toks:
            kept.append(t)
            s.output.append(t)
            if not p.ignore_eos and s.req.eos_token_id is not None and t == s.req.eos_token_id:
                reason = "stop"
            elif t in p.stop_token_ids:
                reason = "stop"
            elif len(s.output) >= p.max_tokens:
                reason = "length"
            if reason:
                break
        if len(kept) < len(toks):             # tokens past the stop are not committed
            s.pos -= len(toks) - len(kept)
            s.shift = len(kept)
        self.counters["generation_tokens"] += len(kept)
        ev = StepEvent(s.seq_id, kept, reason is not None, reason, prompt_tokens=len(s.prompt),
                       cached_tokens=s.cached_tokens, n_drafted=drafted, n_accepted=accepted,
                       step_time_s=dt, first_token=first,
                       logprobs=(lps[:len(kept)] if lps is not None else None),
                       prompt_logprobs=(list(s.prompt_lps) if first and s.req.params.prompt_logprobs is not None else None))
        if reason:
            self._finish(s, reason, ev)
        else:
            self._emit(s, ev)

    def _finish(self, s: Sequence, reason: str, ev: Optional[StepEvent] = None) -> None:
        if s.finished:
            return
        s.finished = True
        if s in self.running:
            self.running.remove(s)
            self.arenas.release(s.blocks, s.slot)
        if s.req.mm is not None and callable(s.req.mm.get("release")):
            s.req.mm["release"]()              # the request's rows of the image arena
            s.req.mm["release"] = None
        if reason == "abort":
            self.counters["requests_aborted"] += 1
        else:
            self.counters["requests_finished"] += 1
        self._emit(s, ev or StepEvent(s.seq_id, [], True, reason, prompt_tokens=len(s.prompt)))

    def _emit(self, s: Sequence, ev: StepEvent) -> None:
        s.stream.put(ev)

    # ------------------------------------------------------------------------------ loop / fatal
    def set_fatal(self, reason: str) -> None:
        """Teardown law: every queued and in-flight request gets the reason, new ones are refused."""
        with self._lock:
            if self.fatal:
                return
            self.fatal = reason
            for s in list(self.waiting) + list(self.running):
                s.finished = True
                s.stream.put(StepEvent(s.seq_id, [], True, "error", error=reason, prompt_tokens=len(s.prompt)))
            self.waiting.clear()
            self.running.clear()
            self._wake.notify_all()

    def spawn_step_loop(self) -> threading.Thread:
        def loop():
            while True:
                with self._lock:
                    # (a victim the scheduler parked is work too: it comes back as soon as nobody waits)
                    while not self._stop and not self.fatal and not self.waiting and not self.running and not self.auto_parked:
                        self._wake.wait(timeout=0.5)
                    if self._stop or self.fatal:
                        return
                try:
                    self.step()
                except Exception as exc:        # step() has already told every request (fatal law)
                    if not self.fatal:
                        self.set_fatal(f"step loop failed: {exc!r}")
                    return
        self._thread = threading.Thread(target=loop, name="saber-step-loop", daemon=True)
        self._thread.start()
        return self._thread

    def shutdown(self) -> None:
        with self._lock:
            self._stop = True
            self._wake.notify_all()
        if self._thread:
            self._thread.join(timeout=5)

    def run_until_idle(self, max_steps: int = 100000) -> int:
        n = 0
        while n < max_steps and self.step():
            n += 1
        return n
