"""StepExecutor over `models.hybrid.HybridModel`: turns the scheduler's run descriptors into index
blobs, replays the captured bucket, and hands back committed tokens and the next drafts.

Parity: `crates/saber-engine/src/executor.rs:1-40` (RealExecutor over ForwardRunner) and the device
thread's step (`crates/saber-engine/src/device.rs:20751`): build index tables, one host->device copy,
graph launch, read picks, commit.  Recurrent-state snapshots for the prefix cache are device
resident copies of the slot's state and conv window (`crates/saber-sched/src/prefix_cache.rs:20-27`).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..models.hybrid import HybridModel, SeqStep, run_bucket
from ..sched.buckets import DEFAULT_DECODE_BATCHES, DEFAULT_PREFILL_RUNGS, select_batch, select_rung
from ..sched.executor import SeqOut, SeqRun


class HybridExecutor:
    def __init__(self, model: HybridModel, decode_batches=DEFAULT_DECODE_BATCHES, decode_widths=(1, 5, 8),
                 prefill_rungs=(128, 512, 2048), prefill_pack: int = 1, capture: bool = True,
                 prebuild: bool = False):
        self.model = model
        self.max_seqs = model.max_seqs
        self.decode_batches = tuple(b for b in decode_batches if b <= model.max_seqs) or (model.max_seqs,)
        self.decode_widths = tuple(w for w in decode_widths if w <= model.max_width)
        self.prefill_rungs = tuple(prefill_rungs)
        self.prefill_pack = prefill_pack
        self.page_tokens = model.cfg.page_tokens
        self.n_kv_blocks = model.kv_blocks
        self.vocab = model.cfg.vocab
        self.capture = capture
        self.census = {"graph_replays": 0, "eager_walks": 0, "launches": 0, "buckets_built": 0}
        if prebuild:
            for b in self.decode_batches:
                for w in self.decode_widths:
                    self._bucket("decode", b, w)
            for r in self.prefill_rungs:
                self._bucket("prefill", self.prefill_pack, r)

    def _bucket(self, kind: str, nseq: int, width: int):
        key = (kind, nseq, width)
        if key not in self.model.buckets:
            self.census["buckets_built"] += 1
        return self.model.build_bucket(kind, nseq, width, capture=self.capture)

    def reset_slot(self, slot: int) -> None:
        self.model.reset_slot(slot)

    @staticmethod
    def _step(r: SeqRun) -> SeqStep:
        return SeqStep(list(r.tokens), r.pos0, r.slot, r.shift, r.blocks, uid=r.uid, step_no=r.step_no,
                       rope_pos=r.rope_pos, rope_delta=r.rope_delta)

    def _count(self, b) -> None:
        self.census["graph_replays" if b.captured else "eager_walks"] += 1
        self.census["launches"] += b.n_launches

    def prefill(self, runs: list) -> list:
        rows = sum(len(r.tokens) for r in runs)
        b = self._bucket("prefill", max(self.prefill_pack, len(runs)), select_rung(rows, self.prefill_rungs))
        res = run_bucket(self.model, b, [self._step(r) for r in runs])
        self._count(b)
        return [SeqOut([res.tokens[j][0]] if r.last_chunk else [], res.drafts[j] if r.last_chunk else [])
                for j, r in enumerate(runs)]

    def decode(self, runs: list, width: int) -> list:
        b = self._bucket("decode", select_batch(len(runs), self.decode_batches), width)
        res = run_bucket(self.model, b, [self._step(r) for r in runs])
        self._count(b)
        return [SeqOut(res.tokens[j], res.drafts[j]) for j in range(len(runs))]

    # ---- prefix-cache snapshots (device resident)
    def snapshot_state(self, slot: int):
        m = self.model
        with torch.cuda.stream(m.stream):      # same stream as the programs: ordered after the chunk
            return {i: (m.gdn_state[i][slot].clone(), m.gdn_hist[i][slot, :3].clone()) for i in m.gdn_state}

    def restore_state(self, slot: int, snap) -> None:
        m = self.model
        with torch.cuda.stream(m.stream):
            for i, (st, win) in snap.items():
                m.gdn_state[i][slot].copy_(st)
                m.gdn_hist[i][slot].zero_()
                m.gdn_hist[i][slot, :3].copy_(win)

    def snapshot_bytes(self) -> int:
        m = self.model
        return sum(t[0].numel() * 4 + 3 * m.gdn_hist[i].shape[2] * 2 for i, t in m.gdn_state.items())  # t[0]: one slot

    def free_snapshot(self, snap) -> None:
        if isinstance(snap, dict):
            snap.clear()

    # ---- session parking: KV pages + the slot's recurrent state and conv window as one image
    def export_session(self, slot: int, blocks: list, n_tokens: int):
        """(header, payload): every tensor of the sequence, in a declared order, read back over a
        pinned staging buffer.  Parity: `crates/saber-engine/src/park.rs:1-30`."""
        m = self.model
        npages = (n_tokens + self.page_tokens - 1) // self.page_tokens
        idx = torch.tensor(blocks[:npages], dtype=torch.long, device=m.device)
        parts, layout, off = [], [], 0
        with torch.cuda.stream(m.stream):
            def add(name, t):
                nonlocal off
                raw = t.contiguous().view(torch.uint8).reshape(-1)
                host = torch.empty(raw.numel(), dtype=torch.uint8).pin_memory()
                host.copy_(raw, non_blocking=True)
                layout.append((name, str(t.dtype), list(t.shape), off, raw.numel()))
                parts.append(host)
                off += raw.numel()
            for i, kv in m.kv.items():
                add(f"kv.{i}", kv[idx])
            for i in m.gdn_state:
                add(f"gdn_state.{i}", m.gdn_state[i][slot])
                add(f"gdn_stash.{i}", m.gdn_stash[i][slot])
                add(f"gdn_hist.{i}", m.gdn_hist[i][slot])
            m.stream.synchronize()
        payload = b"".join(p.numpy().tobytes() for p in parts)
        return {"kind": "hybrid", "n_tokens": n_tokens, "npages": npages, "tensors": layout}, payload

    def import_session(self, slot: int, blocks: list, header: dict, payload: bytes) -> None:
        m = self.model
        npages = header["npages"]
        idx = torch.tensor(blocks[:npages], dtype=torch.long, device=m.device)
        buf = torch.frombuffer(bytearray(payload), dtype=torch.uint8)
        with torch.cuda.stream(m.stream):
            for name, dtype, shape, off, nbytes in header["tensors"]:
                kind, i = name.rsplit(".", 1)
                i = int(i)
                dst = {"kv": m.kv, "gdn_state": m.gdn_state, "gdn_stash": m.gdn_stash, "gdn_hist": m.gdn_hist}[kind][i]
                src = buf[off:off + nbytes].to(m.device).view(dst.dtype).reshape(shape)
                if kind == "kv":
                    dst[idx] = src
                else:
                    dst[slot].copy_(src)
            m.stream.synchronize()
