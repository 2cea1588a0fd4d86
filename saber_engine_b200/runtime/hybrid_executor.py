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

N_SEAM_K = 64


def merge_rank_seams(ids, vals, lse):
    """ids / vals [ranks, rows, K] (each rank's best K of its vocabulary shard, value desc), lse
    [ranks, rows] -> the best K of the union (value desc, id asc) and the log-sum-exp of the whole row."""
    import numpy as np
    R, M, K = ids.shape
    ai = np.transpose(ids, (1, 0, 2)).reshape(M, R * K)
    av = np.transpose(vals, (1, 0, 2)).reshape(M, R * K)
    order = np.lexsort((ai, -av), axis=1)[:, :K]
    top = lse.max(axis=0)
    return (np.take_along_axis(ai, order, 1), np.take_along_axis(av, order, 1),
            top + np.log(np.exp(lse - top[None]).sum(axis=0)))


def gather_rank_seams(ids, vals, lse, device):
    """All-gather of the ranks' seams (a small NCCL collective outside the captured program: only steps
    with a sampled request pay for it), merged identically on every rank."""
    import numpy as np
    import torch.distributed as dist
    if not dist.is_initialized():
        raise RuntimeError("sampled requests on vocabulary-sharded ranks need torch.distributed")
    M, K = ids.shape
    mine = torch.cat([torch.from_numpy(np.ascontiguousarray(ids)).view(torch.int32).reshape(-1),
                      torch.from_numpy(np.ascontiguousarray(vals)).view(torch.int32).reshape(-1),
                      torch.from_numpy(np.ascontiguousarray(lse)).view(torch.int32).reshape(-1)]).to(device)
    world = dist.get_world_size()
    allr = torch.empty(world * mine.numel(), dtype=torch.int32, device=device)
    dist.all_gather_into_tensor(allr, mine)
    a = allr.cpu().numpy().reshape(world, -1)
    return merge_rank_seams(a[:, :M * K].reshape(world, M, K),
                            a[:, M * K: 2 * M * K].view(np.float32).reshape(world, M, K),
                            a[:, 2 * M * K:].view(np.float32).reshape(world, M))


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
        self.image_rows = int(getattr(model, "image_rows", 0))     # token ids [vocab, vocab + image_rows) name rows of the image arena
        self.supports_parking = model.tp == 1
        self.capture = capture
        self.census = {"graph_replays": 0, "eager_walks": 0, "launches": 0, "buckets_built": 0}
        # the head over every prompt row needs the whole vocabulary on one GPU
        self.supports_prompt_logprobs = True      # on vocabulary shards the rows' candidates and successor logits are merged on the device
        if prebuild:
            for b in self.decode_batches:
                for w in self.decode_widths:
                    self._bucket("decode", b, w)
            for r in self.prefill_rungs:
                self._bucket("prefill", self.prefill_pack, r)

    def _bucket(self, kind: str, nseq: int, width: int, seam: bool = False, plp: bool = False):
        key = ((kind, nseq, width, "seam") if seam else (kind, nseq, width)) + (("plp",) if plp else ())
        if key not in self.model.buckets:
            self.census["buckets_built"] += 1
        return self.model.build_bucket(kind, nseq, width, capture=self.capture, seam=seam, plp=plp)

    @staticmethod
    def _prompt_lps(b, runs: list) -> list:
        """Per run: for every row of the chunk that has a successor in the prompt, the successor's
        log-probability (its logit minus the row's log-sum-exp) and the best alternatives."""
        import numpy as np
        K, M = N_SEAM_K, b.M
        a = b.plp_host.numpy()
        ids = a[:M * K].reshape(M, K)
        vals = a[M * K: 2 * M * K].view(np.float32).reshape(M, K)
        lse = a[2 * M * K: 2 * M * K + 2 * M].view(np.float32).reshape(M, 2)[:, 0]
        nxt = a[2 * M * K + 2 * M:].view(np.float32)
        out, row = [], 0
        for r in runs:
            n, res = len(r.tokens), None
            if r.prompt_lp is not None:
                succ = list(r.tokens[1:]) + [r.next_token]
                res = [{"token_id": int(succ[i]), "logprob": float(nxt[row + i] - lse[row + i]),
                        "top": [(int(t), float(v - lse[row + i])) for t, v in zip(ids[row + i][:r.prompt_lp], vals[row + i][:r.prompt_lp])]}
                       for i in range(n) if succ[i] >= 0]
            out.append(res)
            row += n
        return out

    def _seams(self, b, rows_of: list) -> list:
        """Per run: {"ids", "vals", "lse"} over the run's head rows, from the bucket's read-back blob (on
        vocabulary-sharded ranks the program has already merged the ranks' candidates on the device)."""
        import numpy as np
        K, Mh = N_SEAM_K, b.Mh
        a = b.seam_host.numpy()
        ids = a[:Mh * K].reshape(Mh, K)
        vals = a[Mh * K: 2 * Mh * K].view(np.float32).reshape(Mh, K)
        lse = a[2 * Mh * K:].view(np.float32).reshape(Mh, 2)[:, 0]
        return [{"ids": ids[r0:r1].tolist(), "vals": vals[r0:r1].tolist(), "lse": lse[r0:r1].tolist()}
                for r0, r1 in rows_of]

    def reset_slot(self, slot: int) -> None:
        self.model.reset_slot(slot)

    @staticmethod
    def _step(r: SeqRun) -> SeqStep:
        return SeqStep(list(r.tokens), r.pos0, r.slot, r.shift, r.blocks, uid=r.uid, step_no=r.step_no,
                       rope_pos=r.rope_pos, rope_delta=r.rope_delta, next_token=getattr(r, "next_token", -1),
                       sampling=getattr(r, "sampling", None), uniforms=getattr(r, "uniforms", None),
                       blocks_key=getattr(r, "blocks_key", None))

    def _count(self, b) -> None:
        self.census["graph_replays" if b.captured else "eager_walks"] += 1
        self.census["launches"] += b.n_launches

    def prefill(self, runs: list) -> list:
        rows = sum(len(r.tokens) for r in runs)
        want = any(r.want_seam and r.last_chunk for r in runs)
        plp = any(r.prompt_lp is not None for r in runs)
        b = self._bucket("prefill", max(self.prefill_pack, len(runs)), select_rung(rows, self.prefill_rungs), seam=want, plp=plp)
        res = run_bucket(self.model, b, [self._step(r) for r in runs])
        self._count(b)
        seams = self._seams(b, [(j, j + 1) for j in range(len(runs))]) if want else [None] * len(runs)
        plps = self._prompt_lps(b, runs) if plp else [None] * len(runs)
        return [SeqOut([res.tokens[j][0]] if r.last_chunk else [], res.drafts[j] if r.last_chunk else [],
                       seam=seams[j] if (r.want_seam and r.last_chunk) else None, prompt_lps=plps[j])
                for j, r in enumerate(runs)]

    def decode(self, runs: list, width: int) -> list:
        want = any(r.want_seam for r in runs)
        b = self._bucket("decode", select_batch(len(runs), self.decode_batches), width, seam=want)
        res = run_bucket(self.model, b, [self._step(r) for r in runs])
        self._count(b)
        seams = self._seams(b, [(j * width, (j + 1) * width) for j in range(len(runs))]) if want else [None] * len(runs)
        return [SeqOut(res.tokens[j], res.drafts[j], seam=seams[j] if runs[j].want_seam else None)
                for j in range(len(runs))]

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

    def copy_lane(self):
        if getattr(self, "_lane", None) is None:
            from .device_rt import CopyLane
            self._lane = CopyLane(self.model.device)
        return self._lane

    # ---- session parking: KV pages + the slot's recurrent state and conv window as one image
    def export_session(self, slot: int, blocks: list, n_tokens: int):
        """(header, payload): every tensor of the sequence, in a declared order, read back over a
        pinned staging buffer.  Parity: `crates/saber-engine/src/park.rs:1-30`."""
        m = self.model
        npages = (n_tokens + self.page_tokens - 1) // self.page_tokens
        idx = torch.tensor(blocks[:npages], dtype=torch.long, device=m.device)
        parts, layout, off = [], [], 0
        lane = self.copy_lane()
        with torch.cuda.stream(m.stream):          # the gathers run on the step stream (ordered after the last step) ...
            staged = [(f"kv.{i}", kv[idx]) for i, kv in m.kv.items()]
            staged += [(f"draft_kv.{i}", kv[idx]) for i, kv in getattr(m, "draft_kv", {}).items()]   # the drafter's context-KV store
            for i in m.gdn_state:
                staged += [(f"gdn_state.{i}", m.gdn_state[i][slot].clone()), (f"gdn_stash.{i}", m.gdn_stash[i][slot].clone()),
                           (f"gdn_hist.{i}", m.gdn_hist[i][slot].clone())]
        lane.after(m.stream)                       # ... and the bytes leave on the copy lane: later steps do not wait for them
        for name, t in staged:
            raw = t.contiguous().view(torch.uint8).reshape(-1)
            host = lane.pinned(raw.numel(), tag=f"export.{name}")
            lane.d2h(host, raw)
            layout.append((name, str(t.dtype), list(t.shape), off, raw.numel()))
            parts.append(host)
            off += raw.numel()
        lane.wait(self.model.step_timeout_s)
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
                dst = {"kv": m.kv, "draft_kv": getattr(m, "draft_kv", {}), "gdn_state": m.gdn_state, "gdn_stash": m.gdn_stash,
                       "gdn_hist": m.gdn_hist}[kind][i]
                src = buf[off:off + nbytes].to(m.device).view(dst.dtype).reshape(shape)
                if kind in ("kv", "draft_kv"):
                    dst[idx] = src
                else:
                    dst[slot].copy_(src)
            m.stream.synchronize()
