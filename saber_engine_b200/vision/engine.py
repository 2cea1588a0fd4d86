"""Images into the engine: an arena of rows behind the token table (the tower writes them, a prompt
names them as token ids >= vocab), and the builder that turns (token ids with `<|image_pad|>`
placeholders, images) into an `EngineRequest` with three-axis rotary positions.

    vis = VisionFrontend(executor, VisionTowerGPU(cfg, weights), image_pad_id)
    req = vis.build_request(token_ids, [rgb_uint8_array, ...], sampling_params)
    scheduler.submit(req)            # the arena rows are released when the request finishes

Parity: `crates/saber-sched/src/serve.rs:520` (`build_state_with_vision`: the serve plane owns a
tower arena of a fixed number of patches; larger images are downscaled to it, not refused),
`crates/saber-vision-input/src/processor.rs:46-70`, the mrope positions of `crates/saber-exec`.
"""
from __future__ import annotations

import threading
from typing import Callable, Optional, Sequence

import numpy as np
import torch

from ..serve.engine_api import EngineRefused, EngineRequest, SamplingParams
from . import processor as VP


class RowArena:
    """First-fit allocator over `rows` rows; spans are (first row, count)."""

    def __init__(self, rows: int):
        self.rows = rows
        self._free = [(0, rows)] if rows > 0 else []
        self._lock = threading.Lock()

    def alloc(self, n: int) -> Optional[int]:
        with self._lock:
            for i, (a, c) in enumerate(self._free):
                if c >= n:
                    if c == n:
                        self._free.pop(i)
                    else:
                        self._free[i] = (a + n, c - n)
                    return a
        return None

    def free(self, a: int, n: int) -> None:
        with self._lock:
            spans = sorted(self._free + [(a, n)])
            merged = []
            for s, c in spans:
                if merged and merged[-1][0] + merged[-1][1] == s:
                    merged[-1] = (merged[-1][0], merged[-1][1] + c)
                else:
                    merged.append((s, c))
            self._free = merged

    @property
    def free_rows(self) -> int:
        with self._lock:
            return sum(c for _, c in self._free)


class VisionFrontend:
    def __init__(self, executor, tower, image_pad_id: int, proc: VP.ProcessorConfig = VP.ProcessorConfig(),
                 encode: Optional[Callable] = None):
        """`executor.model` must have been built with `image_rows > 0`.  `encode(pixel_values, grids,
        out_rows)` defaults to the tower's forward into the arena rows (tests pass a CPU stand-in)."""
        self.ex, self.tower, self.image_pad_id = executor, tower, image_pad_id
        model = executor.model
        self.vocab = model.cfg.vocab
        self.table = model.embed_table
        self.arena = RowArena(int(getattr(model, "image_rows", 0)))
        if self.arena.rows <= 0:
            raise ValueError("the model was built without image rows")
        merge2 = proc.merge_size ** 2
        cap_patches = min(self.arena.rows * merge2, getattr(tower, "max_patches", self.arena.rows * merge2))
        self.proc = proc.clamped_to_arena(cap_patches)
        self._encode = encode or self._encode_tower
        self._tower_lock = threading.Lock()      # the tower's buffers serve one forward at a time
        self._stream = None
        self.counters = {"images": 0, "patch_rows": 0, "image_tokens": 0, "refused": 0}

    def _encode_tower(self, pixel_values: torch.Tensor, grids, out_rows: torch.Tensor) -> None:
        # A stream of its own: the engine's step loop (another thread) may be capturing a new bucket
        # on the model's stream at this very moment, and nothing else may touch a capturing stream.
        # The rows are complete on the host's clock before the request is submitted, so the prefill
        # that reads them needs no device-side dependency.
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=self.table.device)
        with torch.cuda.stream(self._stream):
            self.tower.forward(pixel_values, grids, out=out_rows, graph=True)
        self._stream.synchronize()

    def build_request(self, token_ids: Sequence[int], images: Sequence[np.ndarray],
                      params: Optional[SamplingParams] = None, **kw) -> EngineRequest:
        params = params or SamplingParams()
        if not images:
            return EngineRequest(list(token_ids), params, **kw)
        done = [VP.process_image(img, self.proc) for img in images]
        grids = [p.grid_thw for p in done]
        merge = self.proc.merge_size
        n_tok = [p.merged_tokens(merge) for p in done]
        total = sum(n_tok)
        row0 = self.arena.alloc(total)
        if row0 is None:
            self.counters["refused"] += 1
            raise EngineRefused("image arena is full", 503)
        try:
            ids = VP.expand_image_pads(token_ids, self.image_pad_id, grids, merge)
            pos, delta = VP.mrope_positions(ids, self.image_pad_id, grids, merge)
            px = torch.from_numpy(np.concatenate([p.pixel_values for p in done], 0))
            if self.table.is_cuda:
                px = px.pin_memory()
            with self._tower_lock:
                self._encode(px, grids, self.table[self.vocab + row0: self.vocab + row0 + total])
        except Exception:
            self.arena.free(row0, total)
            raise
        # placeholders -> arena rows, in order
        out, r = [], self.vocab + row0
        for t in ids:
            if t == self.image_pad_id:
                out.append(r)
                r += 1
            else:
                out.append(int(t))
        self.counters["images"] += len(images)
        self.counters["patch_rows"] += sum(p.patches for p in done)
        self.counters["image_tokens"] += total
        arena = self.arena
        mm = {"rope_pos": pos, "rope_delta": delta, "release": lambda: arena.free(row0, total),
              "grids": grids, "image_tokens": total}
        return EngineRequest(out, params, mm=mm, **kw)
