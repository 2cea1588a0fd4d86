"""The vision tower on the device: every linear is one launch of the tcgen05 GEMM in its bf16 mode
(bias, GELU and the residual add in the epilogue), every normalisation writes the next GEMM's token
operand directly, attention writes the projection's operand.  Attention is a rotary kernel in place on q / k and a
flash-style mma.sync kernel.  Nine launches per block.

    tower = VisionTowerGPU(cfg, weights, "cuda")
    rows = tower.forward(pixel_values, grids)        # bf16 [L / 4, out_hidden]
    tower.forward(pixel_values, grids, out=buf)      # or into a caller's rows (the engine's image arena)

Parity: the reference's vision executor (`crates/saber-kernels/hip/vision.hip:1-30`,
`crates/saber-exec/src/` vision executor and mrope).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence

import numpy as np
import torch

from ..ops import functional as F
from ..ops import layouts as L
from ..ops import native as N
from .tower import VisionConfig, VisionWeights, attn_blocks, pos_gather_table, rope_tables

EPI_NONE, EPI_GELU_TANH, EPI_GELU_ERF, EPI_RES = 0, 1, 2, 3


class _Lin:
    """A bf16 weight in the GEMM's tile order (rows of 64 values = 128 bytes per k-block)."""

    def __init__(self, w: torch.Tensor, b: torch.Tensor, device):
        n, k = w.shape
        self.N, self.K = n, k
        self.K_pad = L.round_up(k, 64)
        wp = torch.zeros(n, self.K_pad, dtype=torch.bfloat16)
        wp[:, :k] = w.to(torch.bfloat16)
        self.tiles = L.tile_weight_int8(wp.view(torch.int8).reshape(n, self.K_pad * 2)).to(device).contiguous()
        self.N_pad = self.tiles.shape[0] * L.TILE_N
        self.bias = b.float().to(device).contiguous()


class VisionTowerGPU:
    def __init__(self, cfg: VisionConfig, wts: VisionWeights, device="cuda", max_patches: int = 16384):
        self.cfg, self.dev = cfg, torch.device(device)
        d = self.dev
        self.patch = _Lin(wts.patch_w, wts.patch_b, d)
        self.pos_table = wts.pos_table.to(torch.bfloat16).to(d).contiguous()
        self.blocks = []
        for b in wts.blocks:
            self.blocks.append(dict(
                ln1=(b["ln1_w"].float().to(d), b["ln1_b"].float().to(d)), qkv=_Lin(b["qkv_w"], b["qkv_b"], d),
                proj=_Lin(b["proj_w"], b["proj_b"], d), ln2=(b["ln2_w"].float().to(d), b["ln2_b"].float().to(d)),
                fc1=_Lin(b["fc1_w"], b["fc1_b"], d), fc2=_Lin(b["fc2_w"], b["fc2_b"], d)))
        m = wts.merger
        self.m_ln = (m["ln_w"].float().to(d), m["ln_b"].float().to(d))
        self.m_fc1, self.m_fc2 = _Lin(m["fc1_w"], m["fc1_b"], d), _Lin(m["fc2_w"], m["fc2_b"], d)
        self.max_patches = max_patches
        self._cap = 0
        self.launches = 0

    # ------------------------------------------------------------------ buffers sized for L rows
    def _reserve(self, Lr: int) -> None:
        if Lr <= self._cap:
            return
        cfg, d = self.cfg, self.dev
        m_pad = L.padded_rows(Lr)
        kmax = max(L.round_up(cfg.patch_row, 64), L.round_up(cfg.mlp, 64), cfg.width * cfg.merge ** 2)
        # token operands are zero-filled once: rows past the live ones and columns past K stay zero
        self.a_buf = torch.zeros(kmax * 2 // 128 * m_pad * 128, dtype=torch.uint8, device=d)
        self.x = torch.empty(Lr, cfg.width, dtype=torch.bfloat16, device=d)
        self.qkv = torch.empty(Lr, 3 * cfg.width, dtype=torch.bfloat16, device=d)
        self.h = torch.empty(Lr, L.round_up(cfg.mlp, 8), dtype=torch.bfloat16, device=d)
        self.mh = torch.empty((Lr + 3) // 4, cfg.width * cfg.merge ** 2, dtype=torch.bfloat16, device=d)
        self._cap, self._m_pad_cap = Lr, m_pad

    # ------------------------------------------------------------------ launches
    def _rows(self, src: torch.Tensor, M: int, K: int, K_pad: int, m_pad: int, ln=None, group: int = 1) -> None:
        p = N.VisRowsParams()
        p.x, p.x_f32, p.ldx = src.data_ptr(), int(src.dtype == torch.float32), src.stride(0)
        p.ln_w, p.ln_b = (ln[0].data_ptr(), ln[1].data_ptr()) if ln is not None else (None, None)
        p.eps, p.tiled = self.cfg.eps, self.a_buf.data_ptr()
        p.M, p.K, p.K_pad, p.M_pad, p.group = M, K, K_pad, m_pad, group
        N.check(N.lib().saber_vis_rows_launch(C.byref(p), N.stream_handle()), "vis_rows")
        self.launches += 1

    def _gemm(self, lin: _Lin, M: int, m_pad: int, out: torch.Tensor, epi: int = EPI_NONE,
              res: Optional[torch.Tensor] = None, k_pad: Optional[int] = None) -> None:
        sc = F.scratch(self.dev)
        p = N.GemmI8Params()
        p.w, p.w_scale, p.a, p.a_scale = lin.tiles.data_ptr(), None, self.a_buf.data_ptr(), None
        p.out, p.ws, p.counters, p.err = out.data_ptr(), sc.ws.data_ptr(), sc.counters.data_ptr(), sc.err.data_ptr()
        p.M, p.M_pad, p.N, p.N_pad, p.K = M, m_pad, lin.N, lin.N_pad, (k_pad or lin.K_pad) * 2
        p.nt, p.splits, p.w4, p.ldo = L.token_tile(M), 1, 3, out.stride(0)
        p.mtiles = getattr(self, "force_pairs", 0)     # tests set 2 to run the paired-tile path on small shapes
        p.bias, p.epi, p.res = lin.bias.data_ptr(), epi, (res.data_ptr() if res is not None else None)
        assert out.stride(0) % 8 == 0 and (res is None or res.stride(0) == out.stride(0))
        N.check(N.lib().saber_gemm_i8_launch(C.byref(p), 0, N.stream_handle()), "vision gemm")
        self.launches += 1

    # ------------------------------------------------------------------ forward
    def _meta(self, grids) -> dict:
        """Host tables of a grid list on the device: position gather, rotary tables, attention blocks."""
        cfg, d = self.cfg, self.dev
        idx, wt = pos_gather_table(grids, cfg)
        cos, sin = rope_tables(grids, cfg)
        blocks = attn_blocks(grids)
        return dict(idx=torch.from_numpy(idx).to(d), wt=torch.from_numpy(wt).to(d), cos=torch.from_numpy(cos).to(d),
                    sin=torch.from_numpy(sin).to(d), blk=torch.from_numpy(blocks).to(d), n_blocks=int(blocks.shape[0]))

    def _run(self, px: torch.Tensor, Lr: int, meta: dict, out: Optional[torch.Tensor], stop_at_hidden: bool) -> None:
        """The launches of one forward on the current stream (nothing here synchronises)."""
        cfg = self.cfg
        m_pad = L.padded_rows(Lr)
        W = cfg.width
        x, qkv, h = self.x[:Lr], self.qkv[:Lr], self.h[:Lr]
        lib = N.lib()
        self._rows(px, Lr, cfg.patch_row, self.patch.K_pad, m_pad)
        self._gemm(self.patch, Lr, m_pad, x)
        pp = N.VisPosAddParams()
        pp.x, pp.ldx, pp.table, pp.ldt = x.data_ptr(), x.stride(0), self.pos_table.data_ptr(), self.pos_table.stride(0)
        pp.idx, pp.wt, pp.M, pp.K = meta["idx"].data_ptr(), meta["wt"].data_ptr(), Lr, W
        N.check(lib.saber_vis_pos_add_launch(C.byref(pp), N.stream_handle()), "vis_pos_add")
        self.launches += 1
        pa = N.VisAttnParams()
        pa.qkv, pa.ldq = qkv.data_ptr(), qkv.stride(0)
        pa.cos_t, pa.sin_t = meta["cos"].data_ptr(), meta["sin"].data_ptr()
        pa.out_tiled, pa.M_pad, pa.blocks = self.a_buf.data_ptr(), m_pad, meta["blk"].data_ptr()
        pa.heads, pa.width, pa.scale = cfg.heads, W, 1.0 / math.sqrt(cfg.head_dim)
        for b in self.blocks:
            self._rows(x, Lr, W, W, m_pad, ln=b["ln1"])
            self._gemm(b["qkv"], Lr, m_pad, qkv)
            N.check(lib.saber_vis_rope_launch(C.byref(pa), Lr, N.stream_handle()), "vis_rope")
            N.check(lib.saber_vis_attn_launch(C.byref(pa), meta["n_blocks"], N.stream_handle()), "vis_attn")
            self.launches += 2
            self._gemm(b["proj"], Lr, m_pad, x, EPI_RES, res=x)
            self._rows(x, Lr, W, W, m_pad, ln=b["ln2"])
            self._gemm(b["fc1"], Lr, m_pad, h, EPI_GELU_TANH)
            self._rows(h, Lr, b["fc1"].N, b["fc2"].K_pad, m_pad)
            self._gemm(b["fc2"], Lr, m_pad, x, EPI_RES, res=x)
        if stop_at_hidden:
            return
        # merger: four consecutive rows (one 2 x 2 neighbourhood) become one row of 4 * width values
        Lm = Lr // (cfg.merge ** 2)
        mm_pad = L.padded_rows(Lm)
        W4 = W * cfg.merge ** 2
        self._rows(x, Lr, W, W, mm_pad, ln=self.m_ln, group=cfg.merge ** 2)
        mh = self.mh[:Lm]
        self._gemm(self.m_fc1, Lm, mm_pad, mh, EPI_GELU_ERF)
        self._rows(mh, Lm, W4, W4, mm_pad)
        self._gemm(self.m_fc2, Lm, mm_pad, out)

    @torch.no_grad()
    def forward(self, pixel_values: torch.Tensor, grids: Sequence[tuple],
                out: Optional[torch.Tensor] = None, return_hidden: bool = False,
                graph: bool = False) -> torch.Tensor:
        """`graph=True`: the launches of a grid list are captured once into a CUDA graph (static input
        and output buffers, at most `max_graphs` shapes kept) and replayed afterwards."""
        cfg, d = self.cfg, self.dev
        grids = [tuple(g) for g in grids]
        Lr = int(pixel_values.shape[0])
        assert Lr == sum(t * h * w for t, h, w in grids) and Lr % (cfg.merge ** 2) == 0
        if Lr > self.max_patches:
            raise ValueError(f"{Lr} patch rows exceed the tower arena ({self.max_patches})")
        Lm = Lr // (cfg.merge ** 2)
        if out is None and not return_hidden:
            out = torch.empty(Lm, cfg.out_hidden, dtype=torch.bfloat16, device=d)
        assert return_hidden or (out.shape[0] >= Lm and out.dtype == torch.bfloat16)
        if graph and not return_hidden:
            self._replay(pixel_values, grids, Lr, out[:Lm])
        else:
            self._reserve(Lr)
            px = pixel_values.to(d, non_blocking=True).float().contiguous()
            self._run(px, Lr, self._meta(grids), out, return_hidden)
        F.scratch(d).check()
        return self.x[:Lr].clone() if return_hidden else out[:Lm]

    max_graphs = 8

    def _replay(self, pixel_values: torch.Tensor, grids: list, Lr: int, out: torch.Tensor) -> None:
        cfg, d = self.cfg, self.dev
        if not hasattr(self, "_graphs"):
            self._reserve(self.max_patches)          # buffers never move under a captured graph
            self._graphs = {}
            self.px_buf = torch.empty(self.max_patches, cfg.patch_row, dtype=torch.float32, device=d)
            self.out_buf = torch.empty(self.max_patches // cfg.merge ** 2, cfg.out_hidden, dtype=torch.bfloat16, device=d)
        key = tuple(grids)
        px, ob = self.px_buf[:Lr], self.out_buf[:out.shape[0]]
        px.copy_(pixel_values, non_blocking=True)
        ent = self._graphs.get(key)
        if ent is None:
            meta = self._meta(grids)
            self._run(px, Lr, meta, ob, False)       # warm-up outside the capture (function attributes, allocator)
            cur = torch.cuda.current_stream(d)
            side = torch.cuda.Stream(device=d)
            side.wait_stream(cur)
            g = torch.cuda.CUDAGraph()
            # thread-local capture mode: the engine's step loop keeps synchronising its own stream in
            # another thread while an image of a new shape is captured here
            with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                self._run(px, Lr, meta, ob, False)
            cur.wait_stream(side)
            if len(self._graphs) >= self.max_graphs:
                self._graphs.pop(next(iter(self._graphs)))
            ent = self._graphs[key] = (g, meta)
            self.graphs_captured = getattr(self, "graphs_captured", 0) + 1
        ent[0].replay()
        out.copy_(ob, non_blocking=True)
