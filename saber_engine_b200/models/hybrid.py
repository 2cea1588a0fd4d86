"""The hybrid decoder (Gated DeltaNet + gated GQA attention, dense MLP or MoE) as native step
programs on one rank.

`HybridModel` owns the weights, the paged fp8 KV pool, the GDN state slots and the index blob, and
builds one `Bucket` per planned shape: decode buckets (batch x width rows, speculative: rows are
verified and the next block is drafted inside the same program) and prefill buckets (a rung of
rows, rows are committed for good).  A bucket is a fixed launch list (`ops.native.Program`) that is
walked eagerly or captured into a CUDA graph; per-step values travel in the index blob only.

Parity: the per-layer op order of the reference's model graph (`crates/saber-model/src/graph.rs:4525-4577`),
its decode buckets batches x widths and prefill rungs (`models.toml:25-36`), the index tables of
`crates/saber-exec/src/forward.rs:587-860` (slot 0 is the null slot; padding rows carry slot_map -1),
and the drafter-after-commit flow of `crates/saber-engine/src/draft_plan.rs:17-30`.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..ops import functional as F
from ..ops import layouts as L
from ..ops import native as N
from .config import HybridConfig, shard
from .weights import ModelWeights, random_init


@dataclass
class BlobLayout:
    """Offsets (in int32 words) of the per-step index tables inside a bucket's index blob."""
    M: int
    nseq: int
    max_blocks: int
    ids: int = 0
    pos: int = 0
    slot_map: int = 0
    cu_rows: int = 0
    slots: int = 0
    shift: int = 0
    kv_len: int = 0
    seq_uid: int = 0
    step_no: int = 0
    last_rows: int = 0
    temps: int = 0
    next_ids: int = 0          # per row: the token that follows it in its prompt (-1: none), for prompt log-probabilities
    samp: int = 0              # per HEAD row: fp32 {temperature, top_k, top_p, min_p} (temperature 0: keep the greedy pick)
    samp_u: int = 0            # per HEAD row: the uniform number of the draw (fp32)
    block_table: int = 0
    words: int = 0

    @staticmethod
    def make(M: int, nseq: int, max_blocks: int) -> "BlobLayout":
        b = BlobLayout(M, nseq, max_blocks)
        off = 0
        def take(n):
            nonlocal off
            o = off
            off += (n + 3) // 4 * 4          # keep every table 16-byte aligned
            return o
        b.ids = take(M)
        b.pos = take(3 * M)
        b.slot_map = take(M)
        b.cu_rows = take(nseq + 1)
        b.slots = take(nseq)
        b.shift = take(nseq)
        b.kv_len = take(nseq)
        b.seq_uid = take(nseq)
        b.step_no = take(nseq)
        b.last_rows = take(nseq)
        b.temps = take(M)
        b.next_ids = take(M)
        b.samp = take(4 * M)
        b.samp_u = take(M)
        b.block_table = take(nseq * max_blocks)
        b.words = off
        return b

    @property
    def header_words(self) -> int:
        return self.block_table


@dataclass
class Bucket:
    """One planned shape: its program, blob layout, output tensors."""
    kind: str                 # "decode" | "prefill"
    nseq: int
    width: int                # rows per sequence (decode) or rung rows (prefill, nseq sequences packed)
    M: int
    layout: BlobLayout
    program: N.Program
    blob_dev: torch.Tensor    # int32 [words]
    blob_host: torch.Tensor   # pinned int32 [words]
    out_dev: torch.Tensor     # int32: n_commit[nseq] | out_tokens[nseq*W] | drafts[nseq*block] | picks[M]
    out_host: torch.Tensor    # pinned mirror
    captured: bool = False
    n_launches: int = 0
    logits: Optional[torch.Tensor] = None
    keep: list = field(default_factory=list)
    bt_rows: dict = field(default_factory=dict)    # row j -> (blocks_key, n blocks) of the block-table row the device holds
    last_h2d_bytes: int = 0                        # index-table bytes the last step copied to the device
    arenas: list = field(default_factory=list)     # pure activation buffers: written before read in every step
    digests: Optional[torch.Tensor] = None         # int64 [n_layers + 1] stage digests (race_check = "shadow")
    sp: bool = False                               # prefill on several ranks: the sequence-parallel chain (rows owned by ranks)
    seam_dev: Optional[torch.Tensor] = None        # int32 blob: ids [Mh*64] | values [Mh*64] fp32 bits | lse [Mh*2] (seam buckets)
    seam_host: Optional[torch.Tensor] = None       # pinned mirror
    plp_dev: Optional[torch.Tensor] = None         # int32 blob of a prompt-log-probability bucket (every row: candidates, lse, next-token logit)
    plp_host: Optional[torch.Tensor] = None


class HybridModel:
    def __init__(self, cfg: HybridConfig, tp: int = 1, rank: int = 0, device="cuda",
                 max_seqs: int = 8, max_ctx: Optional[int] = None, kv_blocks: Optional[int] = None,
                 max_width: int = 8, weights: Optional[ModelWeights] = None, seed: int = 0,
                 comm=None, oracle_p: float = 0.0, oracle_seed: int = 0, gdn_vs: int = 2,
                 use_drafter: bool = True, race_check: str = "off", gdn_prefill: str = "tc", gdn_fused: Optional[bool] = None,
                 image_rows: int = 0, fuse: bool = True, attn_impl: str = "tc", sp_prefill: Optional[bool] = None,
                 prefill_w8: Optional[bool] = None):
        self.cfg, self.tp, self.rank = cfg, tp, rank
        if race_check not in ("off", "shadow"):
            raise ValueError("race_check must be 'off' or 'shadow'")
        self.gdn_prefill = gdn_prefill      # "rows" (row-by-row recurrence) | "chunked" (64-row chunks, fp32) | "tc" (chunks on the tensor cores)
        self.race_check = race_check        # "shadow": a digest of the residual stream after every layer rides with the result
        self.sh = shard(cfg, tp, rank)
        self.device = torch.device(device)
        self.max_seqs = max_seqs
        self.max_ctx = max_ctx or cfg.max_ctx
        self.max_blocks = (self.max_ctx + cfg.page_tokens - 1) // cfg.page_tokens
        self.max_width = max_width
        self.comm = comm
        self.oracle_p, self.oracle_seed = oracle_p, oracle_seed
        # fused decode step of the DeltaNet layers (conv + recurrence + gated norm + quantisation in one
        # launch): one value slice per head and two alternating conv windows per slot.  Off by default:
        # at 8 sequences x 8 rows the three launches overlap with their neighbours (the light kernels
        # trigger their dependents early) and measured 10.7 ms per step against 11.8 ms fused.
        self.gdn_fused = False if gdn_fused is None else bool(gdn_fused)
        if self.gdn_fused:
            gdn_vs = 1
        self.gdn_vs = gdn_vs
        self.step_timeout_s = 120.0         # host-side deadline of one step (graph capture and first launches included)
        self.use_drafter = use_drafter and cfg.drafter is not None
        self.w = weights if weights is not None else random_init(cfg, tp, rank, self.device, seed)
        self.scratch = F.scratch(self.device)
        # Fused forms of the decode chain (launches that stay resident as a whole grid): the row op
        # after a row-parallel linear rides as that GEMM's row tail, silu * mul + quant runs in the
        # epilogue of the (paired) gate | up linear.  fuse=False keeps one launch per op.
        self.fuse = bool(fuse)
        # "tc": tcgen05 attention, KV pages in the order it multiplies in place; "mma": warp-level MMA kernel, [token][dim] pages
        if attn_impl not in ("tc", "mma"):
            raise ValueError("attn_impl must be 'tc' or 'mma'")
        self.attn_impl = attn_impl
        self._held = None
        # sequence-parallel prefill on several ranks: a row-parallel GEMM sends a row's partial sums to the
        # row's owner only (reduce-scatter), the owner adds, normalises and quantises it and stores the
        # quantised row into every rank's buffer (all-gather), and the next GEMM waits per 128-row tile.
        # Parity: the reference's fused GEMM + all-reduce + add-norm-quant (`crates/saber-kernels/hip/macaq_iu8f.hip:1-12`)
        # is the two-rank, all-reduce form of this chain.
        from ..rules import default_rules
        self.sp_prefill = (tp >= default_rules().doc["prefill"]["sequence_parallel_min_ranks"]) if sp_prefill is None else bool(sp_prefill)
        self._sp, self._sp_rpr, self._ag_site, self._qa_ag, self._qa_src_ptr = False, 0, -1, None, 0
        # Prefill rungs of 256 rows and more multiply with an int8 twin of every 4-bit linear (the tile image
        # the decode kernel widens to, made once): at that many rows a GEMM is bound by the tensor pipe and by
        # shared-memory bandwidth, not by the weight stream, and the widening pass takes a third of the latter.
        # Same integers, same scales, so the outputs are the same bytes; the price is memory (twice the 4-bit
        # weights again), which is what a 180 GB part has.  None: on while free memory covers it.
        self.prefill_w8 = prefill_w8
        self._big_prefill = False
        self.twin_bytes = 0
        if self.fuse and cfg.moe is None:
            for lw in self.w.layers:
                if lw.gate_up is not None:
                    lw.gate_up = F.pair_gate_up(lw.gate_up)
            if self.w.drafter is not None:
                for d in self.w.drafter.layers:
                    d["gate_up"] = F.pair_gate_up(d["gate_up"])
        self.k_scale = self.v_scale = 1.0
        # Image rows: the token table is extended by `image_rows` rows that the vision tower writes; a
        # prompt names them as token ids vocab + r, so the embedding gather of every (captured) prefill
        # program splices them in without a kernel of its own.
        self.image_rows = int(image_rows)
        self.embed_table = self.w.embed
        if self.image_rows > 0:
            ext = torch.zeros(cfg.vocab + self.image_rows, cfg.hidden, dtype=torch.bfloat16, device=self.device)
            ext[:cfg.vocab].copy_(self.w.embed)
            self.embed_table = ext
        dev = self.device
        # ---- paged KV pool (fp8): one tensor per attention layer
        if kv_blocks is None:
            kv_blocks = max_seqs * self.max_blocks + 1
        self.kv_blocks = kv_blocks
        self.kv = {}
        for i in range(cfg.n_layers):
            if cfg.is_attention_layer(i):
                self.kv[i] = torch.zeros(kv_blocks, self.sh.n_kv_heads, 2, cfg.page_tokens, cfg.head_dim,
                                         dtype=torch.uint8, device=dev)
        # the drafter's context-KV store: one page pool per drafter attention layer, addressed by the target's block tables
        self.draft_kv = {}
        if cfg.drafter is not None and use_drafter:
            for li in range(getattr(cfg.drafter, "attn_layers", 0)):
                self.draft_kv[li] = torch.zeros(kv_blocks, cfg.drafter.attn_kv_heads, 2, cfg.page_tokens, cfg.head_dim,
                                                dtype=torch.uint8, device=dev)
        # ---- GDN state slots (slot 0 = null slot)
        self.n_slots = max_seqs + 1
        hv, hk, d = self.sh.gdn_v_heads, self.sh.gdn_k_heads, cfg.gdn_head_dim
        self.gdn_state, self.gdn_hist, self.gdn_stash = {}, {}, {}
        for i in range(cfg.n_layers):
            if not cfg.is_attention_layer(i):
                self.gdn_state[i] = torch.zeros(self.n_slots, hv, d, d, dtype=torch.float32, device=dev)
                self.gdn_hist[i] = F.gdn_hist_alloc(self.n_slots, 3 + max_width, self.sh.gdn_conv_c, dev) if self.gdn_fused \
                    else torch.zeros(self.n_slots, 3 + max_width, self.sh.gdn_conv_c, dtype=torch.bfloat16, device=dev)
                self.gdn_stash[i] = torch.zeros(self.n_slots, max_width, hv, gdn_vs,
                                                F.gdn_stash_stride(gdn_vs), dtype=torch.float32, device=dev)
        self.buckets: dict = {}
        self.stream = torch.cuda.Stream(device=dev)

    # ------------------------------------------------------------------------------ state
    def reset_slot(self, slot: int) -> None:
        """Zero the recurrent state of a slot (a new sequence starts from nothing)."""
        with torch.cuda.stream(self.stream):     # ordered with the programs, which run on this stream
            for i in self.gdn_state:
                self.gdn_state[i][slot].zero_()
                self.gdn_hist[i][slot].zero_()

    def state_bytes(self) -> dict:
        kv = sum(t.numel() for t in self.kv.values())
        gdn = sum(t.numel() * 4 for t in self.gdn_state.values()) + \
            sum(t.numel() * 2 for t in self.gdn_hist.values()) + \
            sum(t.numel() * 4 for t in self.gdn_stash.values())
        return {"weights": self.w.nbytes(), "weights_prefill_int8_twin": self.twin_bytes, "kv_pool": kv, "gdn": gdn}

    # ------------------------------------------------------------------------------ helpers
    def _qa(self, M: int, K: int) -> F.QuantAct:
        return F.QuantAct.alloc(M, K, self.device)

    @staticmethod
    def _fmt(a: Optional[F.QuantAct], w) -> Optional[F.QuantAct]:
        """The activation buffer seen in the byte format the consuming linear multiplies with
        (int8 for integer weights, fp8 e4m3 for MXFP4): same storage, different law."""
        if a is None:
            return None
        if getattr(w, "fp4", 0):          # native FP4 linear: NVFP4 rows + scale atoms in the same storage
            v = a.as_fp4(w.fp4)
            v.had_sign = getattr(w, "had_sign", None)
            return v
        return F.QuantAct(a.q, a.scale, a.M, a.K, fp8=bool(getattr(w, "mx", False)), had_sign=getattr(w, "had_sign", None))

    def _flush(self, prog: N.Program) -> None:
        """Add the GEMM that was held back for a row tail as a plain launch."""
        if self._held is not None:
            p, stages, tag = self._held
            self._held = None
            prog.gemm(p, stages, tag=tag)

    def _gemm(self, prog: N.Program, w: F.QuantWeight, a: F.QuantAct, out: torch.Tensor, tag: str,
              tp_site: int = -1, hold: bool = False) -> None:
        """tp_site >= 0: a row-parallel GEMM whose epilogue pushes its partial sums to every rank.
        hold: the launch is kept back until the next op is known -- an add + RMSNorm + quantise that
        consumes this GEMM's output becomes its row tail (`_add_rms`), anything else adds it as it is."""
        self._flush(prog)
        w = self._twin8(w, a.M)
        a = self._fmt(a, w)
        a, ag_site = self._ag_input(a)
        nt = L.token_tile(a.M)
        # A feature-tile count just over a multiple of the SMs (the vocabulary heads: 594 tiles = 4 x 148 + 2)
        # costs a whole extra round of CTAs for a handful of tiles: those tiles run as a GEMM of their own,
        # split along K over the SMs, while the rest fills whole rounds.
        from ..rules import default_rules
        sms = int(default_rules().doc["device"]["sms"])
        n_tiles = w.N_pad // L.TILE_N
        rem = n_tiles % sms
        if (self.fuse and tp_site < 0 and not hold and ag_site < 0 and not w.fp4 and not w.paired and a.M <= 128
                and n_tiles > sms and 0 < rem <= sms // 16 and out.stride(0) % 8 == 0):
            cut = n_tiles - rem
            head = F.QuantWeight(w.tiles[:cut], w.scale[:cut * L.TILE_N], cut * L.TILE_N, w.K, w.w4, mx=w.mx, had_sign=w.had_sign)
            tail = F.QuantWeight(w.tiles[cut:], w.scale[cut * L.TILE_N:], w.N - cut * L.TILE_N, w.K, w.w4, mx=w.mx, had_sign=w.had_sign)
            prog.gemm(F.gemm_params(head, a, out, self.scratch, splits=1), 0, tag=f"{tag}.whole_rounds")
            ksplit = F.pick_splits(rem, 1, w.K // 128)
            prog.gemm(F.gemm_params(tail, a, out[:, cut * L.TILE_N:], self.scratch, splits=ksplit), 0, tag=f"{tag}.last_tiles")
            return
        hit = self._tuned(w, a)
        if hit is not None and tp_site < 0 and not hold:
            halves = int(hit.get("halves", 1))
        else:
            halves = 2 if (self.fuse and tp_site < 0 and not hold and
                           F.pick_halves(w, w.N_pad // L.TILE_N, (a.M + nt - 1) // nt)) else 1
        splits = 1 if halves == 2 else self.pick_splits(w, a)
        if self._sp and tp_site >= 0:
            splits, halves = 1, 1           # one arrival per feature tile at the row's owner
        p = F.gemm_params(w, a, out, self.scratch, splits=splits, halves=halves)
        if ag_site >= 0:
            self.comm.gemm_ag(p, ag_site)
        if tp_site >= 0 and self.tp > 1:
            if self._sp:
                self.comm.gemm_rs(p, tp_site, self._sp_rpr)
            else:
                self.comm.gemm_tp(p, tp_site)
            self._site_parts[tp_site] = N.lib().saber_gemm_i8_parts(C.byref(p))
        # (a row-parallel GEMM on several ranks keeps its consumer as a launch of its own: as a row tail the
        # consumer's cross-rank waits sit inside the GEMM's grid, measured 9.63 against 8.63 ms per step at 8 ranks)
        from ..rules import default_rules
        if hold and self.fuse and not (tp_site >= 0 and self.tp > default_rules().doc["gemm"]["tails"]["row_tail_max_ranks"]):
            self._held = (p, self.gemm_stages(w, a), tag)
        else:
            prog.gemm(p, self.gemm_stages(w, a), tag=tag)

    def _mlp_in(self, prog: N.Program, w: F.QuantWeight, a: F.QuantAct, gu: torch.Tensor, qa_i: F.QuantAct,
                w_down, K_inter: int, M: int, tag: str) -> None:
        """gate | up linear, silu(gate) * up, per-token quantisation into `qa_i`: one launch when the
        weight is paired and the grid stays resident, else GEMM + row kernel."""
        self._flush(prog)
        w = self._twin8(w, a.M)
        a = self._fmt(a, w)
        a, ag_site = self._ag_input(a)
        splits = self.pick_splits(w, a)
        p = F.gemm_params(w, a, gu, self.scratch, splits=splits)
        if ag_site >= 0:
            self.comm.gemm_ag(p, ag_site)
        qi = self._fmt(qa_i, w_down)
        if self.fuse and w.paired and splits == 1 and not qi.fp8 and not qi.fp4 and qi.had_sign is None and F.gemm_tail_ok(p) \
                and qi.M_pad % p.nt == 0 and qi.M_pad <= 256:
            F.gemm_tail_silu_quant(p, qi, self.scratch)
            prog.gemm(p, self.gemm_stages(w, a), tag=f"{tag}.gate_up+silu_mul_quant")
            return
        prog.gemm(p, self.gemm_stages(w, a), tag=f"{tag}.gate_up")
        rp = F.row_params(M, K_inter, a=gu, qa=qi)
        rp.silu_pair = int(w.paired)
        prog.row(N.ROW_SILU_MUL, rp, tag=f"{tag}.silu_mul_quant")

    def _add_rms(self, prog: N.Program, M: int, tag: str, w, res, qa, delta, tp_site: int = -1, out=None,
                 res_copy=None) -> None:
        """residual += (delta | the all-reduced GEMM output of `tp_site`); norm; int8 quant.  When the
        GEMM that produced `delta` is being held (`_gemm(hold=True)`) and its grid stays resident, the
        op becomes that GEMM's row tail instead of a launch of its own."""
        cfg = self.cfg
        sp = self._sp and tp_site >= 0 and self.tp > 1
        if sp and qa is not None:
            # the quantised rows of the owned rows go to every rank's copy of the all-gather buffer
            g = self._qa_ag
            qa = F.QuantAct(g.q, g.scale, M, cfg.hidden, fp8=qa.fp8, had_sign=qa.had_sign)
        p = F.row_params(M, cfg.hidden, a=delta, res=res, w=w, w_offset=cfg.norm_offset, eps=cfg.eps, qa=qa, out=out)
        if res_copy is not None:
            p.res_copy = res_copy.data_ptr()
        if tp_site >= 0 and self.tp > 1:
            nt = self._site_nt.get(tp_site, L.token_tile(M))
            # a producer that signals per split-K part shows up as that many flags per feature tile
            tiles = L.round_up(cfg.hidden, L.TILE_N) // L.TILE_N * self._site_parts.get(tp_site, 1)
            if sp:
                self.comm.row_sp(p, tp_site, nt, tiles, self._sp_rpr)
                self._ag_site = tp_site if qa is not None else -1
            else:
                self.comm.row_tp(p, tp_site, nt, tiles)
        if self._held is not None:
            gp, stages, gtag = self._held
            if cfg.hidden <= 2 * 16 * 320 and (qa is None or qa.had_sign is None) and F.gemm_tail_ok(gp):
                self._held = None
                F.gemm_tail_row(gp, p, self.scratch)
                prog.gemm(gp, stages, tag=f"{gtag}+{tag}")
                return
            self._flush(prog)
        prog.row(N.ROW_ADD_RMS, p, tag=tag)

    def _twin8(self, w: F.QuantWeight, rows: int) -> F.QuantWeight:
        """The int8 twin of a packed 4-bit weight for the big prefill rungs (or the weight itself)."""
        if not self._big_prefill or rows < 256 or self.prefill_w8 is False or not w.w4 or w.mx or w.fp4:
            return w
        tw = getattr(w, "_twin8", None)
        if tw is None:
            need = w.tiles.numel() * 2
            if self.prefill_w8 is None:
                free, _ = torch.cuda.mem_get_info(self.device)
                if free < need + (12 << 30):          # keep room for the buckets' buffers and the graphs
                    self.prefill_w8 = False
                    return w
            t = w.tiles
            img = torch.empty(*t.shape[:-1], 2 * t.shape[-1], dtype=torch.uint8, device=t.device)
            half = t.shape[-1]
            torch.bitwise_and(t << 4, 0xF0, out=img[..., :half])       # low nibbles: the first half of the int8 image (16 w)
            torch.bitwise_and(t, 0xF0, out=img[..., half:])            # high nibbles: the second half
            tw = F.QuantWeight(img, w.scale, w.N, w.K, False, had_sign=w.had_sign, paired=w.paired)
            w._twin8 = tw
            self.twin_bytes += img.numel()
        return tw

    def _ag_input(self, a: F.QuantAct):
        """Sequence-parallel prefill: the rows the last add-norm quantised live in the all-gather buffer
        (every rank's owners stored theirs); a GEMM that reads them waits for their arrival flags."""
        if self._sp and self._ag_site >= 0 and a.q.data_ptr() == self._qa_src_ptr:
            g = self._qa_ag
            return F.QuantAct(g.q, g.scale, a.M, a.K, fp8=a.fp8, had_sign=a.had_sign), self._ag_site
        return a, -1

    def _tuned(self, w: F.QuantWeight, a: F.QuantAct):
        """The measured variant of this (linear, rows) route from the plan's tune table, or None."""
        table = getattr(self, "tune_table", None)
        return table.lookup("gemm_i8", N=w.N_pad, K=w.K, M=a.M, w4=w.fmt_code) if table is not None else None

    def pick_splits(self, w: F.QuantWeight, a: F.QuantAct) -> int:
        table = getattr(self, "tune_table", None)
        if table is not None:
            hit = table.lookup("gemm_i8", N=w.N_pad, K=w.K, M=a.M, w4=w.fmt_code)
            if hit is not None and int(hit.get("halves", 1)) != 2:
                return int(hit.get("splits", 1))
        nt = L.token_tile(a.M)
        return F.pick_splits(w.N_pad // L.TILE_N, (a.M + nt - 1) // nt, w.K // (256 if w.fp4 else 128))

    def gemm_stages(self, w: F.QuantWeight, a: F.QuantAct) -> int:
        table = getattr(self, "tune_table", None)
        if table is not None:
            hit = table.lookup("gemm_i8", N=w.N_pad, K=w.K, M=a.M, w4=w.fmt_code)
            if hit is not None:
                return int(hit.get("stages", 0))
        return 0

    def attn_splits(self, nseq: int, width: int = 16) -> int:
        """KV splits of the decode attention: fill the GPU once (the `decode_splits` law of the launch
        rules, per attention kernel)."""
        from ..rules import default_rules
        if self.attn_impl == "tc" and getattr(self, "tune_table", None) is not None:
            from ..plan.tune_attn import lookup
            hit = lookup(self.tune_table, nseq, width, min(self.max_ctx, getattr(self, "attn_ctx_hint", 4096)),
                         self.sh.n_q_heads, self.sh.n_kv_heads)
            if hit is not None:
                return hit
        return default_rules().attn_decode_splits(self.attn_impl, nseq, self.sh.n_kv_heads,
                                                  self.sh.n_q_heads // self.sh.n_kv_heads, width)

    def tap_layers(self) -> list:
        n = self.cfg.drafter.n_taps if self.cfg.drafter else 0
        L_ = self.cfg.n_layers
        return sorted({min(L_ - 1, max(1, round((k + 1) * L_ / (n + 1)))) for k in range(n)}) if n else []

    # ------------------------------------------------------------------------------ build
    def build_bucket(self, kind: str, nseq: int, width: int, capture: bool = True, seam: bool = False,
                     plp: bool = False) -> Bucket:
        """kind='decode': nseq sequences x width rows.  kind='prefill': up to nseq sequences packed in
        `width` rows in total (ragged through cu_rows), rows committed."""
        # seam = True: the program also leaves the 64 best logits of every head row (ids, values,
        # log-sum-exp) for the host sampler; a bucket of its own so that greedy steps do not pay for it
        # plp = True (prefill only): the head also runs over EVERY row and leaves, per row, the candidate
        # row and the logit of the token that follows it in the prompt (prompt log-probabilities)
        key = (kind, nseq, width, "seam") if seam else (kind, nseq, width)
        if plp:
            if kind != "prefill":
                raise ValueError("prompt log-probabilities: prefill buckets only")
            key = key + ("plp",)
        self._bucket_key, self._want_seam, self._want_plp = key, seam, plp
        if key in self.buckets:
            return self.buckets[key]
        cfg, sh, dev = self.cfg, self.sh, self.device
        decode = kind == "decode"
        M = nseq * width if decode else width
        Mh = M if decode else nseq                      # rows that reach the head
        H, D, d = cfg.hidden, cfg.head_dim, cfg.gdn_head_dim
        lay = BlobLayout.make(M, nseq, self.max_blocks)
        blob = torch.zeros(lay.words, dtype=torch.int32, device=dev)
        blob_host = torch.zeros(lay.words, dtype=torch.int32).pin_memory()
        base = blob.data_ptr()
        at = lambda off: base + 4 * off                 # noqa: E731  device address of a table
        prog = N.Program(f"{kind}-b{nseq}-w{width}")
        self._lay_at = (lay, at, blob)                  # the bucket's index tables, for builders further down
        self._site_nt = {}                              # TP site -> row-tile height its producer signals with
        self._site_parts = {}                           # TP site -> flags per feature tile (split-K parts)
        bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)   # noqa: E731
        f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)   # noqa: E731
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)     # noqa: E731

        h, delta = bf(M, H), bf(M, H)
        qa_h = self._qa(M, H)
        self._sp = bool(not decode and self.tp > 1 and self.sp_prefill and cfg.moe is None and not plp
                        and M % (128 * self.tp) == 0 and M <= min(self.comm.layout.rows_max, 64 * 128)
                        and getattr(cfg, "weight_format", "iu8") == "iu8"
                        and getattr(self.w.layers[0].mixer_in, "had_sign", None) is None
                        and not self.draft_kv)      # (the context-KV store wants the tap rows of every position on every rank)
        self._sp_rpr, self._ag_site, self._qa_src_ptr = M // self.tp, -1, qa_h.q.data_ptr()
        self._qa_ag = self.comm.heap_qact(M, H) if self._sp else None
        sp_used = self._sp
        self._big_prefill = bool(not decode and M >= 256 and cfg.moe is None)
        ld_in = (max(sh.qkv_n, sh.gdn_in_n) + 7) // 8 * 8
        buf_in = bf(M, ld_in)
        conv_out, gdn_o = f32(M, sh.gdn_conv_c), f32(M, sh.gdn_out_k)
        qa_gdn = self._qa(M, sh.gdn_out_k)
        q_rot, attn_out = bf(M, sh.n_q_heads, D), bf(M, sh.n_q_heads, D)
        qa_attn = self._qa(M, sh.o_k)
        taps = self.tap_layers() if self.use_drafter else []
        tap_buf = bf(max(1, len(taps)), M, H)
        splits = self.attn_splits(nseq, width) if decode else 1
        part_o = f32(nseq, sh.n_q_heads, splits, 16, D) if splits > 1 else None
        part_ml = f32(nseq, sh.n_q_heads, splits, 16, 2) if splits > 1 else None
        if cfg.moe is None:
            gu = bf(M, 2 * sh.ffn_inter)
            qa_i = self._qa(M, sh.ffn_inter)
        keep = [blob, h, delta, qa_h, buf_in, conv_out, gdn_o, qa_gdn, q_rot, attn_out, qa_attn,
                tap_buf, part_o, part_ml]

        def row(mode, Mr, K, tag, **kw):
            self._flush(prog)
            prog.row(mode, F.row_params(Mr, K, **kw), tag=tag)

        digests = None
        if self.race_check == "shadow":
            digests = torch.zeros(cfg.n_layers + 1, dtype=torch.int64, device=dev)
            prog.digest_clear(digests, cfg.n_layers + 1, tag="digest.clear")
        prog.embed(self.embed_table, at(lay.ids), h, M, H, 0, cfg.vocab + self.image_rows, H, tag="embed")
        first = True
        chunk_scratch = None
        step_scratch = None
        ar_site = 0
        pending = -1          # site of the TP GEMM whose pushed output the next add-norm consumes
        for i, lw in enumerate(self.w.layers):
            t = f"L{i}"
            # (the drafter's tap of this layer = the residual stream after this add: a second store of the row op)
            self._add_rms(prog, M, f"{t}.in_norm", lw.in_norm, h, self._fmt(qa_h, lw.mixer_in), None if first else delta, pending,
                          res_copy=tap_buf[taps.index(i)] if (i in taps and not first) else None)
            if i in taps and first:
                prog.copy(tap_buf[taps.index(i)], h, tag=f"{t}.tap")
            first = False
            if lw.kind == "gdn":
                n_q = n_k = sh.gdn_k_heads * d
                C_ = sh.gdn_conv_c
                self._gemm(prog, lw.mixer_in, qa_h, buf_in, f"{t}.gdn.in_proj")
                ba = buf_in[:, C_ + sh.gdn_out_k:]
                qo = self._fmt(qa_gdn, lw.mixer_out)
                if self.gdn_fused and decode and width <= 16 and qo.had_sign is None:
                    if step_scratch is None:
                        step_scratch = F.GdnStepScratch(M, sh.gdn_v_heads, nseq, dev)
                        keep.append(step_scratch)
                        qa_gdn.q.zero_()          # rows past M are never written by the fused step
                        qa_gdn.scale.zero_()
                        torch.cuda.current_stream().synchronize()
                    self._flush(prog)
                    gp_ = F.gdn_step_params(buf_in, buf_in[:, C_:], ba, lw.conv_w, lw.A_log, lw.dt_bias, lw.gdn_norm,
                                            self.gdn_hist[i], self.gdn_state[i], self.gdn_stash[i], blob, blob, blob,
                                            step_scratch, qo, n_q, n_k, sh.gdn_v_heads, sh.gdn_k_heads, width,
                                            eps=cfg.eps, ldx=ld_in, ldz=ld_in, ldba=ld_in)
                    gp_.cu_rows, gp_.slots, gp_.shift = at(lay.cu_rows), at(lay.slots), at(lay.shift)
                    prog.gdn_step(gp_, nseq, tag=f"{t}.gdn.step")
                else:
                    cp = F.gdn_conv_params(buf_in, lw.conv_w, self.gdn_hist[i], blob, blob, blob, conv_out,
                                           n_q, n_k, commit=not decode, dual=self.gdn_fused)
                    cp.cu_rows, cp.slots, cp.shift = at(lay.cu_rows), at(lay.slots), at(lay.shift)
                    prog.gdn_conv(cp, nseq, tag=f"{t}.gdn.conv")
                    rp = F.gdn_rec_params(conv_out, ba, lw.A_log, lw.dt_bias, self.gdn_state[i],
                                          self.gdn_stash[i], blob, blob, blob, gdn_o, n_q, n_k,
                                          sh.gdn_v_heads, sh.gdn_k_heads, commit=not decode, ldba=ld_in,
                                          prefill_rows=(not decode and width >= 32),
                                          chunk_impl=int(self.gdn_prefill == "tc"))
                    rp.cu_rows, rp.slots, rp.shift = at(lay.cu_rows), at(lay.slots), at(lay.shift)
                    if not decode and width >= 64 and self.gdn_prefill in ("chunked", "tc"):
                        # prefill: the chunked (64-row) form; one scratch shared by every layer of the bucket
                        if chunk_scratch is None:
                            chunk_scratch = F.gdn_chunk_scratch(M, nseq, sh.gdn_v_heads, dev)
                            keep.append(chunk_scratch)
                        prog.gdn_chunk(rp, nseq, M, chunk_scratch, tag=f"{t}.gdn.rec")
                    else:
                        prog.gdn_rec(rp, nseq, self.gdn_vs, tag=f"{t}.gdn.rec")
                    row(N.ROW_GDN_NORM, M, sh.gdn_out_k, f"{t}.gdn.norm_quant", a_f32=gdn_o,
                        b=buf_in[:, C_:], w=lw.gdn_norm, eps=cfg.eps, qa=qo, ldb=ld_in)
                self._gemm(prog, lw.mixer_out, qa_gdn, delta, f"{t}.gdn.out_proj", tp_site=ar_site, hold=True)
            else:
                nq, nkv = sh.n_q_heads, sh.n_kv_heads
                gate = 2 if cfg.attn_out_gate else 1
                self._gemm(prog, lw.mixer_in, qa_h, buf_in, f"{t}.attn.qkv")
                k_off = nq * D * gate
                rk = F.rope_kv_params(buf_in, q_rot, lw.q_norm, lw.k_norm, blob, blob, self.kv[i], nq, nkv,
                                      0, k_off, k_off + nkv * D, rot_dim=cfg.rot_dim,
                                      sections=cfg.mrope_sections, theta=cfg.rope_theta, eps=cfg.eps,
                                      w_offset=cfg.norm_offset, k_scale=self.k_scale, v_scale=self.v_scale,
                                      page_layout=int(self.attn_impl == "tc"))
                rk.pos, rk.slot_map, rk.ld = at(lay.pos), at(lay.slot_map), ld_in
                prog.rope(rk, tag=f"{t}.attn.rope_kv")
                q_tiles = (width + 15) // 16
                ap = F.attn_params(q_rot, self.kv[i], blob.view(1, -1), blob, blob[:nseq], attn_out, part_o,
                                   part_ml, nkv, splits, q_tiles, self.k_scale, self.v_scale)
                ap.block_table, ap.cu_q, ap.kv_len = at(lay.block_table), at(lay.cu_rows), at(lay.kv_len)
                ap.max_blocks, ap.nseq = self.max_blocks, nseq
                ap.err = self.scratch.err.data_ptr()
                ap.pack_rows = width if (decode and q_tiles == 1) else 0
                ap.impl = int(self.attn_impl == "tc")
                prog.attn(ap, tag=f"{t}.attn.core")
                ao = attn_out.view(M, nq * D)
                if cfg.attn_out_gate:
                    row(N.ROW_GATE_SIG, M, nq * D, f"{t}.attn.gate_quant", a=ao, b=buf_in[:, nq * D:],
                        qa=self._fmt(qa_attn, lw.mixer_out), ldb=ld_in)
                else:
                    row(N.ROW_PLAIN, M, nq * D, f"{t}.attn.quant", a=ao, qa=self._fmt(qa_attn, lw.mixer_out))
                self._gemm(prog, lw.mixer_out, qa_attn, delta, f"{t}.attn.o_proj", tp_site=ar_site, hold=True)
            pending, ar_site = (ar_site, ar_site + 1) if self.tp > 1 else (-1, ar_site)
            self._add_rms(prog, M, f"{t}.post_norm", lw.post_norm, h, self._fmt(qa_h, lw.gate_up), delta, pending)
            if cfg.moe is None:
                self._mlp_in(prog, lw.gate_up, qa_h, gu, qa_i, lw.down, sh.ffn_inter, M, f"{t}.mlp")
                self._gemm(prog, lw.down, qa_i, delta, f"{t}.mlp.down", tp_site=ar_site, hold=True)
            else:
                from .moe_block import add_moe_block
                self._flush(prog)
                self._site_nt[ar_site] = add_moe_block(self, prog, lw, qa_h, h, delta, M, t, keep, tp_site=ar_site)
            pending, ar_site = (ar_site, ar_site + 1) if self.tp > 1 else (-1, ar_site)
            if digests is not None:     # what the layer left in the residual stream and in its MLP output
                self._flush(prog)
                prog.digest(h, M * H * 2, digests.data_ptr() + 8 * i, tag=f"{t}.digest")
        self._build_head(prog, kind, nseq, width, M, Mh, lay, at, h, delta, qa_h, tap_buf, taps, keep,
                         ar_site, pending)
        arenas = [h, delta, buf_in, conv_out, gdn_o, q_rot, attn_out, tap_buf, part_o, part_ml,
                  qa_h.q, qa_h.scale, qa_gdn.q, qa_gdn.scale, qa_attn.q, qa_attn.scale]
        if cfg.moe is None:
            keep += [gu, qa_i]
            arenas += [gu, qa_i.q, qa_i.scale]
        keep.append(digests)
        b = self._finish_bucket(prog, kind, nseq, width, M, lay, blob, blob_host, keep, capture)
        b.arenas = [a for a in arenas if a is not None]
        b.digests = digests
        b.sp = sp_used
        return b

    def _allreduce(self, prog: N.Program, buf: torch.Tensor, n_elems: int, site: int, tag: str) -> int:
        """Row-parallel partial sums -> full sums on every rank (no-op at TP=1)."""
        if self.tp == 1:
            return site
        prog.allreduce(self.comm.allreduce_params(buf, buf, n_elems, site), tag=tag)
        return site + 1

    def _build_head(self, prog, kind, nseq, width, M, Mh, lay, at, h, delta, qa_h, tap_buf, taps, keep,
                    ar_site, pending=-1) -> None:
        cfg, sh, dev = self.cfg, self.sh, self.device
        H = cfg.hidden
        decode = kind == "decode"
        W = width if decode else 1
        block = cfg.drafter.block if self.use_drafter else 0
        # outputs: n_commit[nseq] | out_tokens[nseq * W] | drafts[nseq * block] | picks[Mh]
        n_out = nseq + nseq * W + nseq * max(block, 1) + Mh
        out = torch.zeros(n_out, dtype=torch.int32, device=dev)
        o_commit, o_tokens = out[:nseq], out[nseq:nseq + nseq * W]
        o_drafts = out[nseq + nseq * W: nseq + nseq * W + nseq * max(block, 1)]
        o_picks = out[nseq + nseq * W + nseq * max(block, 1):]
        accept_row = torch.zeros(nseq, dtype=torch.int32, device=dev)
        bonus = torch.zeros(nseq, dtype=torch.int32, device=dev)
        pick_val = torch.zeros(Mh, dtype=torch.float32, device=dev)
        logits = torch.zeros(Mh, (sh.vocab + 7) // 8 * 8, dtype=torch.bfloat16, device=dev)
        self._out_views = None
        if decode:
            self._add_rms(prog, M, "final_norm", self.w.final_norm, h, self._fmt(qa_h, self.w.lm_head), delta, pending)
            qa_head = qa_h
        else:
            normed = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
            last = torch.zeros(nseq, H, dtype=torch.bfloat16, device=dev)
            self._add_rms(prog, M, "final_norm", self.w.final_norm, h, None, delta, pending, out=normed)
            self._flush(prog)
            if self._sp:
                # a row's owner holds its normed values: every rank gathers the last rows it owns (zeros for the
                # others) and the sum over ranks puts every last row on every rank
                r0 = self.rank * self._sp_rpr
                prog.embed(normed[r0:], at(lay.last_rows), last, nseq, H, r0, self._sp_rpr, H, tag="gather_last_rows")
                ar_site = self._allreduce(prog, last, nseq * H, ar_site, "last_rows.allgather")
            else:
                prog.embed(normed, at(lay.last_rows), last, nseq, H, 0, M, H, tag="gather_last_rows")
            qa_head = self._qa(nseq, H)
            prog.row(N.ROW_PLAIN, F.row_params(nseq, H, a=last, qa=self._fmt(qa_head, self.w.lm_head)), tag="head_quant")
            keep += [normed, last, qa_head]
        self._gemm(prog, self.w.lm_head, qa_head, logits, "lm_head")
        prog.argmax(logits, Mh, logits.stride(0), sh.vocab, sh.vocab_first, o_picks, pick_val, tag="argmax")
        if self.tp > 1:
            pm = self.comm.pick_merge_params(o_picks, pick_val, Mh, ar_site)
            prog.pick_merge(pm, tag="pick_merge")
            ar_site += 1
        seam_dev = None
        if self._want_seam:
            # one int32 blob so that the read-back is one copy: ids | values (fp32 bits) | lse pairs
            seam_dev = torch.zeros(Mh * (2 * N.SEAM_K + 2), dtype=torch.int32, device=dev)
            s_ids = seam_dev[:Mh * N.SEAM_K]
            s_vals = seam_dev[Mh * N.SEAM_K: 2 * Mh * N.SEAM_K].view(torch.float32)
            s_lse = seam_dev[2 * Mh * N.SEAM_K:].view(torch.float32)
            prog.seam(logits, Mh, logits.stride(0), sh.vocab, sh.vocab_first, None, s_ids, s_vals, s_lse, tag="topk_seam")
            if self.tp > 1:
                # vocabulary-sharded ranks swap their candidates through the symmetric heap and merge them
                # on the device: every rank then holds the same global best 64 and log-sum-exps
                prog.seam_merge(self.comm.seam_merge_params(s_ids, s_vals, s_lse, Mh, ar_site), tag="seam_merge")
                ar_site += 1
            # device draw for sampled rows: the picks that verify / accept and the drafter see are the
            # sampled tokens (the host repeats the draw from the same candidates and uniforms)
            prog.sample_seam(s_ids, s_vals, at(lay.samp), at(lay.samp_u), o_picks, Mh, tag="sample_seam")
            keep += [seam_dev]
        plp_dev = None
        if self._want_plp:
            K = N.SEAM_K
            qa_all = self._qa(M, H)
            logits_all = torch.zeros(M, (sh.vocab + 7) // 8 * 8, dtype=torch.bfloat16, device=dev)
            # ids [M*K] | values [M*K] | lse [M*2] | logit of the next prompt token [M]
            plp_dev = torch.zeros(M * (2 * K + 3), dtype=torch.int32, device=dev)
            prog.row(N.ROW_PLAIN, F.row_params(M, H, a=normed, qa=self._fmt(qa_all, self.w.lm_head)), tag="plp.head_quant")
            self._gemm(prog, self.w.lm_head, qa_all, logits_all, "plp.lm_head")
            prog.seam(logits_all, M, logits_all.stride(0), sh.vocab, sh.vocab_first, None, plp_dev[:M * K],
                      plp_dev[M * K: 2 * M * K].view(torch.float32), plp_dev[2 * M * K: 2 * M * K + 2 * M].view(torch.float32),
                      tag="plp.topk_seam")
            nxt = plp_dev[2 * M * K + 2 * M:].view(torch.float32)
            prog.logit_gather(logits_all, M, logits_all.stride(0), sh.vocab, sh.vocab_first, at(lay.next_ids), nxt,
                              tag="plp.logit_gather")
            if self.tp > 1:
                # vocabulary shards: the candidates of every row are merged across the ranks on the device, and the
                # successor's logit (minus infinity on the ranks that do not hold its column) by the pick merge
                prog.seam_merge(self.comm.seam_merge_params(plp_dev[:M * K], plp_dev[M * K: 2 * M * K].view(torch.float32),
                                                            plp_dev[2 * M * K: 2 * M * K + 2 * M].view(torch.float32), M, ar_site),
                                tag="plp.seam_merge")
                ar_site += 1
                nxt_ids = torch.zeros(M, dtype=torch.int32, device=dev)
                prog.pick_merge(self.comm.pick_merge_params(nxt_ids, nxt, M, ar_site), tag="plp.next_logit_merge")
                ar_site += 1
                keep.append(nxt_ids)
            keep += [qa_all, logits_all, plp_dev]
            self._plp_logits = logits_all
        if decode:
            vp = N.VerifyParams()
            vp.draft, vp.target, vp.cu_rows = at(lay.ids), o_picks.data_ptr(), at(lay.cu_rows)
            vp.seq_uid, vp.step_no = at(lay.seq_uid), at(lay.step_no)
            vp.n_commit, vp.out_tokens = o_commit.data_ptr(), o_tokens.data_ptr()
            vp.accept_row, vp.bonus = accept_row.data_ptr(), bonus.data_ptr()
            vp.nseq, vp.max_w, vp.oracle_p, vp.seed = nseq, W, self.oracle_p, self.oracle_seed
            prog.verify(vp, tag="verify_accept")
            acc_ptr, bonus_ptr = accept_row.data_ptr(), bonus.data_ptr()
        else:
            acc_ptr, bonus_ptr = at(lay.last_rows), o_picks.data_ptr()
        keep += [out, accept_row, bonus, pick_val, logits]
        self._last_head = dict(out=out, logits=logits, W=W, block=block, Mh=Mh, seam=seam_dev, plp=plp_dev)
        if self.use_drafter:
            ar_site = self._build_drafter(prog, nseq, M, tap_buf, taps, acc_ptr, bonus_ptr, o_drafts, keep, ar_site)
        self._sp = False
        self._big_prefill = False
        if self.tp > 1:
            prog.advance(self.comm.seq_base, ar_site, tag="comm_advance")

    def _build_drafter(self, prog, nseq, M, tap_buf, taps, acc_ptr, bonus_ptr, o_drafts, keep, ar_site: int = 0) -> int:
        """Block drafter: taps of the last committed row -> aux projection -> + token and position
        embeddings -> MLP layers over the block rows -> head -> `block` draft tokens per sequence."""
        cfg, dc, dw, dev = self.cfg, self.cfg.drafter, self.w.drafter, self.device
        H, Hd, B = cfg.hidden, dc.hidden, dc.block
        assert Hd == H, "the drafter shares the target's token embedding"
        nt = len(taps)
        cat = torch.zeros(nseq, dc.n_taps * H, dtype=torch.bfloat16, device=dev)
        for j in range(nt):
            if self._sp:      # tap rows live on their owners: owned rows or zeros, summed over the ranks below
                r0 = self.rank * self._sp_rpr
                prog.embed(tap_buf[j][r0:], acc_ptr, cat[:, j * H:], nseq, H, r0, self._sp_rpr, dc.n_taps * H, tag=f"draft.tap{j}")
            else:
                prog.embed(tap_buf[j], acc_ptr, cat[:, j * H:], nseq, H, 0, M, dc.n_taps * H, tag=f"draft.tap{j}")
        if self._sp and nt:
            ar_site = self._allreduce(prog, cat, nseq * dc.n_taps * H, ar_site, "draft.taps.allgather")
        qa_cat = self._qa(nseq, dc.n_taps * H)
        prog.row(N.ROW_PLAIN, F.row_params(nseq, dc.n_taps * H, a=cat, qa=self._fmt(qa_cat, dw.aux_fc)), tag="draft.tap_quant")
        ctx = torch.zeros(nseq, Hd, dtype=torch.bfloat16, device=dev)
        self._gemm(prog, dw.aux_fc, qa_cat, ctx, "draft.aux_fc")
        tok = torch.zeros(nseq, Hd, dtype=torch.bfloat16, device=dev)
        prog.embed(self.w.embed, bonus_ptr, tok, nseq, H, 0, cfg.vocab, H, tag="draft.tok_embed")
        R = nseq * B
        x = torch.zeros(R, Hd, dtype=torch.bfloat16, device=dev)
        dd = torch.zeros(R, Hd, dtype=torch.bfloat16, device=dev)
        prog.expand(ctx, tok, dw.pos_emb, x, nseq, B, Hd, tag="draft.expand")
        qa_x, qa_di = self._qa(R, Hd), self._qa(R, dc.inter)
        gu = torch.zeros(R, 2 * dc.inter, dtype=torch.bfloat16, device=dev)
        assert Hd == cfg.hidden
        # ---- attention layers: context K | V of this step's rows (from the last tap), then the block rows
        n_attn = len(self.draft_kv)
        if n_attn:
            D, nqd, nkvd = cfg.head_dim, dc.attn_q_heads, dc.attn_kv_heads
            lay_, at_, blob_ = self._lay_at
            tc = int(self.attn_impl == "tc")
            qa_tap = self._qa(M, H)
            kvbuf = torch.zeros(M, 2 * nkvd * D, dtype=torch.bfloat16, device=dev)
            dummy_q = torch.zeros(1, dtype=torch.bfloat16, device=dev)
            prog.row(N.ROW_PLAIN, F.row_params(M, H, a=tap_buf[nt - 1], qa=self._fmt(qa_tap, dw.layers[0]["attn"]["kv_ctx"])), tag="draft.ctx.tap_quant")
            # index tables of the block rows: positions, KV slots, and the length their attention sees
            idx = torch.zeros(3 * R + R + nseq, dtype=torch.int32, device=dev)
            pos_d, slot_d, kvlen_d = idx[:3 * R], idx[3 * R: 4 * R], idx[4 * R:]
            cu_d = torch.arange(0, R + 1, B, dtype=torch.int32, device=dev)
            ip = N.DraftIndexParams()
            ip.pos, ip.cu_rows, ip.kv_len, ip.acc_row = at_(lay_.pos), at_(lay_.cu_rows), at_(lay_.kv_len), acc_ptr
            ip.block_table, ip.pos_out, ip.slot_out, ip.kv_len_out = at_(lay_.block_table), pos_d.data_ptr(), slot_d.data_ptr(), kvlen_d.data_ptr()
            ip.M, ip.nseq, ip.block, ip.max_blocks, ip.page_tokens = M, nseq, B, self.max_blocks, cfg.page_tokens
            prog.draft_index(ip, tag="draft.block_index")
            qkvbuf = torch.zeros(R, (nqd + 2 * nkvd) * D, dtype=torch.bfloat16, device=dev)
            q_rot_d = torch.zeros(R, nqd, D, dtype=torch.bfloat16, device=dev)
            attn_d = torch.zeros(R, nqd, D, dtype=torch.bfloat16, device=dev)
            qa_ad = self._qa(R, nqd * D)
            da = torch.zeros(R, Hd, dtype=torch.bfloat16, device=dev)
            keep += [qa_tap, kvbuf, dummy_q, idx, cu_d, qkvbuf, q_rot_d, attn_d, qa_ad, da]
        for li, lw in enumerate(dw.layers):
            prev = None if li == 0 else dd
            if li < n_attn:
                aw = lw["attn"]
                # context K | V of the step's rows: projected from the target's tap row, normed, rotated, appended
                self._gemm(prog, aw["kv_ctx"], qa_tap, kvbuf, f"draft.L{li}.attn.kv_ctx")
                rk = F.rope_kv_params(kvbuf, dummy_q, aw["q_norm"], aw["k_norm"], blob_, blob_, self.draft_kv[li], 0, nkvd,
                                      0, 0, nkvd * D, rot_dim=cfg.rot_dim, sections=cfg.mrope_sections, theta=cfg.rope_theta,
                                      eps=cfg.eps, w_offset=cfg.norm_offset, k_scale=self.k_scale, v_scale=self.v_scale, page_layout=tc)
                rk.pos, rk.slot_map, rk.ld = at_(lay_.pos), at_(lay_.slot_map), kvbuf.stride(0)
                prog.rope(rk, tag=f"draft.L{li}.attn.ctx_kv_append")
                # the block rows: q | k | v from the drafter's own stream, appended behind the context, causal attention
                self._add_rms(prog, R, f"draft.L{li}.attn.norm", aw["norm"], x, self._fmt(qa_x, aw["qkv"]), prev)
                self._gemm(prog, aw["qkv"], qa_x, qkvbuf, f"draft.L{li}.attn.qkv")
                rb = F.rope_kv_params(qkvbuf, q_rot_d, aw["q_norm"], aw["k_norm"], pos_d, slot_d, self.draft_kv[li], nqd, nkvd,
                                      0, nqd * D, (nqd + nkvd) * D, rot_dim=cfg.rot_dim, sections=cfg.mrope_sections,
                                      theta=cfg.rope_theta, eps=cfg.eps, w_offset=cfg.norm_offset, k_scale=self.k_scale,
                                      v_scale=self.v_scale, page_layout=tc)
                prog.rope(rb, tag=f"draft.L{li}.attn.rope_kv")
                ap = F.attn_params(q_rot_d, self.draft_kv[li], blob_.view(1, -1), cu_d, kvlen_d, attn_d, None, None, nkvd, 1, 1,
                                   self.k_scale, self.v_scale, window=(dc.attn_window if tc else 0))
                ap.block_table, ap.max_blocks, ap.nseq = at_(lay_.block_table), self.max_blocks, nseq
                ap.err = self.scratch.err.data_ptr()
                ap.pack_rows, ap.impl = B, tc
                prog.attn(ap, tag=f"draft.L{li}.attn.core")
                self._flush(prog)
                prog.row(N.ROW_PLAIN, F.row_params(R, nqd * D, a=attn_d.view(R, nqd * D), qa=self._fmt(qa_ad, aw["o_proj"])),
                         tag=f"draft.L{li}.attn.quant")
                self._gemm(prog, aw["o_proj"], qa_ad, da, f"draft.L{li}.attn.o_proj", hold=True)
                prev = da
            self._add_rms(prog, R, f"draft.L{li}.norm", lw["norm"], x, self._fmt(qa_x, lw["gate_up"]), prev)
            self._mlp_in(prog, lw["gate_up"], qa_x, gu, qa_di, lw["down"], dc.inter, R, f"draft.L{li}")
            self._gemm(prog, lw["down"], qa_di, dd, f"draft.L{li}.down", hold=True)
        self._add_rms(prog, R, "draft.final_norm", dw.final_norm, x, self._fmt(qa_x, dw.head), dd if dw.layers else None)
        dlogits = torch.zeros(R, (cfg.vocab + 7) // 8 * 8, dtype=torch.bfloat16, device=dev)
        self._gemm(prog, dw.head, qa_x, dlogits, "draft.head")
        prog.argmax(dlogits, R, dlogits.stride(0), cfg.vocab, 0, o_drafts, None, tag="draft.argmax")
        keep += [cat, qa_cat, ctx, tok, x, dd, qa_x, qa_di, gu, dlogits]
        return ar_site

    def _finish_bucket(self, prog, kind, nseq, width, M, lay, blob, blob_host, keep, capture) -> Bucket:
        self._flush(prog)
        if self.fuse:
            prog.link_prefetch()
        head = self._last_head
        out = head["out"]
        out_host = torch.zeros(out.numel(), dtype=torch.int32).pin_memory()
        prog.keep(*[k for k in keep if k is not None], self.w)
        b = Bucket(kind, nseq, width, M, lay, prog, blob, blob_host, out, out_host,
                   n_launches=prog.declared_launches, logits=head["logits"], keep=keep)
        b.W, b.block, b.Mh = head["W"], head["block"], head["Mh"]
        b.seam_dev = head.get("seam")
        b.plp_dev = head.get("plp")
        b.plp_logits = getattr(self, "_plp_logits", None) if b.plp_dev is not None else None
        b.plp_host = torch.zeros(b.plp_dev.numel(), dtype=torch.int32).pin_memory() if b.plp_dev is not None else None
        b.seam_host = torch.zeros(b.seam_dev.numel(), dtype=torch.int32).pin_memory() if b.seam_dev is not None else None
        if capture:
            # one eager walk first: sets function attributes and warms lazy module loading
            with torch.cuda.stream(self.stream):
                prog.run(self.stream)
                self.stream.synchronize()
                self.scratch.check()
                prog.capture(self.stream)
            self.stream.synchronize()
            b.captured = True
        self.buckets[self._bucket_key] = b
        return b


@dataclass
class SeqStep:
    """What one sequence contributes to a step."""
    tokens: list              # token ids of this step's rows (decode: [last committed, drafts...])
    pos0: int                 # position of the first row
    slot: int                 # GDN state slot (>= 1)
    shift: int                # rows of the previous decode step that were committed (0 after prefill)
    blocks: list              # physical KV block ids covering positions [0, pos0 + len(tokens))
    uid: int = 0
    step_no: int = 0
    rope_pos: Optional[object] = None   # int [3, rows]: three-axis rotary positions of the rows (prompts with images)
    rope_delta: int = 0       # added to the index of every row for the rotary position (after an image)
    next_token: int = -1      # the prompt token after this chunk's last row (-1: none), for prompt log-probabilities
    sampling: Optional[tuple] = None   # (temperature, top_k, top_p, min_p) of a sampled sequence the device may draw for
    uniforms: Optional[list] = None    # one uniform number per head row of this step (decode: every row; prefill: the last)
    blocks_key: Optional[object] = None   # identity of `blocks` (same key = same list contents): the block table row is then uploaded once


@dataclass
class StepResult:
    n_commit: list            # per sequence: tokens committed (decode) / 1 (prefill last chunk)
    tokens: list              # per sequence: committed token ids
    drafts: list              # per sequence: next block of draft tokens
    picks: list


def fill_blob(b: Bucket, seqs: list, page_tokens: int = 16) -> list:
    """Write the index tables of one step into the bucket's pinned blob.  Returns the word ranges
    [(first, count), ...] that have to reach the device: the header (every per-row and per-sequence
    table) and the block-table rows that changed.  A sequence's KV blocks are allocated up front
    and never change, so a row whose `blocks_key` is the one the device already holds is skipped:
    in steady-state decode no block-table byte crosses the bus (the reference sends the table only
    on page-crossing steps, `crates/saber-engine/src/tp2.rs:1897`)."""
    import numpy as np
    lay = b.layout
    a = b.blob_host.numpy()
    M, nseq = lay.M, lay.nseq
    hdr = lay.header_words
    a[:hdr] = 0
    a[lay.slot_map:lay.slot_map + M] = -1
    a[lay.next_ids:lay.next_ids + M] = -1
    a[lay.slots:lay.slots + nseq] = -1
    ranges = [(0, hdr)]
    row = 0
    for j, s in enumerate(seqs):
        n = len(s.tokens)
        a[lay.ids + row: lay.ids + row + n] = s.tokens
        a[lay.next_ids + row: lay.next_ids + row + n] = list(s.tokens[1:]) + [s.next_token]
        if s.sampling is not None and s.uniforms:
            hr0, hn = (row, n) if b.kind == "decode" else (j, 1)      # head rows of this sequence
            fa = a.view(np.float32)
            for r in range(min(hn, len(s.uniforms))):
                fa[lay.samp + 4 * (hr0 + r): lay.samp + 4 * (hr0 + r) + 4] = s.sampling
                fa[lay.samp_u + hr0 + r] = s.uniforms[r]
        pos = np.arange(s.pos0, s.pos0 + n, dtype=np.int32)
        for ax in range(3):
            a[lay.pos + ax * M + row: lay.pos + ax * M + row + n] = \
                pos + s.rope_delta if s.rope_pos is None else np.asarray(s.rope_pos[ax], dtype=np.int32)[:n]
        nblk = len(s.blocks)
        first_page, last_page = s.pos0 // page_tokens, (s.pos0 + n - 1) // page_tokens
        touched = np.asarray(s.blocks[first_page:last_page + 1], dtype=np.int32)     # pages this step's rows write
        a[lay.slot_map + row: lay.slot_map + row + n] = touched[pos // page_tokens - first_page] * page_tokens + pos % page_tokens
        a[lay.cu_rows + j] = row
        a[lay.slots + j] = s.slot
        a[lay.shift + j] = s.shift
        a[lay.kv_len + j] = s.pos0 + n
        a[lay.seq_uid + j] = s.uid
        a[lay.step_no + j] = s.step_no
        a[lay.last_rows + j] = row + n - 1
        bt = lay.block_table + j * lay.max_blocks
        sig = (s.blocks_key, nblk) if s.blocks_key is not None else None
        held = getattr(b, "bt_rows", None)
        if sig is None or held is None or held.get(j) != sig:
            a[bt: bt + nblk] = np.asarray(s.blocks, dtype=np.int32)
            ranges.append((bt, nblk))
            if held is not None:
                held[j] = sig
        row += n
    for j in range(len(seqs), nseq + 1):
        a[lay.cu_rows + j] = row
    assert row <= M, (row, M)
    return ranges


def run_bucket(model: "HybridModel", b: Bucket, seqs: list, eager: bool = False) -> StepResult:
    """One step: index tables host->device (pinned; only what changed), the program (graph replay
    or eager walk), results device->host, then parse."""
    ranges = fill_blob(b, seqs, model.cfg.page_tokens)
    st = model.stream
    with torch.cuda.stream(st):
        nbytes = 0
        for first, count in ranges:
            if count > 0:
                b.blob_dev[first:first + count].copy_(b.blob_host[first:first + count], non_blocking=True)
                nbytes += 4 * count
        b.last_h2d_bytes = nbytes
        if b.captured and not eager:
            b.program.replay(st)
        else:
            b.program.run(st)
        b.out_host.copy_(b.out_dev, non_blocking=True)
        if getattr(b, "seam_dev", None) is not None:
            b.seam_host.copy_(b.seam_dev, non_blocking=True)
        if getattr(b, "plp_dev", None) is not None:
            b.plp_host.copy_(b.plp_dev, non_blocking=True)
    # bounded: a step that never completes (a kernel wait that did not run out, a lost peer) raises,
    # and the scheduler's fatal law ends the engine instead of leaving this thread blocked
    from ..runtime.device_rt import bounded_wait
    bounded_wait(st, model.step_timeout_s, f"the {b.kind} step")
    return parse_result(b, len(seqs))


def parse_result(b: Bucket, n_live: int) -> StepResult:
    o = b.out_host.numpy()
    nseq, W, block, Mh = b.nseq, b.W, b.block, b.Mh
    o_commit = o[:nseq]
    o_tokens = o[nseq:nseq + nseq * W].reshape(nseq, W)
    nd = max(block, 1)
    o_drafts = o[nseq + nseq * W: nseq + nseq * W + nseq * nd].reshape(nseq, nd)
    o_picks = o[nseq + nseq * W + nseq * nd:]
    if b.kind == "decode":
        n_commit = [int(o_commit[j]) for j in range(n_live)]
        tokens = [o_tokens[j, :n_commit[j]].tolist() for j in range(n_live)]
    else:
        n_commit = [1] * n_live
        tokens = [[int(o_picks[j])] for j in range(n_live)]
    drafts = [o_drafts[j, :block].tolist() for j in range(n_live)]
    return StepResult(n_commit, tokens, drafts, o_picks.tolist())
