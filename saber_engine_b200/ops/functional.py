"""Eager wrappers over the native kernels (one launch each, on the current CUDA stream).

These are what tests and the prefill path call; captured decode buckets use `native.Program` with
the same parameter blocks.  Every wrapper requires a CUDA tensor and the native library: there is
no PyTorch fallback here (references live in `ops.reference`).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import layouts as L
from . import native as N


@dataclass
class QuantWeight:
    """A linear layer's weight in GEMM-ready form."""
    tiles: torch.Tensor      # uint8 [N_pad/256, K/128, 16384 | 32768]
    scale: torch.Tensor      # fp32 [N_pad] (W4: already divided by 16)
    N: int
    K: int
    w4: bool
    mx: bool = False         # MXFP4 tiles (e2m1 codes + block shifts): fp8 activations, fp32 accumulate
    had_sign: Optional[torch.Tensor] = None   # fp32 [K] +-1: the input must be rotated (sign, 32-point Hadamard) before quantisation
    paired: bool = False     # merged gate | up linear regrouped so that tile t holds gate and up features [128 t, 128 t + 128)
    fp4: int = 0             # native block-scaled FP4 tiles: 4 = NVFP4 (ue4m3 per 16), 5 = MXFP4 (ue8m0 per 32); FP4 activations

    @property
    def N_pad(self) -> int:
        return self.tiles.shape[0] * L.TILE_N

    @property
    def fmt_code(self) -> int:
        """The kernel's weight-format selector: 0 int8, 1 int4, 2 MXFP4 (widened to fp8), 4 / 5 native FP4."""
        if self.fp4:
            return self.fp4
        return 2 if self.mx else int(self.w4)

    @staticmethod
    def from_nvfp4(codes: torch.Tensor, block_scale: torch.Tensor, g, device=None) -> "QuantWeight":
        """e2m1 codes uint8 [N, K] + e4m3-valued block scales fp32 [N, K/16] + the tensor's fp32 scale:
        tiles for the native block-scaled MMA (nothing is requantised)."""
        Nn, K = codes.shape
        sf = block_scale.to(torch.float8_e4m3fn).view(torch.uint8)
        tiles = L.tile_weight_fp4(codes, sf, 16)
        dev = device if device is not None else codes.device
        sc = torch.full((tiles.shape[0] * L.TILE_N,), float(g), dtype=torch.float32)
        return QuantWeight(tiles.to(dev), sc.to(dev), Nn, K, True, fp4=4)

    @staticmethod
    def from_mxfp4_native(codes: torch.Tensor, e8m0: torch.Tensor, device=None) -> "QuantWeight":
        Nn, K = codes.shape
        tiles = L.tile_weight_fp4(codes, e8m0, 32)
        dev = device if device is not None else codes.device
        return QuantWeight(tiles.to(dev), torch.ones(tiles.shape[0] * L.TILE_N, dtype=torch.float32, device=dev), Nn, K, True, fp4=5)

    @staticmethod
    def from_mxfp4(codes: torch.Tensor, e8m0: torch.Tensor, device=None) -> "QuantWeight":
        """e2m1 codes uint8 [N, K] + e8m0 block scales uint8 [N, K/32] (the pack's MXFP4 records)."""
        from ..pack import quant_fp4 as Q
        Nn, K = codes.shape
        shift, row_scale = Q.fold_mxfp4(codes, e8m0)
        tiles = L.tile_weight_mxfp4(codes, shift)
        sc = torch.zeros(tiles.shape[0] * L.TILE_N, dtype=torch.float32)
        sc[:Nn] = row_scale
        dev = device if device is not None else codes.device
        return QuantWeight(tiles.to(dev).contiguous(), sc.to(dev), Nn, K, True, mx=True)

    @staticmethod
    def from_float(w: torch.Tensor, bits: int = 4, device=None) -> "QuantWeight":
        q, s = L.quantize_weight_rows(w, bits)
        return QuantWeight.from_int(q, s, bits, device)

    @staticmethod
    def from_int(q: torch.Tensor, s: torch.Tensor, bits: int, device=None) -> "QuantWeight":
        Nn, K = q.shape
        tiles = L.tile_weight_int4(q) if bits == 4 else L.tile_weight_int8(q)
        n_pad = tiles.shape[0] * L.TILE_N
        sc = torch.zeros(n_pad, dtype=torch.float32)
        sc[:Nn] = s.float() / (16.0 if bits == 4 else 1.0)
        dev = device if device is not None else q.device
        return QuantWeight(tiles.to(dev).contiguous(), sc.to(dev), Nn, K, bits == 4)


def pair_gate_up(w: QuantWeight) -> QuantWeight:
    """The merged gate | up linear with its tiles regrouped for the fused silu * mul epilogue (see
    `layouts.pair_gate_up_int4`); weights that cannot be paired (int8, MXFP4, ragged) come back unchanged."""
    if w.paired or not w.w4 or w.mx or w.fp4 or w.N % 256 or (w.N // 2) % 128:
        return w
    tiles, scale = L.pair_gate_up_int4(w.tiles, w.scale, w.N // 2)
    return QuantWeight(tiles, scale, w.N, w.K, True, had_sign=w.had_sign, paired=True)


def unpair_gate_up(w: QuantWeight) -> QuantWeight:
    """The canonical (gate rows, then up rows) form of a paired weight."""
    if not w.paired:
        return w
    tiles, scale = L.unpair_gate_up_int4(w.tiles, w.scale, w.N // 2)
    return QuantWeight(tiles, scale, w.N, w.K, True, had_sign=w.had_sign, paired=False)


@dataclass
class QuantAct:
    """Quantised activations in the tiled layout."""
    q: torch.Tensor          # int8 [K/128, M_pad, 128]
    scale: torch.Tensor      # fp32 [M_pad]
    M: int
    K: int
    fp8: bool = False        # bytes are fp8 e4m3 (scale = amax / 448) instead of int8 (amax / 127)
    fp4: int = 0             # 4 / 5: packed e2m1 rows [K/256, M_pad, 128] with block scales in `sf` (NVFP4 / MXFP4)
    sf: Optional[torch.Tensor] = None         # uint8 scale atoms [K/256, ceil(M_pad/128), atoms * 512]
    had_sign: Optional[torch.Tensor] = None   # rotation the producer applies before it quantises into this buffer

    @property
    def M_pad(self) -> int:
        return self.q.shape[1]

    @staticmethod
    def alloc(M: int, K: int, device, fp8: bool = False) -> "QuantAct":
        m_pad = L.padded_rows(M)
        return QuantAct(torch.empty(K // 128, m_pad, 128, dtype=torch.int8, device=device),
                        torch.empty(m_pad, dtype=torch.float32, device=device), M, K, fp8)

    def as_fp4(self, fmt: int = 4) -> "QuantAct":
        """The same storage seen as NVFP4 rows (half the bytes of the int8 rows) with scale atoms beside
        them (allocated on first use, zero: padding rows keep zero scales)."""
        assert self.K % 256 == 0, "FP4 rows come in k-blocks of 256 values"
        if getattr(self, "_sf", None) is None:
            self._sf = torch.zeros(self.K // 256, (self.M_pad + 127) // 128, 2048, dtype=torch.uint8, device=self.q.device)
        q = self.q.view(-1)[: self.K // 256 * self.M_pad * 128].view(self.K // 256, self.M_pad, 128)
        return QuantAct(q, self.scale, self.M, self.K, fp4=fmt, sf=self._sf, had_sign=self.had_sign)


class GemmScratch:
    """Split-K scratch of one device: int32 partial tiles [split][M_pad][N_pad], arrival counters
    and the status word.  Partials are overwritten by every launch and counters are left at zero,
    so one instance serves every GEMM launched in stream order on the device.
    """

    def __init__(self, device, max_rows: int = 256, max_cols: int = 262144):
        self.ws = torch.zeros(max_rows * max_cols, dtype=torch.int32, device=device)
        self.counters = torch.zeros(8192, dtype=torch.int32, device=device)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        # words of the fused tails (zero between launches): [0] grid-barrier counter, then one 128-byte line per row for the row maxima
        self.tail_sync = torch.zeros(64 + 256 * 32 + 256, dtype=torch.int32, device=device)
        # split-K accumulator blocks (nt x 256 int32 per tile), zero between launches
        self.acc = torch.zeros(80 * 32768, dtype=torch.int32, device=device)
        # blocks of the GEMMs whose row tail reads the accumulators itself: cleaned by each launch, not between launches
        self.acc_tail = torch.zeros(40 * 32768, dtype=torch.int32, device=device)
        self.capacity = max_rows * max_cols

    def check(self) -> None:
        code = int(self.err.item())
        if code != 0:
            self.err.zero_()
            self.counters.zero_()       # a kernel that gave up half-way leaves its arrival words behind
            self.tail_sync.zero_()
            self.acc.zero_()
            raise N.NativeError(f"kernel wait timed out: {N.ERR_NAMES.get(code, code)}")


_SCRATCH: dict = {}


def scratch(device) -> GemmScratch:
    key = torch.device(device).index or 0
    if key not in _SCRATCH:
        _SCRATCH[key] = GemmScratch(device)
    return _SCRATCH[key]


def pick_splits(n_tiles: int, m_tiles: int, kb: int, sms: Optional[int] = None) -> int:
    """Split-K factor that fills the SMs when the tile grid alone does not: the law and its numbers
    are the `[gemm.splits]` table of the launch rules (one wave, at most 8 parts, no empty part)."""
    from ..rules import default_rules
    return default_rules().gemm_splits(n_tiles, m_tiles, kb)


def gemm_params(w: QuantWeight, a: QuantAct, out: torch.Tensor, sc: GemmScratch,
                splits: Optional[int] = None, nt: Optional[int] = None, coop: int = 0, mtiles: int = 0,
                halves: int = 1) -> N.GemmI8Params:
    assert a.K == w.K, (a.K, w.K)
    nt = nt or L.token_tile(a.M)
    assert a.M_pad % nt == 0
    m_tiles = (a.M + nt - 1) // nt
    if splits is None:
        splits = pick_splits(w.N_pad // L.TILE_N, m_tiles, w.K // (256 if w.fp4 else 128))
    if splits > 1:   # one 128 x 256 int32 block per (split, tile)
        assert splits * m_tiles * (w.N_pad // L.TILE_N) * 32768 <= sc.capacity, "split-K scratch too small"
    p = N.GemmI8Params()
    p.w, p.w_scale, p.a, p.a_scale = w.tiles.data_ptr(), w.scale.data_ptr(), a.q.data_ptr(), a.scale.data_ptr()
    p.out, p.ws, p.counters, p.err = out.data_ptr(), sc.ws.data_ptr(), sc.counters.data_ptr(), sc.err.data_ptr()
    p.M, p.M_pad, p.N, p.N_pad, p.K = a.M, a.M_pad, w.N, w.N_pad, w.K
    assert bool(getattr(w, 'mx', False)) == bool(a.fp8), "MXFP4 weights take fp8 activations, integer weights int8"
    assert w.fp4 == a.fp4, "native FP4 weights take FP4 activations of the same block format"
    if w.fp4:
        p.a_sf = a.sf.data_ptr()
    p.nt, p.splits, p.w4, p.ldo = nt, splits, w.fmt_code, out.stride(0)
    p.coop = coop
    if splits > 1 and not getattr(w, "mx", False) and not w.fp4 and m_tiles * (w.N_pad // L.TILE_N) * nt * 256 <= sc.acc.numel():
        p.acc = sc.acc.data_ptr()       # integer partial sums meet in L2 (bulk reduction) instead of private copies
        if m_tiles * (w.N_pad // L.TILE_N) * nt * 256 <= sc.acc_tail.numel():
            p.acc_tail = sc.acc_tail.data_ptr()
    p.halves = halves      # 2: two CTAs per weight tile, each on 128 of its rows (packed int4, splits == 1)
    p.mtiles = mtiles      # 0: the launcher decides; 2: pair token tiles whenever the shape allows; -1: never
    assert out.stride(0) % 8 == 0, "GEMM output rows must be 16-byte aligned"
    return p


def quant_act_fp4(x: torch.Tensor, fmt: int, device=None) -> QuantAct:
    """Host-side (torch) FP4 quantiser of activation rows, the arithmetic the device producer follows.
    fmt 4 = NVFP4: per-token fp32 scale g = amax / (6 * 448), one e4m3 scale per 16 values, e2m1 codes;
    fmt 5 = MXFP4: one power-of-two scale per 32 values (token scale 1)."""
    from ..pack import quant_fp4 as Q
    x = x.to(torch.bfloat16).float().cpu()
    M, K = x.shape
    m_pad = L.padded_rows(M)
    if fmt == 4:
        g = (x.abs().amax(dim=1) / (6.0 * 448.0)).clamp_min(1e-30)
        b = x.reshape(M, K // 16, 16)
        bs = Q._e4m3_round((b.abs().amax(dim=-1) / 6.0 / g[:, None]).clamp(max=448.0))
        denom = (bs * g[:, None]).clamp_min(1e-30)
        codes = Q.e2m1_encode(b / denom[..., None]).reshape(M, K)
        sf = bs.to(torch.float8_e4m3fn).view(torch.uint8)
        q, at = L.tile_act_fp4(codes, sf, 16, m_pad)
    else:
        codes, e = Q.quantize_mxfp4(x)
        g = torch.ones(M)
        q, at = L.tile_act_fp4(codes, e, 32, m_pad)
    scale = torch.zeros(m_pad, dtype=torch.float32)
    scale[:M] = g
    dev = device if device is not None else x.device
    qa = QuantAct(q.to(dev), scale.to(dev), M, K, fp4=fmt, sf=at.to(dev))
    qa._codes, qa._g = codes, g             # (kept for tests: the exact dequantisation)
    return qa


def gemm_tail_silu_quant(p: N.GemmI8Params, qa_out: QuantAct, sc: GemmScratch) -> N.GemmI8Params:
    """Turn `p` (a paired gate | up linear, splits == 1) into the fused form: silu(gate) * up and the
    per-token int8 quantisation run in the epilogue and land in `qa_out` (K = N / 2)."""
    p.tail_mode = 1
    p.tail_q, p.tail_scale, p.tail_M_pad = qa_out.q.data_ptr(), qa_out.scale.data_ptr(), qa_out.M_pad
    p.tail_sync = sc.tail_sync.data_ptr()
    return p


def gemm_tail_row(p: N.GemmI8Params, row_p: N.RowOpParams, sc: GemmScratch) -> N.GemmI8Params:
    """Attach the add + RMSNorm + quantise row op `row_p` (which reads this GEMM's output) as the
    GEMM's row tail: it runs inside the same launch, after a grid-wide barrier."""
    p.tail_mode, p.tail_row_mode = 2, N.ROW_ADD_RMS
    p.tail_row = C.addressof(row_p)
    p._tail_keep = row_p                 # the block must outlive the launch / the add to a program
    p.tail_sync = sc.tail_sync.data_ptr()
    return p


def gemm_tail_ok(p: N.GemmI8Params) -> bool:
    """True when the launch of `p` keeps its whole grid resident (the condition of both fused tails)."""
    return bool(N.lib().saber_gemm_i8_tail_ok(C.byref(p)))


def gemm_i8(w: QuantWeight, a: QuantAct, out: Optional[torch.Tensor] = None,
            splits: Optional[int] = None, stages: int = 0, nt: Optional[int] = None, coop: int = 0, mtiles: int = 0,
            halves: int = 1) -> torch.Tensor:
    """out[M, N] = bf16(int32 accumulate * a_scale[m] * w_scale[n])."""
    dev = a.q.device
    if out is None:
        out = torch.empty(a.M, w.N, dtype=torch.bfloat16, device=dev)
    p = gemm_params(w, a, out, scratch(dev), splits, nt, coop, mtiles, halves)
    N.check(N.lib().saber_gemm_i8_launch(C.byref(p), stages, N.stream_handle()), "gemm_i8")
    return out


def pick_halves(w: QuantWeight, n_tiles: int, m_tiles: int, sms: Optional[int] = None) -> bool:
    """Half tiles instead of split-K (`[gemm.halves]` of the launch rules): packed int4 weights whose
    whole-tile grid fills between a quarter and a half of the SMs."""
    from ..rules import default_rules
    fmt = "fp4" if w.fp4 else ("mxfp4" if getattr(w, "mx", False) else ("int4" if w.w4 else "int8"))
    return default_rules().gemm_halves(fmt, n_tiles, m_tiles)


def row_params(M: int, K: int, *, a=None, a_f32=None, b=None, res=None, w=None, w_offset=0.0,
               eps=1e-6, out=None, qa: Optional[QuantAct] = None, lda=None, ldb=None) -> N.RowOpParams:
    p = N.RowOpParams()
    p.a, p.a_f32, p.b, p.res, p.w = N.ptr(a), N.ptr(a_f32), N.ptr(b), N.ptr(res), N.ptr(w)
    p.w_offset, p.eps = w_offset, eps
    p.out = N.ptr(out)
    p.q = qa.q.data_ptr() if qa is not None else None
    p.scale = qa.scale.data_ptr() if qa is not None else None
    p.M, p.M_pad, p.K = M, (qa.M_pad if qa is not None else M), K
    src = a if a is not None else a_f32
    p.lda = lda if lda is not None else (src.stride(0) if src is not None else 0)
    p.ldb = ldb if ldb is not None else (b.stride(0) if b is not None else 0)
    p.ldres = res.stride(0) if res is not None else 0
    p.ldout = out.stride(0) if out is not None else 0
    p.qfmt = (2 if qa.fp4 else int(qa.fp8)) if qa is not None else 0
    if qa is not None and qa.fp4:
        assert qa.fp4 == 4, "the device producers write NVFP4 rows"
        p.q_sf, p.sf_m_tiles = qa.sf.data_ptr(), qa.sf.shape[1]
    p.had_sign = N.ptr(qa.had_sign) if qa is not None else None
    return p


def _row(mode: int, p: N.RowOpParams) -> None:
    N.check(N.lib().saber_row_producer_launch(mode, C.byref(p), N.stream_handle()), "row_producer")


def add_rms_quant(x: Optional[torch.Tensor], res: Optional[torch.Tensor], w: torch.Tensor,
                  eps: float = 1e-6, w_offset: float = 1.0, want_out: bool = False,
                  quant: bool = True):
    """res += x (in place); n = rmsnorm(res) * (w_offset + w); returns (QuantAct | None, bf16 n | None)."""
    src = x if x is not None else res
    M, K = src.shape
    qa = QuantAct.alloc(M, K, src.device) if quant else None
    out = torch.empty(M, K, dtype=torch.bfloat16, device=src.device) if want_out else None
    _row(N.ROW_ADD_RMS, row_params(M, K, a=x, res=res, w=w, w_offset=w_offset, eps=eps, out=out, qa=qa))
    return qa, out


def silu_mul_quant(gu: torch.Tensor, want_out: bool = False, paired: bool = False):
    """paired: `gu` is the output of a paired gate | up linear (gate and up of feature 128 t + c sit at
    columns 256 t + c and 256 t + 128 + c)."""
    M, K2 = gu.shape
    K = K2 // 2
    qa = QuantAct.alloc(M, K, gu.device)
    out = torch.empty(M, K, dtype=torch.bfloat16, device=gu.device) if want_out else None
    p = row_params(M, K, a=gu, out=out, qa=qa)
    p.silu_pair = int(paired)
    _row(N.ROW_SILU_MUL, p)
    return qa, out


def gate_sigmoid_quant(a: torch.Tensor, gate: torch.Tensor, want_out: bool = False):
    M, K = a.shape
    qa = QuantAct.alloc(M, K, a.device)
    out = torch.empty(M, K, dtype=torch.bfloat16, device=a.device) if want_out else None
    _row(N.ROW_GATE_SIG, row_params(M, K, a=a, b=gate, out=out, qa=qa))
    return qa, out


def gdn_norm_quant(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float = 1e-6,
                   want_out: bool = False):
    """o fp32 [M, H*128], z bf16 [M, H*128] (may be a strided view), w fp32 [128]."""
    M, K = o.shape
    qa = QuantAct.alloc(M, K, o.device)
    out = torch.empty(M, K, dtype=torch.bfloat16, device=o.device) if want_out else None
    _row(N.ROW_GDN_NORM, row_params(M, K, a_f32=o, b=z, w=w, eps=eps, out=out, qa=qa))
    return qa, out


def plain_quant(x: torch.Tensor, fp8: bool = False) -> QuantAct:
    M, K = x.shape
    qa = QuantAct.alloc(M, K, x.device, fp8)
    _row(N.ROW_PLAIN, row_params(M, K, a=x, qa=qa))
    return qa


def embed_gather(table: torch.Tensor, ids: torch.Tensor, vocab_lo: int = 0) -> torch.Tensor:
    M, H = ids.numel(), table.shape[1]
    out = torch.empty(M, H, dtype=torch.bfloat16, device=table.device)
    N.check(N.lib().saber_embed_gather_launch(table.data_ptr(), ids.data_ptr(), out.data_ptr(), M, H,
                                              vocab_lo, table.shape[0], H, N.stream_handle()), "embed")
    return out


def argmax(logits: torch.Tensor, id_offset: int = 0):
    R, V = logits.shape
    idx = torch.empty(R, dtype=torch.int32, device=logits.device)
    val = torch.empty(R, dtype=torch.float32, device=logits.device)
    N.check(N.lib().saber_argmax_launch(logits.data_ptr(), R, logits.stride(0), V, id_offset,
                                        idx.data_ptr(), val.data_ptr(), N.stream_handle()), "argmax")
    return idx, val


def topk_seam(logits: torch.Tensor, temps: Optional[torch.Tensor] = None, id_offset: int = 0):
    R, V = logits.shape
    ids = torch.empty(R, N.SEAM_K, dtype=torch.int32, device=logits.device)
    vals = torch.empty(R, N.SEAM_K, dtype=torch.float32, device=logits.device)
    lse = torch.empty(R, 2, dtype=torch.float32, device=logits.device)
    N.check(N.lib().saber_topk_seam_launch(logits.data_ptr(), R, logits.stride(0), V, id_offset,
                                           N.ptr(temps), ids.data_ptr(), vals.data_ptr(),
                                           lse.data_ptr(), N.stream_handle()), "topk_seam")
    return ids, vals, lse


def verify_accept(draft, target, cu_rows, seq_uid, step_no, max_w: int, oracle_p: float = 0.0,
                  seed: int = 0):
    nseq = cu_rows.numel() - 1
    n_commit = torch.empty(nseq, dtype=torch.int32, device=draft.device)
    out_tokens = torch.zeros(nseq, max_w, dtype=torch.int32, device=draft.device)
    p = N.VerifyParams()
    p.draft, p.target, p.cu_rows = draft.data_ptr(), target.data_ptr(), cu_rows.data_ptr()
    p.seq_uid, p.step_no = seq_uid.data_ptr(), step_no.data_ptr()
    p.n_commit, p.out_tokens = n_commit.data_ptr(), out_tokens.data_ptr()
    p.accept_row, p.bonus = None, None
    p.nseq, p.max_w, p.oracle_p, p.seed = nseq, max_w, oracle_p, seed
    N.check(N.lib().saber_verify_launch(C.byref(p), N.stream_handle()), "verify")
    return n_commit, out_tokens


# ----------------------------------------------------------------------------------- GDN
def gdn_stash_stride(vs: int) -> int:
    return 128 + 128 // vs + 4


def gdn_conv_params(x, conv_w, hist, cu_rows, slots, shift, out, n_q, n_k, commit, ldx=None, dual: bool = False):
    """dual: a slot of `hist` holds two windows and the word naming the current one ([2 R + 1][C])."""
    p = N.GdnConvParams()
    p.x, p.conv_w, p.hist = x.data_ptr(), conv_w.data_ptr(), hist.data_ptr()
    p.cu_rows, p.slots, p.shift, p.out = cu_rows.data_ptr(), slots.data_ptr(), shift.data_ptr(), out.data_ptr()
    p.C, p.n_q, p.n_k = conv_w.shape[0], n_q, n_k
    p.ldx = ldx if ldx is not None else x.stride(0)
    p.hist_rows, p.commit, p.q_scale = ((hist.shape[1] - 1) // 2 if dual else hist.shape[1]), int(commit), 1.0 / math.sqrt(128.0)
    p.max_rows = x.shape[0]
    p.dual = int(dual)
    return p


def gdn_conv(x, conv_w, hist, cu_rows, slots, shift, n_q, n_k, commit=False, dual=False):
    """x bf16 [M, >=C] (first C columns are q|k|v); returns fp32 [M, C]."""
    M = x.shape[0]
    out = torch.empty(M, conv_w.shape[0], dtype=torch.float32, device=x.device)
    p = gdn_conv_params(x, conv_w, hist, cu_rows, slots, shift, out, n_q, n_k, commit, dual=dual)
    N.check(N.lib().saber_gdn_conv_launch(C.byref(p), slots.numel(), N.stream_handle()), "gdn_conv")
    return out


def gdn_rec_params(qkv, ba, A_log, dt_bias, state, stash, cu_rows, slots, shift, out, n_q, n_k,
                   HV, HK, commit, ldba=None, prefill_rows: bool = False, chunk_impl: int = 0):
    p = N.GdnRecParams()
    p.qkv, p.ba, p.A_log, p.dt_bias = qkv.data_ptr(), ba.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr()
    p.state, p.stash = state.data_ptr(), stash.data_ptr()
    p.cu_rows, p.slots, p.shift, p.out = cu_rows.data_ptr(), slots.data_ptr(), shift.data_ptr(), out.data_ptr()
    p.C, p.n_q, p.n_k, p.HV, p.HK = qkv.shape[1], n_q, n_k, HV, HK
    p.ldba = ldba if ldba is not None else ba.stride(0)
    p.stash_rows, p.commit = stash.shape[1], int(commit)
    p.prefill_rows = int(prefill_rows) if commit else 0      # 1: two state rows per thread (default), 2: one, 3: four
    p.chunk_impl = int(chunk_impl)                           # chunked prefill: 1 = tensor cores
    p.err = scratch(qkv.device).err.data_ptr() if qkv.is_cuda else 0
    return p


def gdn_recurrent(qkv, ba, A_log, dt_bias, state, stash, cu_rows, slots, shift, n_q, n_k, HV, HK,
                  commit=False, vs=2, prefill_rows: bool = False):
    M = qkv.shape[0]
    out = torch.empty(M, HV * 128, dtype=torch.float32, device=qkv.device)
    p = gdn_rec_params(qkv, ba, A_log, dt_bias, state, stash, cu_rows, slots, shift, out, n_q, n_k,
                       HV, HK, commit, prefill_rows=prefill_rows)
    N.check(N.lib().saber_gdn_recurrent_launch(C.byref(p), slots.numel(), vs, N.stream_handle()), "gdn_rec")
    return out


class GdnStepScratch:
    """Buffers between the phases of the fused decode step of one DeltaNet layer (shared by the layers
    of a program: launches are ordered): normed head outputs, row maxima per head, sequence tickets."""

    def __init__(self, M: int, HV: int, nseq: int, device):
        self.hout = torch.empty(M, HV * 128, dtype=torch.bfloat16, device=device)
        self.amax = torch.zeros(M, HV, dtype=torch.float32, device=device)
        self.tickets = torch.zeros(max(nseq, 1), dtype=torch.int32, device=device)


def gdn_hist_alloc(n_slots: int, rows: int, C_: int, device) -> torch.Tensor:
    """Conv windows of the fused decode step: two windows of `rows` rows per slot and a last row whose
    first word names the current one (zero = window 0)."""
    return torch.zeros(n_slots, 2 * rows + 1, C_, dtype=torch.bfloat16, device=device)


def gdn_step_params(x, z, ba, conv_w, A_log, dt_bias, norm_w, hist, state, stash, cu_rows, slots, shift,
                    scratch: GdnStepScratch, qa: QuantAct, n_q, n_k, HV, HK, max_rows, *, eps=1e-6,
                    w_offset=0.0, ldx=None, ldz=None, ldba=None) -> N.GdnStepParams:
    """Fused conv + recurrence + gated norm + quantisation of one decode step (`stash` is laid out
    for one value slice per head: [slots][rows][HV][1][260])."""
    p = N.GdnStepParams()
    p.x, p.z, p.ba = x.data_ptr(), z.data_ptr(), ba.data_ptr()
    p.conv_w, p.A_log, p.dt_bias, p.norm_w = conv_w.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr(), norm_w.data_ptr()
    p.hist, p.state, p.stash = hist.data_ptr(), state.data_ptr(), stash.data_ptr()
    p.cu_rows, p.slots, p.shift = cu_rows.data_ptr(), slots.data_ptr(), shift.data_ptr()
    p.hout, p.amax_part, p.tickets = scratch.hout.data_ptr(), scratch.amax.data_ptr(), scratch.tickets.data_ptr()
    p.q, p.scale = qa.q.data_ptr(), qa.scale.data_ptr()
    p.C, p.n_q, p.n_k, p.HV, p.HK = conv_w.shape[0], n_q, n_k, HV, HK
    p.ldx = ldx if ldx is not None else x.stride(0)
    p.ldz = ldz if ldz is not None else z.stride(0)
    p.ldba = ldba if ldba is not None else ba.stride(0)
    assert stash.shape[3] == 1 and stash.shape[4] == 260, "the fused step wants one value slice per head"
    p.hist_rows, p.stash_rows, p.M_pad = (hist.shape[1] - 1) // 2, stash.shape[1], qa.M_pad
    p.qfmt, p.max_rows = int(qa.fp8), max_rows
    p.q_scale, p.eps, p.w_offset = 1.0 / math.sqrt(128.0), eps, w_offset
    return p


def gdn_step(x, z, ba, conv_w, A_log, dt_bias, norm_w, hist, state, stash, cu_rows, slots, shift,
             qa: QuantAct, n_q, n_k, HV, HK, max_rows, eps=1e-6, w_offset=0.0, scratch=None):
    scratch = scratch or GdnStepScratch(x.shape[0], HV, slots.numel(), x.device)
    p = gdn_step_params(x, z, ba, conv_w, A_log, dt_bias, norm_w, hist, state, stash, cu_rows, slots, shift,
                        scratch, qa, n_q, n_k, HV, HK, max_rows, eps=eps, w_offset=w_offset)
    N.check(N.lib().saber_gdn_step_launch(C.byref(p), slots.numel(), N.stream_handle()), "gdn_step")
    return scratch


def gdn_chunk_scratch(total_rows: int, nseq: int, HV: int, device) -> torch.Tensor:
    n = N.lib().saber_gdn_chunk_scratch_bytes(total_rows, nseq, HV)
    return torch.empty(n // 4, dtype=torch.float32, device=device)


def gdn_chunked(qkv, ba, A_log, dt_bias, state, stash, cu_rows, slots, shift, n_q, n_k, HV, HK, max_rows: int,
                impl: int = 0):
    """Committing (prefill) recurrence by 64-row chunks; same contract as gdn_recurrent(commit=True).
    impl = 1: pair products on tf32 tiles, the chunk scan on tcgen05 with the state in tensor memory."""
    M = qkv.shape[0]
    out = torch.empty(M, HV * 128, dtype=torch.float32, device=qkv.device)
    p = gdn_rec_params(qkv, ba, A_log, dt_bias, state, stash, cu_rows, slots, shift, out, n_q, n_k, HV, HK, True,
                       chunk_impl=impl)
    scratch_t = gdn_chunk_scratch(M, slots.numel(), HV, qkv.device)
    N.check(N.lib().saber_gdn_chunk_launch(C.byref(p), slots.numel(), max_rows, scratch_t.data_ptr(), N.stream_handle()),
            "gdn_chunk")
    return out


# ----------------------------------------------------------------------------------- attention
def rope_kv_params(qkv, q_out, q_norm_w, k_norm_w, pos, slot_map, kv_cache, nq, nkv, q_off, k_off,
                   v_off, rot_dim=64, sections=(11, 11, 10), theta=1e7, eps=1e-6, w_offset=1.0,
                   k_scale=1.0, v_scale=1.0, page_layout: int = 0):
    p = N.RopeKvParams()
    p.qkv, p.q_out = qkv.data_ptr(), q_out.data_ptr()
    p.q_norm_w, p.k_norm_w = q_norm_w.data_ptr(), k_norm_w.data_ptr()
    p.pos, p.slot_map, p.kv_cache = pos.data_ptr(), slot_map.data_ptr(), kv_cache.data_ptr()
    p.M, p.ld, p.nq, p.nkv = qkv.shape[0], qkv.stride(0), nq, nkv
    p.q_off, p.k_off, p.v_off = q_off, k_off, v_off
    p.rot_dim, p.sec_h, p.sec_w = rot_dim, sections[1], sections[2]
    p.theta, p.eps, p.w_offset = theta, eps, w_offset
    p.k_inv_scale, p.v_inv_scale = 1.0 / k_scale, 1.0 / v_scale
    p.page_layout = page_layout      # 1: the tcgen05 attention's core-matrix page order
    return p


def rope_kv(qkv, q_norm_w, k_norm_w, pos, slot_map, kv_cache, nq, nkv, q_off, k_off, v_off, **kw):
    q_out = torch.empty(qkv.shape[0], nq, 256, dtype=torch.bfloat16, device=qkv.device)
    p = rope_kv_params(qkv, q_out, q_norm_w, k_norm_w, pos, slot_map, kv_cache, nq, nkv, q_off,
                       k_off, v_off, **kw)
    N.check(N.lib().saber_rope_kv_launch(C.byref(p), N.stream_handle()), "rope_kv")
    return q_out


def attn_params(q, kv_cache, block_table, cu_q, kv_len, out, part_o, part_ml, nkv, splits, q_tiles,
                k_scale=1.0, v_scale=1.0, sm_scale=None, pack_rows: int = 0, impl: int = 0, window: int = 0):
    p = N.AttnParams()
    p.q, p.kv_cache, p.block_table = q.data_ptr(), kv_cache.data_ptr(), block_table.data_ptr()
    p.cu_q, p.kv_len, p.out = cu_q.data_ptr(), kv_len.data_ptr(), out.data_ptr()
    p.part_o, p.part_ml = N.ptr(part_o), N.ptr(part_ml)
    p.nseq, p.nq, p.nkv = kv_len.numel(), q.shape[1], nkv
    p.max_blocks, p.splits, p.q_tiles = block_table.shape[1], splits, q_tiles
    p.sm_scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(256.0)
    p.k_scale, p.v_scale = k_scale, v_scale
    p.err = scratch(q.device).err.data_ptr()
    p.n_blocks = kv_cache.shape[0]
    p.pack_rows = pack_rows if q_tiles == 1 else 0
    p.impl = impl                    # 1: tcgen05 kernel (pages in core-matrix order)
    p.window = window                # > 0: a row sees its last `window` keys only (tcgen05 kernel)
    return p


def attention(q, kv_cache, block_table, cu_q, kv_len, nkv, max_rows_per_seq: int, splits: int = 1,
              k_scale=1.0, v_scale=1.0, impl: int = 0, window: int = 0):
    """q bf16 [M, nq, 256]; returns bf16 [M, nq, 256]."""
    out = torch.empty_like(q)
    nseq, nq = kv_len.numel(), q.shape[1]
    q_tiles = (max_rows_per_seq + 15) // 16
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty(nseq, nq, splits, 16, 256, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(nseq, nq, splits, 16, 2, dtype=torch.float32, device=q.device)
    p = attn_params(q, kv_cache, block_table, cu_q, kv_len, out, part_o, part_ml, nkv, splits,
                    q_tiles, k_scale, v_scale, pack_rows=max_rows_per_seq, impl=impl, window=window)
    N.check(N.lib().saber_attn_launch(C.byref(p), N.stream_handle()), "attn")
    return out
