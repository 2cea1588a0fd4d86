"""The mixture-of-experts MLP block as step-program ops.

    router GEMM (replicated) -> route (top-k, expert-major placement, tile table)
    -> gather quantised rows into expert order -> grouped gate_up GEMM -> silu*mul + int8 quant
    -> grouped down GEMM -> shared expert (gate_up, silu*mul, down)
    -> combine: sum_k w_k * y_k + sigmoid(g) * shared, written to `delta` (one GPU) or pushed to every
       rank's receive region over peer memory (expert parallel), where the next add-norm sums ranks.

The grouped GEMMs are the same tcgen05 int8 kernel as every other linear, in its grouped mode:
blockIdx.y walks the device-built tile table, so the grid is static and the block captures into a
CUDA graph although the routing changes every step.

With tensor-parallel attention the normed hidden state is already replicated on every GPU, so the
"dispatch" half of expert parallelism is a local filter (each rank keeps the routes of the experts it
owns) and only the combine crosses NVLink.

Parity: `crates/saber-kernels/hip/moe_route.hip:1-30`, `moe_grouped.hip` (tile = expert, row0, rows),
`moe_grouped_far.hip` (expert output all-reduce fused into the combine), `crates/saber-kernels/src/moe.rs:19-27`.
"""
from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops import layouts as L
from ..ops import native as N


def rows_capacity(M: int, top_k: int, e_n: int) -> int:
    """Upper bound of the 16-row-padded expert-major row space."""
    routes = M * top_k
    return L.round_up(routes + 15 * min(e_n, routes), 16)


def group_tile_rows(M: int, top_k: int, n_experts: int) -> int:
    avg = -(-M * top_k // n_experts)
    for nt in (16, 32, 64, 128):
        if avg <= nt:
            return nt
    return 128


class MoeWorkspace:
    """Per-bucket buffers of the MoE block (shared by all layers of the bucket)."""

    def __init__(self, cfg, e_n: int, M: int, device, shared_inter: int):
        m = cfg.moe
        self.mx = getattr(m, "expert_format", "iu8") == "mxfp4"     # the experts' rows are fp8 e4m3
        dev = device
        H, I, K = cfg.hidden, m.expert_inter, m.top_k
        self.M, self.e_n = M, e_n
        self.nt = group_tile_rows(M, K, m.n_experts)
        self.rows_cap = rows_capacity(M, K, e_n)
        m_pad = L.round_up(self.rows_cap, 128) + 128       # slack: a tile's loads may run past the live rows
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)       # noqa: E731
        bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)     # noqa: E731
        self.e_ld = L.round_up(m.n_experts, 8)
        self.logits = bf(M, self.e_ld)
        self.topk_id, self.topk_w = i32(M, K), torch.zeros(M, K, dtype=torch.float32, device=dev)
        self.counts, self.offsets, self.cursors = i32(e_n), i32(e_n + 1), i32(e_n)
        self.tiles = i32(m_pad // 16 + 1, 4)
        self.ntiles = i32(2)
        self.src_row, self.slot_of = i32(m_pad), i32(M, K)
        self.qa_sorted = F.QuantAct(torch.zeros(H // 128, m_pad, 128, dtype=torch.int8, device=dev),
                                    torch.zeros(m_pad, dtype=torch.float32, device=dev), self.rows_cap, H, fp8=self.mx)
        self.gu = bf(m_pad, 2 * I)
        self.qa_inter = F.QuantAct(torch.zeros(I // 128, m_pad, 128, dtype=torch.int8, device=dev),
                                   torch.zeros(m_pad, dtype=torch.float32, device=dev), self.rows_cap, I, fp8=self.mx)
        self.y = bf(m_pad, H)
        self.shared_inter = shared_inter
        if shared_inter:
            self.sgu_ld = L.round_up(2 * shared_inter + 1, 8)
            self.sgu = bf(M, self.sgu_ld)
            self.qa_si = F.QuantAct.alloc(M, shared_inter, dev)
            self.shared_out = bf(M, H)


def route_params(ws: MoeWorkspace, cfg, e_lo: int) -> N.MoeRouteParams:
    m = cfg.moe
    p = N.MoeRouteParams()
    p.logits, p.topk_id, p.topk_w = ws.logits.data_ptr(), ws.topk_id.data_ptr(), ws.topk_w.data_ptr()
    p.counts, p.offsets, p.cursors = ws.counts.data_ptr(), ws.offsets.data_ptr(), ws.cursors.data_ptr()
    p.tiles, p.ntiles = ws.tiles.data_ptr(), ws.ntiles.data_ptr()
    p.src_row, p.slot_of = ws.src_row.data_ptr(), ws.slot_of.data_ptr()
    p.M, p.ld, p.E, p.top_k, p.nt, p.rows_cap = ws.M, ws.e_ld, m.n_experts, m.top_k, ws.nt, ws.src_row.numel()
    p.e_lo, p.e_n, p.norm_topk = e_lo, ws.e_n, int(m.norm_topk_prob)
    return p


def grouped_gemm_params(stack, a: F.QuantAct, out: torch.Tensor, ws: MoeWorkspace, sc: F.GemmScratch) -> N.GemmI8Params:
    p = N.GemmI8Params()
    p.w, p.w_scale, p.a, p.a_scale = stack.tiles.data_ptr(), stack.scale.data_ptr(), a.q.data_ptr(), a.scale.data_ptr()
    p.out, p.ws, p.counters, p.err = out.data_ptr(), sc.ws.data_ptr(), sc.counters.data_ptr(), sc.err.data_ptr()
    p.M, p.M_pad, p.N, p.N_pad, p.K = a.M_pad, a.M_pad, stack.N, stack.N_pad, stack.K
    p.nt, p.splits, p.w4, p.ldo = ws.nt, 1, (2 if getattr(stack, "mx", False) else 1), out.stride(0)
    p.group_tiles, p.group_ntiles, p.group_w_stride = ws.tiles.data_ptr(), ws.ntiles.data_ptr(), stack.stride_bytes
    return p


def combine_params(ws: MoeWorkspace, cfg, out: torch.Tensor, comm=None, tp_site: int = -1) -> N.MoeCombineParams:
    p = N.MoeCombineParams()
    H = cfg.hidden
    p.y, p.topk_w, p.slot_of, p.out = ws.y.data_ptr(), ws.topk_w.data_ptr(), ws.slot_of.data_ptr(), out.data_ptr()
    if ws.shared_inter:
        p.shared = ws.shared_out.data_ptr()
        p.shared_gate = ws.sgu.data_ptr() + 2 * ws.shared_inter * 2
        p.ldg = ws.sgu_ld
    p.M, p.H, p.top_k = ws.M, H, cfg.moe.top_k
    tiles_n = L.round_up(H, 256) // 256
    nt = 16
    while tiles_n * ((ws.M + nt - 1) // nt) > N.TP_MAX_TILES:
        nt *= 2
    p.nt = nt
    if comm is not None and tp_site >= 0:
        g = N.GemmI8Params()
        comm.gemm_tp(g, tp_site)
        for r in range(comm.nranks):
            p.tp_recv[r], p.tp_flags[r] = g.tp_recv[r], g.tp_flags[r]
        p.tp_seq_base, p.tp_nranks, p.tp_rank, p.tp_site = g.tp_seq_base, g.tp_nranks, g.tp_rank, g.tp_site
        p.tp_rows, p.tp_ld = g.tp_rows, g.tp_ld
    return p


def add_moe_ops(prog: N.Program, ws: MoeWorkspace, cfg, moe: dict, qa_h: F.QuantAct, out: torch.Tensor,
                sc: F.GemmScratch, tag: str, comm=None, tp_site: int = -1, pick_splits=None) -> int:
    """Appends the block; returns the combine's row-tile height (the consumer's `tp_nt`)."""
    M = ws.M

    def dense(w, a, o, name):
        splits = pick_splits(w, a) if pick_splits else None
        prog.gemm(F.gemm_params(w, a, o, sc, splits=splits), 0, tag=f"{tag}.{name}")

    dense(moe["router"], qa_h, ws.logits, "router")
    prog.add_moe_route(route_params(ws, cfg, moe["e_lo"]), tag=f"{tag}.route")
    prog.add_moe_gather(qa_h, ws.src_row, ws.ntiles, ws.qa_sorted, ws.rows_cap, tag=f"{tag}.gather", to_fp8=ws.mx)
    prog.gemm(grouped_gemm_params(moe["gate_up"], ws.qa_sorted, ws.gu, ws, sc), 0, tag=f"{tag}.experts.gate_up")
    rp = F.row_params(ws.rows_cap, cfg.moe.expert_inter, a=ws.gu, qa=ws.qa_inter)
    rp.m_live = ws.ntiles.data_ptr() + 4
    prog.row(N.ROW_SILU_MUL, rp, tag=f"{tag}.experts.silu_mul_quant")
    prog.gemm(grouped_gemm_params(moe["down"], ws.qa_inter, ws.y, ws, sc), 0, tag=f"{tag}.experts.down")
    if ws.shared_inter:
        dense(moe["shared_gate_up"], qa_h, ws.sgu, "shared.gate_up")
        prog.row(N.ROW_SILU_MUL, F.row_params(M, ws.shared_inter, a=ws.sgu, qa=ws.qa_si), tag=f"{tag}.shared.silu_mul_quant")
        dense(moe["shared_down"], ws.qa_si, ws.shared_out, "shared.down")
    cp = combine_params(ws, cfg, out, comm, tp_site)
    prog.add_moe_combine(cp, tag=f"{tag}.combine")
    return cp.nt


def add_moe_block(model, prog: N.Program, lw, qa_h: F.QuantAct, h, delta, M: int, tag: str, keep: list,
                  tp_site: int = -1) -> int:
    """Called by the hybrid model's bucket builder for every layer with experts."""
    ws = getattr(prog, "_moe_ws", None)
    if ws is None:
        si = max((l.moe["shared_inter"] for l in model.w.layers if l.moe), default=0)
        ws = MoeWorkspace(model.cfg, lw.moe["e_n"], M, model.device, si)
        prog._moe_ws = ws
        keep.append(ws)
    comm = model.comm if model.tp > 1 else None
    return add_moe_ops(prog, ws, model.cfg, lw.moe, qa_h, delta, model.scratch, f"{tag}.moe", comm, tp_site,
                       pick_splits=model.pick_splits)
