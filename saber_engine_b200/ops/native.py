"""ctypes binding of the native library (`_lib/libsaber_b200.so`).

The library exposes plain-C launchers that take a parameter block and a CUDA stream.  This module
mirrors the parameter blocks as `ctypes.Structure`s, loads the library once, and offers:

* `lib()`         the loaded CDLL (raises loudly when the library is missing on a GPU box: a silent
                  PyTorch fallback would hide that no native code ran),
* small helpers to turn torch tensors into device pointers,
* `Program`       the native step program (eager walk or CUDA-graph capture/replay).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional

import torch

from .. import build as _build

_LIB: Optional[C.CDLL] = None

P = C.c_void_p
I = C.c_int
F = C.c_float
U32 = C.c_uint32
U64 = C.c_uint64
MAX_RANKS = 8
AR_BLOCKS = 32
SEAM_K = 64
TP_MAX_TILES = 512

ROW_ADD_RMS, ROW_SILU_MUL, ROW_GATE_SIG, ROW_GDN_NORM, ROW_PLAIN = range(5)

ERR_NAMES = {
    0: "ok", 1: "wait_full", 2: "wait_empty", 3: "wait_ready", 4: "wait_acc", 5: "wait_peer",
    6: "wait_drain", 7: "bad_args", 8: "wait_split", 9: "bad_index",
}


class GemmI8Params(C.Structure):
    _fields_ = [("w", P), ("w_scale", P), ("a", P), ("a_scale", P), ("out", P), ("ws", P),
                ("counters", P), ("err", P), ("M", I), ("M_pad", I), ("N", I), ("N_pad", I),
                ("K", I), ("nt", I), ("splits", I), ("w4", I), ("ldo", I), ("dbg_mma", I), ("tp_recv", P * 8), ("tp_flags", P * 8), ("tp_seq_base", P),
                ("tp_nranks", I), ("tp_rank", I), ("tp_site", I), ("tp_rows", I), ("tp_ld", I), ("tp_rpr", I), ("ag_flags", P), ("ag_seq_base", P), ("ag_site", I),
                ("group_tiles", P), ("group_ntiles", P), ("group_w_stride", U64), ("coop", I), ("mtiles", I), ("dbg", P), ("bias", P), ("res", P), ("epi", I),
                ("tail_mode", I), ("tail_row_mode", I), ("tail_row", P), ("tail_q", P), ("tail_scale", P), ("tail_M_pad", I),
                ("tail_sync", P), ("next_w", P), ("next_tiles", I), ("next_splits", I), ("next_KB", I), ("next_kb_per", I),
                ("next_wbytes", I), ("next_pref", I), ("acc", P), ("acc_tail", P), ("halves", I), ("a_sf", P)]


class RowOpParams(C.Structure):
    _fields_ = [("a", P), ("a_f32", P), ("b", P), ("res", P), ("w", P), ("w_offset", F),
                ("eps", F), ("out", P), ("q", P), ("scale", P), ("M", I), ("M_pad", I), ("K", I),
                ("lda", I), ("ldb", I), ("ldres", I), ("ldout", I), ("tp_recv", P), ("tp_flags", P),
                ("tp_seq_base", P), ("err", P), ("tp_nranks", I), ("tp_site", I), ("tp_rows", I), ("tp_ld", I),
                ("tp_nt", I), ("tp_tiles_n", I), ("m_live", P), ("qfmt", I), ("had_sign", P),
                ("sp_q", P * MAX_RANKS), ("sp_scale", P * MAX_RANKS), ("sp_flags", P * MAX_RANKS), ("sp_counter", P),
                ("sp_rpr", I), ("sp_rank", I), ("res_copy", P), ("silu_pair", I),
                ("acc", P), ("acc_a_scale", P), ("acc_w_scale", P), ("acc_nt", I), ("acc_tiles_n", I),
                ("q_sf", P), ("sf_m_tiles", I)]


class GdnConvParams(C.Structure):
    _fields_ = [("x", P), ("conv_w", P), ("hist", P), ("cu_rows", P), ("slots", P), ("shift", P),
                ("out", P), ("C", I), ("n_q", I), ("n_k", I), ("ldx", I), ("hist_rows", I),
                ("commit", I), ("q_scale", F), ("max_rows", I), ("dual", I)]


class GdnStepParams(C.Structure):
    _fields_ = [("x", P), ("z", P), ("ba", P), ("conv_w", P), ("A_log", P), ("dt_bias", P), ("norm_w", P),
                ("hist", P), ("state", P), ("stash", P), ("cu_rows", P), ("slots", P), ("shift", P),
                ("hout", P), ("amax_part", P), ("tickets", P), ("q", P), ("scale", P),
                ("C", I), ("n_q", I), ("n_k", I), ("HV", I), ("HK", I), ("ldx", I), ("ldz", I), ("ldba", I),
                ("hist_rows", I), ("stash_rows", I), ("M_pad", I), ("qfmt", I), ("max_rows", I),
                ("q_scale", F), ("eps", F), ("w_offset", F)]


class GdnRecParams(C.Structure):
    _fields_ = [("qkv", P), ("ba", P), ("A_log", P), ("dt_bias", P), ("state", P), ("stash", P),
                ("cu_rows", P), ("slots", P), ("shift", P), ("out", P), ("C", I), ("n_q", I),
                ("n_k", I), ("HV", I), ("HK", I), ("ldba", I), ("stash_rows", I), ("commit", I), ("prefill_rows", I),
                ("chunk_impl", I), ("err", P)]


class RopeKvParams(C.Structure):
    _fields_ = [("qkv", P), ("q_out", P), ("q_norm_w", P), ("k_norm_w", P), ("pos", P),
                ("slot_map", P), ("kv_cache", P), ("M", I), ("ld", I), ("nq", I), ("nkv", I),
                ("q_off", I), ("k_off", I), ("v_off", I), ("rot_dim", I), ("sec_h", I),
                ("sec_w", I), ("theta", F), ("eps", F), ("w_offset", F), ("k_inv_scale", F),
                ("v_inv_scale", F), ("page_layout", I)]


class AttnParams(C.Structure):
    _fields_ = [("q", P), ("kv_cache", P), ("block_table", P), ("cu_q", P), ("kv_len", P),
                ("out", P), ("part_o", P), ("part_ml", P), ("nseq", I), ("nq", I), ("nkv", I),
                ("max_blocks", I), ("splits", I), ("q_tiles", I), ("sm_scale", F), ("k_scale", F),
                ("v_scale", F), ("err", P), ("pack_rows", I), ("n_blocks", I), ("impl", I), ("window", I)]


class DraftIndexParams(C.Structure):
    _fields_ = [("pos", P), ("cu_rows", P), ("kv_len", P), ("acc_row", P), ("block_table", P), ("pos_out", P),
                ("slot_out", P), ("kv_len_out", P), ("M", I), ("nseq", I), ("block", I), ("max_blocks", I), ("page_tokens", I)]


class VerifyParams(C.Structure):
    _fields_ = [("draft", P), ("target", P), ("cu_rows", P), ("seq_uid", P), ("step_no", P),
                ("n_commit", P), ("out_tokens", P), ("accept_row", P), ("bonus", P), ("nseq", I), ("max_w", I), ("oracle_p", F),
                ("seed", U64)]


class AllReduceParams(C.Structure):
    _fields_ = [("inp", P), ("out", P), ("peer_recv", P * MAX_RANKS), ("peer_flags", P * MAX_RANKS),
                ("seq_base", P), ("err", P), ("n_elems", I), ("max_elems", I), ("site", I),
                ("nranks", I), ("rank", I), ("spin_limit_us", U32), ("diag", P), ("chk_fault", I)]


class ArEmulParams(C.Structure):
    _fields_ = [("r", AllReduceParams * MAX_RANKS), ("nranks", I), ("checked", I)]


AR_DIAG = {"blocks": 0, "mismatch": 1, "converged": 2, "never": 3, "ahead": 4, "drift": 5, "timeout": 6,
           "first_seq": 8, "first_block": 9, "first_src": 10, "polls": 11, "last_seq": 12}


class SeamMergeParams(C.Structure):
    _fields_ = [("ids", P), ("vals", P), ("lse", P), ("peer_win", P * MAX_RANKS), ("peer_flags", P * MAX_RANKS),
                ("seq_base", P), ("err", P), ("rows", I), ("rows_max", I), ("site", I), ("nranks", I), ("rank", I)]


class SeamEmulParams(C.Structure):
    _fields_ = [("r", SeamMergeParams * MAX_RANKS), ("nranks", I)]


class PickMergeParams(C.Structure):
    _fields_ = [("idx", P), ("val", P), ("peer_win", P * MAX_RANKS), ("peer_flags", P * MAX_RANKS),
                ("seq_base", P), ("err", P), ("rows", I), ("rows_max", I), ("site", I), ("nranks", I), ("rank", I)]


class MoeRouteParams(C.Structure):
    _fields_ = [("logits", P), ("topk_id", P), ("topk_w", P), ("counts", P), ("offsets", P), ("cursors", P),
                ("tiles", P), ("ntiles", P), ("src_row", P), ("slot_of", P), ("M", I), ("ld", I), ("E", I),
                ("top_k", I), ("nt", I), ("rows_cap", I), ("e_lo", I), ("e_n", I), ("norm_topk", I)]


class MoeCombineParams(C.Structure):
    _fields_ = [("y", P), ("shared", P), ("shared_gate", P), ("topk_w", P), ("slot_of", P), ("out", P),
                ("M", I), ("H", I), ("top_k", I), ("nt", I), ("ldg", I), ("tp_recv", P * MAX_RANKS),
                ("tp_flags", P * MAX_RANKS), ("tp_seq_base", P), ("tp_nranks", I), ("tp_rank", I),
                ("tp_site", I), ("tp_rows", I), ("tp_ld", I)]


class VisRowsParams(C.Structure):
    _fields_ = [("x", P), ("x_f32", I), ("ldx", I), ("ln_w", P), ("ln_b", P), ("eps", F), ("tiled", P),
                ("M", I), ("K", I), ("K_pad", I), ("M_pad", I), ("group", I)]


class VisPosAddParams(C.Structure):
    _fields_ = [("x", P), ("ldx", I), ("table", P), ("ldt", I), ("idx", P), ("wt", P), ("M", I), ("K", I)]


class VisAttnParams(C.Structure):
    _fields_ = [("qkv", P), ("ldq", I), ("cos_t", P), ("sin_t", P), ("out_tiled", P), ("M_pad", I),
                ("blocks", P), ("heads", I), ("width", I), ("scale", F)]


def lib() -> C.CDLL:
    """Load the native library (building it first when absent and a compiler is present)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _build.lib_path()
    if not path.exists():
        try:
            _build.build()
        except Exception as exc:  # pragma: no cover - depends on the box
            raise RuntimeError(
                f"native library {path} is missing and could not be built: {exc}. "
                "Run `python -m saber_engine_b200.build`.") from exc
    _LIB = C.CDLL(str(path))
    _declare(_LIB)
    if os.environ.get("SABER_GEMM_2SM", "") != "":       # A/B switch: int8 prefill GEMMs on CTA pairs (1) or not (0)
        _LIB.saber_set_gemm_2sm(int(os.environ["SABER_GEMM_2SM"]))
    return _LIB


def set_gemm_2sm(on: bool) -> None:
    """int8-weight GEMMs over long row runs on CTA pairs (`tcgen05.mma.cta_group::2`) from now on."""
    lib().saber_set_gemm_2sm(int(bool(on)))


def set_pdl(mode: int) -> None:
    """Programmatic dependent launch for kernels launched from now on: 0 off, 1 every kernel,
    2 only the GEMMs."""
    lib().saber_set_pdl(int(mode))


def available() -> bool:
    try:
        lib()
        return True
    except Exception:
        return False


def _declare(L: C.CDLL) -> None:
    S = C.c_void_p  # cudaStream_t
    sig = {
        "saber_gemm_i8_launch": (I, [C.POINTER(GemmI8Params), I, S]),
        "saber_gemm_i8_parts": (I, [C.POINTER(GemmI8Params)]),
        "saber_gemm_i8_smem_bytes": (I, [I, I]),
        "saber_gemm_i8_smem_bytes_w": (I, [I, I, I]),
        "saber_row_producer_launch": (I, [I, C.POINTER(RowOpParams), S]),
        "saber_embed_gather_launch": (I, [P, P, P, I, I, I, I, I, S]),
        "saber_block_expand_launch": (I, [P, P, P, P, I, I, I, S]),
        "saber_gdn_conv_launch": (I, [C.POINTER(GdnConvParams), I, S]),
        "saber_gdn_recurrent_launch": (I, [C.POINTER(GdnRecParams), I, I, S]),
        "saber_gdn_step_launch": (I, [C.POINTER(GdnStepParams), I, S]),
        "saber_program_add_gdn_step": (I, [P, C.POINTER(GdnStepParams), I, C.c_char_p]),
        "saber_gdn_chunk_scratch_bytes": (C.c_size_t, [I, I, I]),
        "saber_gdn_chunk_launch": (I, [C.POINTER(GdnRecParams), I, I, P, S]),
        "saber_program_add_gdn_chunk": (I, [P, C.POINTER(GdnRecParams), I, I, P, C.c_char_p]),
        "saber_rope_kv_launch": (I, [C.POINTER(RopeKvParams), S]),
        "saber_attn_launch": (I, [C.POINTER(AttnParams), S]),
        "saber_argmax_launch": (I, [P, I, I, I, I, P, P, S]),
        "saber_topk_seam_launch": (I, [P, I, I, I, I, P, P, P, P, S]),
        "saber_verify_launch": (I, [C.POINTER(VerifyParams), S]),
        "saber_allreduce_launch": (I, [C.POINTER(AllReduceParams), S]),
        "saber_allreduce_chk_launch": (I, [C.POINTER(AllReduceParams), S]),
        "saber_allreduce_emul_launch": (I, [C.POINTER(ArEmulParams), S]),
        "saber_pick_merge_launch": (I, [C.POINTER(PickMergeParams), S]),
        "saber_seam_merge_launch": (I, [C.POINTER(SeamMergeParams), S]),
        "saber_seam_merge_emul_launch": (I, [C.POINTER(SeamEmulParams), S]),
        "saber_program_add_seam_merge": (I, [P, C.POINTER(SeamMergeParams), C.c_char_p]),
        "saber_program_add_pick_merge": (I, [P, C.POINTER(PickMergeParams), C.c_char_p]),
        "saber_comm_advance_launch": (I, [P, U32, S]),
        "saber_ipc_get_handle": (I, [P, P]),
        "saber_ipc_open_handle": (I, [P, C.POINTER(P)]),
        "saber_ipc_close": (I, [P]),
        "saber_dev_malloc": (I, [C.POINTER(P), C.c_size_t]),
        "saber_dev_free": (I, [P]),
        "saber_dev_memset": (I, [P, I, C.c_size_t]),
        "saber_dev_read_u32": (I, [P, C.POINTER(U32)]),
        "saber_program_create": (P, []),
        "saber_program_destroy": (None, [P]),
        "saber_program_add_gemm": (I, [P, C.POINTER(GemmI8Params), I, C.c_char_p]),
        "saber_program_add_row": (I, [P, I, C.POINTER(RowOpParams), C.c_char_p]),
        "saber_program_link_prefetch": (I, [P, I]),
        "saber_gemm_i8_tail_ok": (I, [C.POINTER(GemmI8Params)]),
        "saber_set_coop_launch": (None, [I]),
        "saber_gemm_i8_noalloc_status": (I, [S]),
        "saber_program_add_embed": (I, [P, P, P, P, I, I, I, I, I, C.c_char_p]),
        "saber_program_add_expand": (I, [P, P, P, P, P, I, I, I, C.c_char_p]),
        "saber_program_add_advance": (I, [P, P, U32, C.c_char_p]),
        "saber_program_add_gdn_conv": (I, [P, C.POINTER(GdnConvParams), I, C.c_char_p]),
        "saber_program_add_gdn_rec": (I, [P, C.POINTER(GdnRecParams), I, I, C.c_char_p]),
        "saber_program_add_rope": (I, [P, C.POINTER(RopeKvParams), C.c_char_p]),
        "saber_program_add_attn": (I, [P, C.POINTER(AttnParams), C.c_char_p]),
        "saber_program_add_argmax": (I, [P, P, I, I, I, I, P, P, C.c_char_p]),
        "saber_program_add_seam": (I, [P, P, I, I, I, I, P, P, P, P, C.c_char_p]),
        "saber_program_add_logit_gather": (I, [P, P, I, I, I, I, P, P, C.c_char_p]),
        "saber_program_add_sample_seam": (I, [P, P, P, P, P, P, I, C.c_char_p]),
        "saber_sample_seam_launch": (I, [P, P, P, P, P, I, S]),
        "saber_program_add_verify": (I, [P, C.POINTER(VerifyParams), C.c_char_p]),
        "saber_program_add_memset": (I, [P, P, I, C.c_size_t, C.c_char_p]),
        "saber_program_add_copy": (I, [P, P, P, C.c_size_t, C.c_char_p]),
        "saber_program_add_allreduce": (I, [P, C.POINTER(AllReduceParams), C.c_char_p]),
        "saber_digest_launch": (I, [P, C.c_size_t, P, S]),
        "saber_digest_clear_launch": (I, [P, I, S]),
        "saber_program_add_digest": (I, [P, P, C.c_size_t, P, C.c_char_p]),
        "saber_program_add_digest_clear": (I, [P, P, I, C.c_char_p]),
        "saber_set_pdl": (None, [I]),
        "saber_get_pdl": (I, []),
        "saber_draft_index_launch": (I, [C.POINTER(DraftIndexParams), S]),
        "saber_program_add_draft_index": (I, [P, C.POINTER(DraftIndexParams), C.c_char_p]),
        "saber_set_gemm_2sm": (None, [I]),
        "saber_set_gemm_2sm_persistent": (None, [I]),
        "saber_get_gemm_2sm": (I, []),
        "saber_gemm_w8_2sm_ok": (I, [C.POINTER(GemmI8Params)]),
        "saber_gemm_w8_2sm_launch": (I, [C.POINTER(GemmI8Params), I, S]),
        "saber_moe_route_launch": (I, [C.POINTER(MoeRouteParams), S]),
        "saber_moe_combine_launch": (I, [C.POINTER(MoeCombineParams), S]),
        "saber_moe_gather_launch": (I, [P, P, I, P, P, P, P, I, I, I, I, S]),
        "saber_program_add_moe_gather": (I, [P, P, P, I, P, P, P, P, I, I, I, I, C.c_char_p]),
        "saber_program_add_moe_route": (I, [P, C.POINTER(MoeRouteParams), C.c_char_p]),
        "saber_program_add_moe_combine": (I, [P, C.POINTER(MoeCombineParams), C.c_char_p]),
        "saber_vis_rows_launch": (I, [C.POINTER(VisRowsParams), S]),
        "saber_vis_pos_add_launch": (I, [C.POINTER(VisPosAddParams), S]),
        "saber_vis_attn_launch": (I, [C.POINTER(VisAttnParams), I, S]),
        "saber_vis_rope_launch": (I, [C.POINTER(VisAttnParams), I, S]),
        "saber_program_num_ops": (I, [P]),
        "saber_program_declared_launches": (I, [P]),
        "saber_program_op_tag": (C.c_char_p, [P, I]),
        "saber_program_last_failed_op": (I, [P]),
        "saber_program_run": (I, [P, S]),
        "saber_program_run_range": (I, [P, I, I, S]),
        "saber_program_capture": (I, [P, S]),
        "saber_program_replay": (I, [P, S]),
        "saber_program_captured_nodes": (I, [P]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name, None)
        if fn is None:
            continue
        fn.restype = res
        fn.argtypes = args


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    """Device pointer of a tensor (None stays a null pointer)."""
    if t is None:
        return None
    if isinstance(t, int):
        return t          # already a device address
    return t.data_ptr()


def stream_handle(stream: Optional[torch.cuda.Stream] = None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


class NativeError(RuntimeError):
    pass


def check(code: int, what: str) -> None:
    if code != 0:
        raise NativeError(f"{what}: CUDA error {code}")


class Program:
    """Native step program: fixed launch list, eager walk or graph capture + replay.

    Tensors named in parameter blocks must outlive the program; `keep()` pins references.
    """

    def __init__(self, name: str = ""):
        self.name = name
        self._L = lib()
        self._h = self._L.saber_program_create()
        self._keep: list = []
        self.captured = False

    def keep(self, *objs) -> None:
        self._keep.extend(objs)

    # ---- op builders -------------------------------------------------------------------------
    def gemm(self, p: GemmI8Params, stages: int = 0, tag: str = "gemm") -> int:
        return self._L.saber_program_add_gemm(self._h, C.byref(p), stages, tag.encode())

    def link_prefetch(self, pref_bytes: int = 96 * 1024) -> int:
        """Chain the program's GEMMs so that each asks L2 for the next one's leading weight tiles."""
        return self._L.saber_program_link_prefetch(self._h, int(pref_bytes))

    def row(self, mode: int, p: RowOpParams, tag: str = "row") -> int:
        return self._L.saber_program_add_row(self._h, mode, C.byref(p), tag.encode())

    def embed(self, table, ids, out, M, H, vocab_lo, vocab_n, ldout=0, tag="embed") -> int:
        return self._L.saber_program_add_embed(self._h, ptr(table), ptr(ids), ptr(out), M, H,
                                               vocab_lo, vocab_n, ldout, tag.encode())

    def expand(self, ctx, tok, pos, out, nseq, block, H, tag="block_expand") -> int:
        return self._L.saber_program_add_expand(self._h, ptr(ctx), ptr(tok), ptr(pos), ptr(out),
                                                nseq, block, H, tag.encode())

    def advance(self, seq_base, by: int, tag="comm_advance") -> int:
        return self._L.saber_program_add_advance(self._h, ptr(seq_base), by, tag.encode())

    def gdn_conv(self, p: GdnConvParams, nseq: int, tag="gdn_conv") -> int:
        return self._L.saber_program_add_gdn_conv(self._h, C.byref(p), nseq, tag.encode())

    def gdn_step(self, p: GdnStepParams, nseq: int, tag="gdn_step") -> int:
        return self._L.saber_program_add_gdn_step(self._h, C.byref(p), nseq, tag.encode())

    def gdn_rec(self, p: GdnRecParams, nseq: int, vs: int, tag="gdn_rec") -> int:
        return self._L.saber_program_add_gdn_rec(self._h, C.byref(p), nseq, vs, tag.encode())

    def rope(self, p: RopeKvParams, tag="rope_kv") -> int:
        return self._L.saber_program_add_rope(self._h, C.byref(p), tag.encode())

    def attn(self, p: AttnParams, tag="attn") -> int:
        return self._L.saber_program_add_attn(self._h, C.byref(p), tag.encode())

    def argmax(self, logits, rows, ld, V, id_offset, idx, val, tag="argmax") -> int:
        return self._L.saber_program_add_argmax(self._h, ptr(logits), rows, ld, V, id_offset,
                                                ptr(idx), ptr(val), tag.encode())

    def sample_seam(self, ids, vals, samp, u, picks, rows, tag="sample_seam") -> int:
        return self._L.saber_program_add_sample_seam(self._h, ptr(ids), ptr(vals), ptr(samp), ptr(u), ptr(picks), rows, tag.encode())

    def logit_gather(self, logits, rows, ld, V, id_offset, ids, out, tag="logit_gather") -> int:
        return self._L.saber_program_add_logit_gather(self._h, ptr(logits), rows, ld, V, id_offset,
                                                      ptr(ids), ptr(out), tag.encode())

    def seam(self, logits, rows, ld, V, id_offset, temps, ids, vals, lse, tag="seam") -> int:
        return self._L.saber_program_add_seam(self._h, ptr(logits), rows, ld, V, id_offset,
                                              ptr(temps), ptr(ids), ptr(vals), ptr(lse), tag.encode())

    def draft_index(self, p: "DraftIndexParams", tag="draft_index") -> int:
        return self._L.saber_program_add_draft_index(self._h, C.byref(p), tag.encode())

    def verify(self, p: VerifyParams, tag="verify") -> int:
        return self._L.saber_program_add_verify(self._h, C.byref(p), tag.encode())

    def memset(self, t: torch.Tensor, value: int = 0, tag="memset") -> int:
        return self._L.saber_program_add_memset(self._h, ptr(t), value, t.numel() * t.element_size(),
                                                tag.encode())

    def copy(self, dst: torch.Tensor, src: torch.Tensor, tag="copy") -> int:
        nbytes = src.numel() * src.element_size()
        return self._L.saber_program_add_copy(self._h, ptr(dst), ptr(src), nbytes, tag.encode())

    def seam_merge(self, p: "SeamMergeParams", tag="seam_merge") -> int:
        return self._L.saber_program_add_seam_merge(self._h, C.byref(p), tag.encode())

    def pick_merge(self, p: "PickMergeParams", tag="pick_merge") -> int:
        return self._L.saber_program_add_pick_merge(self._h, C.byref(p), tag.encode())

    def allreduce(self, p: AllReduceParams, tag="allreduce") -> int:
        return self._L.saber_program_add_allreduce(self._h, C.byref(p), tag.encode())

    def gdn_chunk(self, p: "GdnRecParams", nseq: int, max_rows: int, scratch, tag: str = "gdn_chunk") -> int:
        return self._L.saber_program_add_gdn_chunk(self._h, C.byref(p), nseq, max_rows, ptr(scratch), tag.encode())

    def digest(self, buf, nbytes: int, out_word, tag: str = "digest") -> int:
        """XOR-splitmix digest of `nbytes` of `buf` into the 8-byte word at `out_word` (cleared by digest_clear)."""
        return self._L.saber_program_add_digest(self._h, ptr(buf), nbytes, ptr(out_word), tag.encode())

    def digest_clear(self, out, n: int, tag: str = "digest_clear") -> int:
        return self._L.saber_program_add_digest_clear(self._h, ptr(out), n, tag.encode())

    def add_moe_route(self, p: "MoeRouteParams", tag: str = "moe_route") -> int:
        return self._L.saber_program_add_moe_route(self._h, C.byref(p), tag.encode())

    def add_moe_gather(self, src, src_row, ntiles, dst, rows_cap: int, tag: str = "moe_gather", to_fp8: bool = False) -> int:
        """src / dst: objects with .q (tiled int8), .scale, .M_pad, .K (QuantAct); to_fp8: the sorted rows
        leave as e4m3 (MXFP4 experts multiply fp8 x fp8)."""
        return self._L.saber_program_add_moe_gather(self._h, ptr(src.q), ptr(src.scale), src.M_pad, ptr(src_row),
                                                    ptr(ntiles), ptr(dst.q), ptr(dst.scale), rows_cap, dst.M_pad,
                                                    src.K, int(to_fp8), tag.encode())

    def add_moe_combine(self, p: "MoeCombineParams", tag: str = "moe_combine") -> int:
        return self._L.saber_program_add_moe_combine(self._h, C.byref(p), tag.encode())

    # ---- execution ---------------------------------------------------------------------------
    @property
    def num_ops(self) -> int:
        return self._L.saber_program_num_ops(self._h)

    @property
    def declared_launches(self) -> int:
        return self._L.saber_program_declared_launches(self._h)

    def tags(self) -> list[str]:
        return [self._L.saber_program_op_tag(self._h, i).decode() for i in range(self.num_ops)]

    def run(self, stream: Optional[torch.cuda.Stream] = None, first: int = 0, last: int = -1) -> None:
        code = self._L.saber_program_run_range(self._h, first, last, stream_handle(stream))
        if code != 0:
            i = self._L.saber_program_last_failed_op(self._h)
            tag = self._L.saber_program_op_tag(self._h, i).decode()
            raise NativeError(f"program {self.name!r}: op {i} ({tag}) failed with CUDA error {code}")

    def capture(self, stream: torch.cuda.Stream) -> int:
        """Capture into a CUDA graph; returns the node count and asserts it equals the declared one."""
        n = self._L.saber_program_capture(self._h, stream.cuda_stream)
        if n < 0:
            raise NativeError(f"program {self.name!r}: capture failed with CUDA error {-n}")
        if n != self.declared_launches:
            raise NativeError(
                f"program {self.name!r}: captured {n} nodes but ops declared {self.declared_launches}")
        self.captured = True
        return n

    def replay(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        check(self._L.saber_program_replay(self._h, stream_handle(stream)), f"replay {self.name!r}")

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self._L.saber_program_destroy(self._h)
                self._h = None
        except Exception:
            pass
