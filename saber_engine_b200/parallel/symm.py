"""Symmetric heap over NVLink peer memory and the parameter blocks of the fused TP paths.

Every rank allocates the same regions at the same offsets of one device allocation, exports it with
CUDA IPC, and maps every peer's allocation; kernels then store straight into peers and signal with
system-scope flags.  `torch.distributed` (NCCL) is used for bootstrap only: exchanging the 64-byte
IPC handles and a protocol digest that must agree on every rank before anything launches.

Parity: `crates/saber-exec/src/peer.rs:8-15,140` (IPC handle exchange + ProtocolDigest agreement:
a boot-time disagreement is a refusal, not a hang), `crates/saber-exec/src/tp2.rs:468`
(agree_on_collectives).  New here: up to 8 ranks, sequence-numbered slots, and the GEMM-epilogue
push that makes the all-reduce part of the GEMM and of the following norm kernel.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import json
from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import native as N


class _Raw:
    """A raw device allocation seen through the CUDA array interface (zero-copy torch view)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _raw_tensor(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_Raw(ptr, nbytes), device=device)


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


@dataclass
class HeapLayout:
    nranks: int
    rows_max: int
    hidden: int
    gemm_recv: int = 0
    gemm_flags: int = 0
    ar_recv: int = 0
    ar_flags: int = 0
    pick_win: int = 0
    pick_flags: int = 0
    seam_win: int = 0      # [2 parity][nranks][rows_max][130 words] sampling candidates of the other ranks
    seam_flags: int = 0
    ag_q: int = 0          # all-gathered quantised activations [hidden / 128][rows_pad][128] bytes
    ag_scale: int = 0      # [rows_pad] fp32
    ag_flags: int = 0      # [2 parity][64 row tiles] arrival flags
    ag_counter: int = 0    # [64 row tiles] rows-done counters (local use)
    rows_pad: int = 0
    total: int = 0

    @staticmethod
    def make(nranks: int, rows_max: int, hidden: int, ar_max_elems: int) -> "HeapLayout":
        L = HeapLayout(nranks, rows_max, hidden)
        off = 0
        def take(n):
            nonlocal off
            o = off
            off = _align(off + n)
            return o
        L.gemm_recv = take(2 * nranks * rows_max * hidden * 2)
        L.gemm_flags = take(2 * nranks * N.TP_MAX_TILES * 4)
        L.ar_recv = take(2 * nranks * ar_max_elems * 2)
        L.ar_flags = take(2 * nranks * N.AR_BLOCKS * 4)
        L.pick_win = take(2 * nranks * rows_max * 8)
        L.pick_flags = take(2 * nranks * 4)
        L.seam_win = take(2 * nranks * rows_max * 130 * 4)
        L.seam_flags = take(2 * nranks * 4)
        L.rows_pad = (rows_max + 127) // 128 * 128
        L.ag_q = take(L.rows_pad * max(128, (hidden + 127) // 128 * 128))
        L.ag_scale = take(L.rows_pad * 4)
        L.ag_flags = take(2 * 64 * 4)
        L.ag_counter = take(64 * 4)
        L.total = off
        L.ar_max_elems = ar_max_elems
        return L

    def digest(self) -> str:
        d = {k: getattr(self, k) for k in ("nranks", "rows_max", "hidden", "gemm_recv", "gemm_flags", "ar_recv",
                                            "ar_flags", "pick_win", "pick_flags", "seam_win", "seam_flags", "ag_q", "ag_scale", "ag_flags",
                                            "ag_counter", "total")}
        d["protocol"] = "saber-b200-symm/3"
        return hashlib.sha256(json.dumps(d, sort_keys=True).encode()).hexdigest()


class SymmetricComm:
    def __init__(self, rank: int, nranks: int, device, max_elems: int, rows_max: Optional[int] = None,
                 hidden: Optional[int] = None, bases: Optional[list] = None, own_base: Optional[int] = None):
        """max_elems: largest all-reduce message (elements); rows_max x hidden: largest GEMM output.
        `bases`/`own_base` are only given by `local_group` (several emulated ranks in one process)."""
        self.rank, self.nranks, self.device = rank, nranks, torch.device(device)
        hidden = hidden or 1
        rows_max = rows_max or max(1, max_elems // hidden)
        self.layout = HeapLayout.make(nranks, rows_max, hidden, max_elems)
        self._L = N.lib()
        self._owned = []
        if bases is None:
            torch.cuda.set_device(self.device)
            own = self._malloc(self.layout.total)
            bases = self._exchange(own)
        else:
            own = own_base
        self.bases = bases
        self.own = own
        self.seq_base = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.sites = 0

    # ---- allocation / bootstrap
    def _malloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        N.check(self._L.saber_dev_malloc(C.byref(p), nbytes), "symmetric heap allocation")
        N.check(self._L.saber_dev_memset(p, 0, nbytes), "symmetric heap clear")
        self._owned.append(p.value)
        return p.value

    def _exchange(self, own: int) -> list:
        import torch.distributed as dist
        handle = (C.c_char * 64)()
        N.check(self._L.saber_ipc_get_handle(own, handle), "cudaIpcGetMemHandle")
        mine = {"rank": self.rank, "handle": bytes(handle), "digest": self.layout.digest()}
        everyone = [None] * self.nranks
        dist.all_gather_object(everyone, mine)
        bad = [e["rank"] for e in everyone if e["digest"] != mine["digest"]]
        if bad:
            raise RuntimeError(f"rank {self.rank}: protocol digest disagrees with ranks {bad}; refusing to launch")
        bases = []
        for e in everyone:
            if e["rank"] == self.rank:
                bases.append(own)
            else:
                p = C.c_void_p()
                N.check(self._L.saber_ipc_open_handle(e["handle"], C.byref(p)), f"open IPC handle of rank {e['rank']}")
                bases.append(p.value)
        dist.barrier()
        return bases

    @staticmethod
    def local_group(nranks: int, device, max_elems: int, rows_max: int, hidden: int) -> list:
        """`nranks` emulated ranks in ONE process on ONE device (tests): every rank gets its own heap
        and sees the others through ordinary device pointers."""
        lay = HeapLayout.make(nranks, rows_max, hidden, max_elems)
        L = N.lib()
        bases = []
        for _ in range(nranks):
            p = C.c_void_p()
            N.check(L.saber_dev_malloc(C.byref(p), lay.total), "heap")
            N.check(L.saber_dev_memset(p, 0, lay.total), "clear")
            bases.append(p.value)
        group = [SymmetricComm(r, nranks, device, max_elems, rows_max, hidden, bases=list(bases), own_base=bases[r])
                 for r in range(nranks)]
        group[0]._owned = list(bases)
        return group

    # ---- parameter blocks
    def gemm_tp(self, p: N.GemmI8Params, site: int) -> None:
        """Turn a row-parallel GEMM into GEMM + push-to-all-ranks (its `out` is no longer written)."""
        lay = self.layout
        for r in range(self.nranks):
            p.tp_recv[r] = self.bases[r] + lay.gemm_recv
            p.tp_flags[r] = self.bases[r] + lay.gemm_flags
        p.tp_seq_base = self.seq_base.data_ptr()
        p.tp_nranks, p.tp_rank, p.tp_site = self.nranks, self.rank, site
        p.tp_rows, p.tp_ld = lay.rows_max, lay.hidden

    # ---- sequence-parallel building blocks (reduce-scatter epilogue, all-gather by peer stores)
    def heap_qact(self, M: int, K: int):
        """The all-gather target as a QuantAct: tiled int8 rows + scales living in THIS rank's heap at
        the same offset on every rank, so that owners can store their rows into every rank's copy."""
        from ..ops.functional import QuantAct
        lay = self.layout
        assert K <= max(128, (lay.hidden + 127) // 128 * 128) and M <= lay.rows_max and K % 128 == 0
        q = _raw_tensor(self.own + lay.ag_q, (K // 128) * lay.rows_pad * 128, self.device).view(torch.int8)
        sc = _raw_tensor(self.own + lay.ag_scale, lay.rows_pad * 4, self.device).view(torch.float32)
        return QuantAct(q.reshape(K // 128, lay.rows_pad, 128), sc, M, K)

    def gemm_rs(self, p: N.GemmI8Params, site: int, rows_per_rank: int) -> None:
        """Row-parallel GEMM whose epilogue reduce-scatters: a row's partial goes to its owner only."""
        self.gemm_tp(p, site)
        p.tp_rpr = rows_per_rank

    def gemm_ag(self, p: N.GemmI8Params, site: int) -> None:
        """A GEMM whose token rows arrive by all-gather: wait per 128-row tile for the owners' flags."""
        p.ag_flags = self.own + self.layout.ag_flags
        p.ag_seq_base = self.seq_base.data_ptr()
        p.ag_site = site
        p.err = self.err.data_ptr()

    def row_sp(self, p: N.RowOpParams, site: int, nt: int, tiles_n: int, rows_per_rank: int) -> None:
        """ADD_RMS on the rows this rank owns; the quantised rows go to every rank's heap_qact."""
        self.row_tp(p, site, nt, tiles_n)
        lay = self.layout
        for r in range(self.nranks):
            p.sp_q[r] = self.bases[r] + lay.ag_q
            p.sp_scale[r] = self.bases[r] + lay.ag_scale
            p.sp_flags[r] = self.bases[r] + lay.ag_flags
        p.sp_counter = self.own + lay.ag_counter
        p.sp_rpr, p.sp_rank = rows_per_rank, self.rank

    def row_tp(self, p: N.RowOpParams, site: int, nt: int, tiles_n: int) -> None:
        """Make an ADD_RMS producer the consumer of the GEMM pushed at `site`."""
        lay = self.layout
        p.tp_recv = self.own + lay.gemm_recv
        p.tp_flags = self.own + lay.gemm_flags
        p.tp_seq_base = self.seq_base.data_ptr()
        p.err = self.err.data_ptr()
        p.tp_nranks, p.tp_site, p.tp_rows, p.tp_ld = self.nranks, site, lay.rows_max, lay.hidden
        p.tp_nt, p.tp_tiles_n = nt, tiles_n

    def allreduce_params(self, inp: torch.Tensor, out: torch.Tensor, n_elems: int, site: int) -> N.AllReduceParams:
        lay = self.layout
        p = N.AllReduceParams()
        p.inp, p.out = inp.data_ptr(), out.data_ptr()
        for r in range(self.nranks):
            p.peer_recv[r] = self.bases[r] + lay.ar_recv
            p.peer_flags[r] = self.bases[r] + lay.ar_flags
        p.seq_base, p.err = self.seq_base.data_ptr(), self.err.data_ptr()
        p.n_elems, p.max_elems, p.site, p.nranks, p.rank = n_elems, lay.ar_max_elems, site, self.nranks, self.rank
        p.spin_limit_us = 0
        return p

    def seam_merge_params(self, ids: torch.Tensor, vals: torch.Tensor, lse: torch.Tensor, rows: int, site: int) -> N.SeamMergeParams:
        """Swap and merge the ranks' sampling candidates (64 per head row and shard) on the device."""
        lay = self.layout
        p = N.SeamMergeParams()
        p.ids, p.vals, p.lse = ids.data_ptr(), vals.data_ptr(), lse.data_ptr()
        for r in range(self.nranks):
            p.peer_win[r] = self.bases[r] + lay.seam_win
            p.peer_flags[r] = self.bases[r] + lay.seam_flags
        p.seq_base, p.err = self.seq_base.data_ptr(), self.err.data_ptr()
        p.rows, p.rows_max, p.site, p.nranks, p.rank = rows, lay.rows_max, site, self.nranks, self.rank
        return p

    def pick_merge_params(self, idx: torch.Tensor, val: torch.Tensor, rows: int, site: int) -> N.PickMergeParams:
        lay = self.layout
        p = N.PickMergeParams()
        p.idx, p.val = idx.data_ptr(), val.data_ptr()
        for r in range(self.nranks):
            p.peer_win[r] = self.bases[r] + lay.pick_win
            p.peer_flags[r] = self.bases[r] + lay.pick_flags
        p.seq_base, p.err = self.seq_base.data_ptr(), self.err.data_ptr()
        p.rows, p.rows_max, p.site, p.nranks, p.rank = rows, lay.rows_max, site, self.nranks, self.rank
        return p

    def check(self) -> None:
        code = int(self.err.item())
        if code:
            self.err.zero_()
            raise N.NativeError(f"rank {self.rank}: a peer wait ran out ({N.ERR_NAMES.get(code, code)})")

    def close(self) -> None:
        for r, b in enumerate(self.bases):
            if b not in self._owned and b is not None and r != self.rank and not getattr(self, "_local", False):
                try:
                    self._L.saber_ipc_close(b)
                except Exception:
                    pass
        for p in self._owned:
            self._L.saber_dev_free(p)
        self._owned = []
