"""`sp-gate`: the sequence-parallel chain across real GPUs -- row-parallel GEMM with a reduce-scatter
epilogue, add-norm-quant on the owned rows with an all-gather by peer stores, next GEMM waiting on the
arrival flags -- checked against a CPU restatement and timed against the push-to-all-ranks chain the
decode path uses.  Run under torchrun, one rank per GPU:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29551 \\
        -m saber_engine_b200.parallel.sp_gate --rows 2048

Timing: CUDA events on the launching stream around `--iters` repetitions of the three-kernel chain,
after a warm-up and a barrier, max over ranks.  Roofline of one chain: weights of both GEMMs / HBM
bandwidth against the bytes a rank sends (reduce-scatter bf16 partials + all-gather int8 rows) / link
bandwidth.

Parity: the reference's `arnq` fusions (`crates/saber-kernels/hip/macaq_iu8f.hip:1-12`: GEMM + 2-rank
all-reduce + add-RMSNorm + quant in one launch) are the 2-rank, all-reduce form of this chain.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import layouts as L
from ..ops import native as N
from ..ops import reference as R
from .symm import SymmetricComm


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--k-full", type=int, default=17408, help="reduction dim of the row-parallel GEMM (unsharded)")
    ap.add_argument("--n2", type=int, default=4096, help="output features per rank of the GEMM after the all-gather")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--check-rows", type=int, default=64, help="rows compared against the CPU restatement")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    M, H = a.rows, a.hidden
    Kr = a.k_full // world // 128 * 128
    rpr = M // world
    assert M % (128 * world) == 0, "rows must split into whole 128-row tiles per rank"
    comm = SymmetricComm(rank, world, dev, max_elems=M * H, rows_max=M, hidden=H)
    g = torch.Generator().manual_seed(3)                      # every rank draws the same tensors
    w_full = torch.randn(H, Kr * world, generator=g) * 0.02
    x_full = torch.randn(M, Kr * world, generator=g)
    w2 = torch.randn(a.n2, H, generator=g) * 0.02
    res = torch.randn(M, H, generator=g).to(torch.bfloat16)
    nw = torch.randn(H, generator=g) * 0.1
    wq_full, ws_full = L.quantize_weight_rows(w_full, 4)
    ks = slice(rank * Kr, (rank + 1) * Kr)
    qw1 = F.QuantWeight.from_int(wq_full[:, ks].contiguous(), ws_full, 4, dev)
    qa1 = F.plain_quant(x_full[:, ks].to(torch.bfloat16).to(dev))
    qw2 = F.QuantWeight.from_float(w2, 4, dev)
    sc = F.scratch(dev)
    lib = N.lib()
    stream = torch.cuda.current_stream()
    dummy = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
    nt = L.token_tile(M)

    def chain(mode: str, out: torch.Tensor, res_d: torch.Tensor, site: int):
        p1 = F.gemm_params(qw1, qa1, dummy, sc, splits=1)
        qa_mid = comm.heap_qact(M, H) if mode == "sp" else qa_plain
        pr = F.row_params(M, H, a=None, res=res_d, w=nw_d, w_offset=1.0, qa=qa_mid)
        p2 = F.gemm_params(qw2, qa_mid, out, sc, splits=1)
        if mode == "sp":
            comm.gemm_rs(p1, site, rpr)
            comm.row_sp(pr, site, nt, L.round_up(H, 256) // 256, rpr)
            comm.gemm_ag(p2, site)
        else:
            comm.gemm_tp(p1, site)
            comm.row_tp(pr, site, nt, L.round_up(H, 256) // 256)
        N.check(lib.saber_gemm_i8_launch(C.byref(p1), 0, N.stream_handle()), "gemm 1")
        N.check(lib.saber_row_producer_launch(N.ROW_ADD_RMS, C.byref(pr), N.stream_handle()), "add-norm-quant")
        N.check(lib.saber_gemm_i8_launch(C.byref(p2), 0, N.stream_handle()), "gemm 2")

    nw_d = nw.to(dev)
    qa_plain = F.QuantAct.alloc(M, H, dev)
    report = {"world": world, "rows": M, "hidden": H, "k_per_rank": Kr, "n2": a.n2}
    results = {}
    for mode in ("all", "sp"):
        out = torch.zeros(M, a.n2, dtype=torch.bfloat16, device=dev)
        times = []
        for it in range(a.iters + 2):
            res_d = res.to(dev).clone()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            chain(mode, out, res_d, 0)
            N.check(lib.saber_comm_advance_launch(comm.seq_base.data_ptr(), 1, N.stream_handle()), "advance")
            e1.record(stream)
            torch.cuda.synchronize()
            if it >= 2:
                times.append(e0.elapsed_time(e1))
        sc.check()
        comm.check()
        t = torch.tensor([sorted(times)[len(times) // 2]], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[mode] = (float(t.item()), out.float().cpu())
        report[f"{mode}_ms"] = float(t.item())
    # ---- check a few rows against the CPU restatement of the tensor-parallel arithmetic
    rows = slice(0, a.check_rows)
    acc = torch.zeros(a.check_rows, H)
    for r in range(world):
        kk = slice(r * Kr, (r + 1) * Kr)
        aq, asc = L.quantize_act_rows(x_full[rows, kk])
        acc += R.gemm_i8(wq_full[:, kk], ws_full, aq, asc).float()
    _, n_ref = R.add_rms(R.bf16_round(acc), res[rows], nw)
    aq2, asc2 = L.quantize_act_rows(n_ref)
    want = R.gemm_i8(*L.quantize_weight_rows(w2, 4), aq2, asc2).float()
    ok = True
    for mode in ("all", "sp"):
        err = (results[mode][1][rows] - want).abs().max().item()
        report[f"{mode}_max_err"] = err
        ok = ok and err <= 0.05 * want.abs().max().item() + 1e-3
    report["sp_equals_all"] = bool(torch.equal(results["sp"][1], results["all"][1]))
    sent_all = (world - 1) * M * H * 2
    sent_sp = (world - 1) * rpr * H * 2 + (world - 1) * rpr * H
    report["bytes_sent_per_rank"] = {"all": sent_all, "sp": sent_sp}
    hbm_us = (qw1.tiles.numel() + qw2.tiles.numel()) / 6.5e12 * 1e6
    mma_us = 2.0 * M * (H * Kr + a.n2 * H) / 4.5e15 * 1e6
    report["roofline_us"] = {"weights_hbm": hbm_us, "int8_tensor_peak": mma_us, "link_all": sent_all / 770e9 * 1e6,
                             "link_sp": sent_sp / 770e9 * 1e6}
    gathered = [None] * world
    dist.all_gather_object(gathered, ok)
    report["pass"] = all(gathered)
    if rank == 0:
        print(json.dumps(report), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if report["pass"] else 1


if __name__ == "__main__":
    sys.exit(main())
