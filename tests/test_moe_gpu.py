"""Mixture-of-experts path on the GPU: routing / placement against the PyTorch law, the whole block
(router -> route -> gather -> grouped GEMMs -> combine) against the fp32 oracle, and the MoE hybrid
model end to end (prefill logits vs oracle, speculative == greedy)."""
import pytest
import torch

from saber_engine_b200.models import config as C
from saber_engine_b200.ops import functional as F
from saber_engine_b200.ops import layouts as L
from saber_engine_b200.ops import native as N

pytestmark = pytest.mark.gpu

MOE = C.MoEConfig(n_experts=32, top_k=4, expert_inter=128, shared_inter=128)


def _cfg(**kw):
    return C.scaled_hybrid(name="hybrid-mini-moe", moe=MOE, **kw)


def _moe_layer(cfg, seed=3):
    from saber_engine_b200.models.moe_weights import random_moe_layer
    g = torch.Generator(device="cuda").manual_seed(seed)
    return random_moe_layer(cfg, 1, 0, torch.device("cuda"), g, 0.02)


@pytest.mark.parametrize("M", [1, 9, 72, 300])
def test_route_placement(M):
    from saber_engine_b200.models.moe_block import MoeWorkspace, route_params
    from saber_engine_b200.models.reference_hybrid import moe_route_ref
    cfg = _cfg()
    ws = MoeWorkspace(cfg, MOE.n_experts, M, "cuda", 0)
    g = torch.Generator().manual_seed(M)
    logits = (torch.randn(M, MOE.n_experts, generator=g) * 2).to(torch.bfloat16)
    ws.logits[:, : MOE.n_experts] = logits.cuda()
    prog = N.Program("route")
    prog.add_moe_route(route_params(ws, cfg, 0))
    for _ in range(2):                 # twice: the counts must come back to zero by themselves
        prog.run()
    torch.cuda.synchronize()
    ids, wts = moe_route_ref(logits.float(), MOE.top_k, True)
    assert torch.equal(ws.topk_id.cpu().long(), ids)
    assert torch.allclose(ws.topk_w.cpu(), wts, rtol=2e-3, atol=1e-6)
    # placement: every route sits inside its expert's segment and points back at its token
    counts = torch.bincount(ids.flatten(), minlength=MOE.n_experts)
    offs = ws.offsets.cpu()
    padded = (counts + 15) // 16 * 16
    assert torch.equal(offs[1:] - offs[:-1], padded.int())
    slot = ws.slot_of.cpu().long()
    src = ws.src_row.cpu()
    assert len(set(slot.flatten().tolist())) == M * MOE.top_k
    for m in range(M):
        for k in range(MOE.top_k):
            e, s = int(ids[m, k]), int(slot[m, k])
            assert offs[e] <= s < offs[e] + counts[e]
            assert int(src[s]) == m
    total = int(padded.sum())
    assert int(ws.ntiles.cpu()[1]) == total
    live = src[:total] >= 0
    assert int(live.sum()) == M * MOE.top_k
    # tile table covers every live row exactly once
    nt_live = int(ws.ntiles.cpu()[0])
    tiles = ws.tiles.cpu()[:nt_live]
    covered = torch.zeros(total, dtype=torch.int32)
    for e, r0, rows, _ in tiles.tolist():
        assert offs[e] <= r0 and r0 + rows <= offs[e] + counts[e] and r0 % 16 == 0 and 0 < rows <= ws.nt
        covered[r0:r0 + rows] += 1
    assert torch.equal(covered.bool(), live) and int(covered.max()) == 1
    assert int(ws.counts.abs().sum()) == 0


@pytest.mark.parametrize("M,fmt", [(5, "iu8"), (72, "iu8"), (200, "iu8"), (5, "mxfp4"), (200, "mxfp4")])
def test_moe_block_matches_oracle(M, fmt):
    """fmt = mxfp4: the routed experts are MXFP4 (e2m1 / e8m0 per 32) and their rows fp8 e4m3, made from the
    layer's int8 rows by the gather; router and shared expert stay integer."""
    import dataclasses
    from saber_engine_b200.models.moe_block import MoeWorkspace, add_moe_ops
    from saber_engine_b200.models.reference_hybrid import moe_mlp_ref
    cfg = _cfg() if fmt == "iu8" else C.scaled_hybrid(name="hybrid-mini-moe-mx", moe=dataclasses.replace(MOE, expert_format="mxfp4"))
    moe = _moe_layer(cfg)
    H = cfg.hidden
    g = torch.Generator().manual_seed(100 + M)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16)
    qa = F.plain_quant(x.cuda())
    ws = MoeWorkspace(cfg, MOE.n_experts, M, "cuda", moe["shared_inter"])
    out = torch.zeros(M, H, dtype=torch.bfloat16, device="cuda")
    prog = N.Program("moe")
    add_moe_ops(prog, ws, cfg, moe, qa, out, F.scratch("cuda"), "L0.moe")
    prog.run()
    torch.cuda.synchronize()
    F.scratch("cuda").check()
    assert moe["gate_up"].mx == (fmt == "mxfp4")
    ref = moe_mlp_ref(cfg, moe, x.float())
    got = out.float().cpu()
    err = (got - ref).abs().max()
    # (fp8 rows: a silu output that sits on a rounding edge moves one e4m3 step, 6 %, in one of the 128 terms)
    assert err <= (0.02 if fmt == "iu8" else 0.04) * ref.abs().max() + 1e-4, (float(err), float(ref.abs().max()))
    # graph replay gives the same bytes as the eager walk
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        assert prog.capture(st) == prog.declared_launches
        out.zero_()
        prog.replay(st)
    st.synchronize()
    assert torch.equal(out.float().cpu(), got)


def test_moe_model_prefill_and_spec_decode():
    from saber_engine_b200.models.hybrid import HybridModel, SeqStep, run_bucket
    from saber_engine_b200.models.reference_hybrid import forward_full
    cfg = _cfg()
    model = HybridModel(cfg, device="cuda", max_seqs=4, max_ctx=512, max_width=5, seed=1)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    blocks = list(range(1, 33))
    model.reset_slot(1)
    pb = model.build_bucket("prefill", 1, 48)
    res = run_bucket(model, pb, [SeqStep(prompt, 0, 1, 0, blocks)])
    got = pb.logits[0, : cfg.vocab].float().cpu()
    ref = forward_full(cfg, model.w, torch.tensor(prompt))["logits"][-1]
    assert (got - ref).abs().max() < 0.05 * ref.abs().max() + 1e-3

    def decode(slot, blocks, first, drafts, width, steps=16):
        out, pos, shift, k = [first], len(prompt), 0, 0
        b = model.build_bucket("decode", 1, width)
        while len(out) < steps:
            rows = [out[-1]] + list(drafts[: width - 1])
            r = run_bucket(model, b, [SeqStep(rows, pos, slot, shift, blocks, uid=3, step_no=k)])
            out += r.tokens[0]
            pos += r.n_commit[0]
            shift, drafts, k = r.n_commit[0], r.drafts[0], k + 1
        return out[:steps]

    plain = decode(1, blocks, res.tokens[0][0], [], 1)
    model.reset_slot(2)
    b2 = list(range(40, 72))
    res2 = run_bucket(model, pb, [SeqStep(prompt, 0, 2, 0, b2)])
    assert res2.tokens == res.tokens
    assert decode(2, b2, res2.tokens[0][0], res2.drafts[0], 5) == plain
    model.scratch.check()


@pytest.mark.parametrize("nranks,M", [(2, 9), (4, 72)])
def test_expert_parallel_combine_push(nranks, M):
    """Expert parallelism on ONE GPU with emulated ranks: every rank routes the replicated rows,
    runs its own experts and pushes its partial sums into every rank's receive region; afterwards
    every rank's add-norm sums the ranks.  All producers run before any consumer."""
    import ctypes as Ct
    from saber_engine_b200.models.moe_block import MoeWorkspace, add_moe_ops
    from saber_engine_b200.models.moe_weights import random_moe_layer
    from saber_engine_b200.models.reference_hybrid import moe_mlp_ref
    from saber_engine_b200.ops import reference as R
    from saber_engine_b200.parallel.symm import SymmetricComm
    cfg = _cfg()
    H = cfg.hidden
    full = _moe_layer(cfg, seed=11)
    group = SymmetricComm.local_group(nranks, "cuda", max_elems=128 * H, rows_max=128, hidden=H)
    for g_ in group:
        g_._local = True
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(M, H, generator=gen).to(torch.bfloat16)
    res = torch.randn(M, H, generator=gen).to(torch.bfloat16)
    nw = torch.randn(H, generator=gen) * 0.1
    qa = F.plain_quant(x.cuda())
    sc = F.scratch("cuda")
    keep, nts = [], []
    for r, comm in enumerate(group):
        gg = torch.Generator(device="cuda").manual_seed(11)
        moe = random_moe_layer(cfg, nranks, r, torch.device("cuda"), gg, 0.02)
        ws = MoeWorkspace(cfg, moe["e_n"], M, "cuda", moe["shared_inter"])
        dummy = torch.zeros(M, H, dtype=torch.bfloat16, device="cuda")
        prog = N.Program(f"moe-r{r}")
        nts.append(add_moe_ops(prog, ws, cfg, moe, qa, dummy, sc, "moe", comm, 0))
        prog.run()
        keep.append((moe, ws, dummy, prog))
    torch.cuda.synchronize()
    sc.check()
    ref_delta = moe_mlp_ref(cfg, full, x.float(), tp=nranks)
    res_ref, n_ref = R.add_rms(ref_delta, res, nw)
    first = None
    for r, comm in enumerate(group):
        res_d = res.cuda().clone()
        qa_out = F.QuantAct.alloc(M, H, "cuda")
        normed = torch.zeros(M, H, dtype=torch.bfloat16, device="cuda")
        p = F.row_params(M, H, a=None, res=res_d, w=nw.cuda(), w_offset=1.0, qa=qa_out, out=normed)
        comm.row_tp(p, 0, nts[r], H // 256)
        N.check(N.lib().saber_row_producer_launch(N.ROW_ADD_RMS, Ct.byref(p), N.stream_handle()), "consumer")
        torch.cuda.synchronize()
        comm.check()
        assert torch.allclose(res_d.float().cpu(), res_ref.float(), atol=3e-2, rtol=2e-2), r
        if first is None:
            first = normed.clone()
        else:
            assert torch.equal(normed, first)
    group[0].close()


def test_mxfp4_hybrid_prefill_matches_oracle_and_spec_equals_greedy():
    """The dense hybrid with MXFP4 linears (fp8 activations) end to end."""
    import dataclasses
    from saber_engine_b200.models.hybrid import HybridModel, SeqStep, run_bucket
    from saber_engine_b200.models.reference_hybrid import forward_full
    cfg = dataclasses.replace(C.scaled_hybrid(name="hybrid-mini-mx"), weight_format="mxfp4")
    model = HybridModel(cfg, device="cuda", max_seqs=2, max_ctx=512, max_width=5, seed=2)
    assert model.w.layers[0].mixer_in.mx and not model.w.lm_head.mx
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    blocks = list(range(1, 33))
    model.reset_slot(1)
    pb = model.build_bucket("prefill", 1, 48)
    res = run_bucket(model, pb, [SeqStep(prompt, 0, 1, 0, blocks)])
    got = pb.logits[0, : cfg.vocab].float().cpu()
    ref = forward_full(cfg, model.w, torch.tensor(prompt))["logits"][-1]
    assert (got - ref).abs().max() < 0.06 * ref.abs().max() + 1e-3

    def decode(slot, blk, first, drafts, width, steps=14):
        out, pos, shift, k = [first], len(prompt), 0, 0
        b = model.build_bucket("decode", 1, width)
        while len(out) < steps:
            rows = [out[-1]] + list(drafts[: width - 1])
            r = run_bucket(model, b, [SeqStep(rows, pos, slot, shift, blk, uid=3, step_no=k)])
            out += r.tokens[0]
            pos += r.n_commit[0]
            shift, drafts, k = r.n_commit[0], r.drafts[0], k + 1
        return out[:steps]

    plain = decode(1, blocks, res.tokens[0][0], [], 1)
    model.reset_slot(2)
    b2 = list(range(40, 72))
    res2 = run_bucket(model, pb, [SeqStep(prompt, 0, 2, 0, b2)])
    assert decode(2, b2, res2.tokens[0][0], res2.drafts[0], 5) == plain
    model.scratch.check()


def test_hadamard_rotated_activations_match_oracle():
    """act_hadamard: the row producers rotate (sign, 32-point Hadamard) before they quantise, the
    weights are rotated the same way; logits follow the oracle that restates the rotation."""
    import dataclasses
    from saber_engine_b200.models.hybrid import HybridModel, SeqStep, run_bucket
    from saber_engine_b200.models.reference_hybrid import forward_full
    from saber_engine_b200.ops import layouts as LL
    # the kernel's rotation alone: quantised bytes of a rotated row
    x = torch.randn(7, 512).to(torch.bfloat16)
    sign = (torch.randint(0, 2, (512,)).float() * 2 - 1)
    qa = F.QuantAct.alloc(7, 512, "cuda")
    qa.had_sign = sign.cuda()
    F._row(N.ROW_PLAIN, F.row_params(7, 512, a=x.cuda(), qa=qa))
    torch.cuda.synchronize()
    want = LL.hadamard32_rows(x.float(), sign).to(torch.bfloat16).float()
    assert torch.allclose(qa.scale[:7].cpu(), want.abs().amax(1) / 127.0, rtol=1e-2, atol=1e-6)
    cfg = dataclasses.replace(C.scaled_hybrid(name="hybrid-mini-had"), act_hadamard=True)
    model = HybridModel(cfg, device="cuda", max_seqs=2, max_ctx=512, max_width=5, seed=2)
    assert model.w.layers[0].mixer_in.had_sign is not None
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    model.reset_slot(1)
    pb = model.build_bucket("prefill", 1, 48)
    run_bucket(model, pb, [SeqStep(prompt, 0, 1, 0, list(range(1, 33)))])
    got = pb.logits[0, : cfg.vocab].float().cpu()
    ref = forward_full(cfg, model.w, torch.tensor(prompt))["logits"][-1]
    assert (got - ref).abs().max() < 0.06 * ref.abs().max() + 1e-3
    model.scratch.check()
