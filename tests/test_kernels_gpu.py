"""Native sm_100a kernels (row producers, GDN, attention, head, step program) against plain PyTorch
fp32 references of the same ops."""
import math

import pytest
import torch

from saber_engine_b200.ops import functional as F
from saber_engine_b200.ops import layouts as L
from saber_engine_b200.ops import native as N
from saber_engine_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check_quant(qa: F.QuantAct, h_ref: torch.Tensor):
    """The tiled int8 output must dequantise to the bf16 row within half a quantisation step."""
    q = L.untile_act_int8(qa.q.cpu(), qa.M)
    s = qa.scale.cpu()[: qa.M]
    amax = h_ref.abs().amax(1)
    assert torch.allclose(s, amax / 127, rtol=1e-2, atol=1e-8)
    deq = q.float() * s[:, None]
    assert (deq - h_ref).abs().max() <= 0.51 * s.max() + 2e-2 * h_ref.abs().max()
    # padding rows are zero
    if qa.M_pad > qa.M:
        assert int(qa.q[:, qa.M:, :].abs().max().item()) == 0


def test_add_rms_quant():
    torch.manual_seed(0)
    M, K = 9, 5120
    x = torch.randn(M, K).to(torch.bfloat16)
    res = torch.randn(M, K).to(torch.bfloat16)
    w = torch.randn(K) * 0.1
    res_ref, n_ref = R.add_rms(x, res, w)
    res_d = res.to(DEV)
    qa, out = F.add_rms_quant(x.to(DEV), res_d, w.to(DEV), want_out=True)
    torch.cuda.synchronize()
    assert torch.allclose(res_d.float().cpu(), res_ref.float(), atol=2e-2, rtol=1e-2)
    assert torch.allclose(out.float().cpu(), n_ref, atol=3e-2, rtol=2e-2)
    _check_quant(qa, out.float().cpu())


def test_silu_mul_and_gate_and_plain_quant():
    torch.manual_seed(1)
    M, K = 5, 1024
    gu = torch.randn(M, 2 * K).to(torch.bfloat16)
    qa, out = F.silu_mul_quant(gu.to(DEV), want_out=True)
    ref = R.silu_mul(gu)
    assert torch.allclose(out.float().cpu(), ref, atol=2e-2, rtol=2e-2)
    _check_quant(qa, out.float().cpu())
    a = torch.randn(M, K).to(torch.bfloat16)
    g = torch.randn(M, K).to(torch.bfloat16)
    qa, out = F.gate_sigmoid_quant(a.to(DEV), g.to(DEV), want_out=True)
    assert torch.allclose(out.float().cpu(), R.gate_sigmoid(a, g), atol=2e-2, rtol=2e-2)
    _check_quant(qa, out.float().cpu())
    qa = F.plain_quant(a.to(DEV))
    _check_quant(qa, a.float())


def test_gdn_norm_quant():
    torch.manual_seed(2)
    M, H = 7, 6
    o = torch.randn(M, H * 128)
    z = torch.randn(M, H * 128).to(torch.bfloat16)
    w = torch.rand(128) + 0.5
    qa, out = F.gdn_norm_quant(o.to(DEV), z.to(DEV), w.to(DEV), want_out=True)
    ref = R.gdn_gated_norm(o, z, w)
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=2e-2)
    _check_quant(qa, out.float().cpu())


def test_embed_and_argmax_and_seam():
    torch.manual_seed(3)
    V, H = 1000, 256
    table = torch.randn(V, H).to(torch.bfloat16).to(DEV)
    ids = torch.tensor([3, 999, 0, 1200], dtype=torch.int32, device=DEV)
    out = F.embed_gather(table, ids)
    assert torch.equal(out[0], table[3]) and torch.equal(out[1], table[999])
    assert float(out[3].abs().max()) == 0.0
    logits = torch.randn(6, 4096).to(torch.bfloat16)
    logits[2, 17] = float("nan")
    logits[4, 100] = logits[4, 50] = 30.0   # tie: lower id wins
    idx, val = F.argmax(logits.to(DEV))
    lf = logits.float().nan_to_num(nan=-1e30)
    assert idx.cpu().tolist()[:4] == lf.argmax(1).tolist()[:4]
    assert idx[4].item() == 50 and val[4].item() == 30.0
    temps = torch.tensor([1.0, 0.7, 0.5, 2.0, 1.0, 1.3])
    sid, sval, lse = F.topk_seam(logits.to(DEV), temps.to(DEV))
    tv, ti = torch.topk(lf, 64, dim=1)
    assert torch.allclose(sval.cpu(), tv, atol=0, rtol=0)
    for r in (0, 1, 3, 5):   # ids name the values they claim (ties at the cut may pick other ids)
        ids_r = sid[r].cpu().long()
        assert len(set(ids_r.tolist())) == 64
        assert torch.equal(lf[r][ids_r], sval[r].cpu())
    lse1 = torch.logsumexp(lf, 1)
    lseT = torch.logsumexp(lf / temps[:, None], 1)
    assert torch.allclose(lse[:, 0].cpu(), lse1, atol=1e-2)
    assert torch.allclose(lse[:, 1].cpu(), lseT, atol=2e-2)


def test_verify_accept_greedy_and_oracle():
    cu = torch.tensor([0, 5, 10, 15], dtype=torch.int32, device=DEV)
    draft = torch.tensor([1, 2, 3, 4, 5, 9, 8, 7, 6, 5, 4, 4, 4, 4, 4], dtype=torch.int32, device=DEV)
    target = torch.tensor([2, 3, 9, 9, 9, 8, 7, 6, 5, 1, 0, 0, 0, 0, 0], dtype=torch.int32, device=DEV)
    uid = torch.arange(3, dtype=torch.int32, device=DEV)
    step = torch.zeros(3, dtype=torch.int32, device=DEV)
    n, toks = F.verify_accept(draft, target, cu, uid, step, 5)
    assert n.cpu().tolist() == [3, 5, 1]
    assert toks[0, :3].cpu().tolist() == [2, 3, 9]
    assert toks[1, :5].cpu().tolist() == [8, 7, 6, 5, 1]
    assert toks[2, :1].cpu().tolist() == [0]
    counts = []
    for s in range(200):
        step.fill_(s)
        n, _ = F.verify_accept(draft, target, cu, uid, step, 5, oracle_p=0.75, seed=1234)
        counts += n.cpu().tolist()
    mean = sum(counts) / len(counts)
    expect = 1 + sum(0.75 ** k for k in range(1, 5))
    assert abs(mean - expect) < 0.25, (mean, expect)
    n2, _ = F.verify_accept(draft, target, cu, uid, step, 5, oracle_p=0.75, seed=1234)
    assert torch.equal(n, n2)   # seeded: same (seed, uid, step) -> same draw


def _gdn_setup(nseq, W, HV=6, HK=2, seed=0):
    torch.manual_seed(seed)
    n_q = n_k = HK * 128
    Cc = n_q + n_k + HV * 128
    conv_w = torch.randn(Cc, 4) * 0.5
    A_log = torch.randn(HV) * 0.5
    dt_bias = torch.randn(HV) * 0.5
    nslots = nseq + 1
    hist = torch.randn(nslots, 3 + W, Cc).to(torch.bfloat16)
    state = torch.randn(nslots, HV, 128, 128) * 0.1
    return dict(n_q=n_q, n_k=n_k, C=Cc, HV=HV, HK=HK, conv_w=conv_w, A_log=A_log, dt_bias=dt_bias,
                hist=hist, state=state, nslots=nslots)


@pytest.mark.parametrize("vs", [1, 2, 4])
def test_gdn_decode_replay_matches_sequential_reference(vs):
    nseq, W = 2, 5
    s = _gdn_setup(nseq, W)
    HV, HK, n_q, n_k, Cc = s["HV"], s["HK"], s["n_q"], s["n_k"], s["C"]
    dev = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in s.items()}
    stash = torch.zeros(s["nslots"], W, HV, vs, F.gdn_stash_stride(vs), device=DEV)
    slots = torch.tensor([1, 2], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, W, 2 * W], dtype=torch.int32, device=DEV)
    accepted = [3, 1]   # rows of step 1 that get committed, per sequence

    def step(xba, shift):
        x = xba.to(DEV)
        sh = torch.tensor(shift, dtype=torch.int32, device=DEV)
        qkv = F.gdn_conv(x, dev["conv_w"], dev["hist"], cu, slots, sh, n_q, n_k)
        o = F.gdn_recurrent(qkv, x[:, Cc:], dev["A_log"], dev["dt_bias"], dev["state"], stash, cu,
                            slots, sh, n_q, n_k, HV, HK, vs=vs)
        torch.cuda.synchronize()
        return o.cpu()

    x1 = (torch.randn(nseq * W, Cc + 2 * HV)).to(torch.bfloat16)
    x2 = (torch.randn(nseq * W, Cc + 2 * HV)).to(torch.bfloat16)
    o1 = step(x1, [0, 0])
    o2 = step(x2, accepted)

    for b in range(nseq):
        slot = b + 1
        win = s["hist"][slot, :3].float()
        S0 = s["state"][slot]
        r1 = x1[b * W:(b + 1) * W].float()
        q1, allx = R.gdn_conv_step(r1[:, :Cc], win, s["conv_w"], n_q, n_k)
        ref1, states1 = R.gdn_recurrent_step(S0, q1, r1[:, Cc:Cc + HV], r1[:, Cc + HV:], s["A_log"],
                                             s["dt_bias"], n_q, n_k, HV, HK)
        assert torch.allclose(o1[b * W:(b + 1) * W], ref1, atol=2e-3, rtol=2e-3)
        a = accepted[b]
        win2 = allx[a:a + 3]
        S1 = states1[a - 1]
        r2 = x2[b * W:(b + 1) * W].float()
        q2, _ = R.gdn_conv_step(r2[:, :Cc], win2, s["conv_w"], n_q, n_k)
        ref2, _ = R.gdn_recurrent_step(S1, q2, r2[:, Cc:Cc + HV], r2[:, Cc + HV:], s["A_log"],
                                       s["dt_bias"], n_q, n_k, HV, HK)
        assert torch.allclose(o2[b * W:(b + 1) * W], ref2, atol=3e-3, rtol=3e-3)
        # the state in memory is the committed state after replaying `a` rows
        assert torch.allclose(dev["state"][slot].cpu(), S1, atol=2e-3, rtol=2e-3)


def test_gdn_prefill_commit_then_decode():
    nseq, W = 1, 4
    s = _gdn_setup(nseq, W, seed=5)
    HV, HK, n_q, n_k, Cc = s["HV"], s["HK"], s["n_q"], s["n_k"], s["C"]
    dev = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in s.items()}
    vs = 2
    stash = torch.zeros(s["nslots"], W, HV, vs, F.gdn_stash_stride(vs), device=DEV)
    slots = torch.tensor([1], dtype=torch.int32, device=DEV)
    T = 37
    xp = torch.randn(T, Cc + 2 * HV).to(torch.bfloat16)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    zero = torch.zeros(1, dtype=torch.int32, device=DEV)
    qkv = F.gdn_conv(xp.to(DEV), dev["conv_w"], dev["hist"], cu, slots, zero, n_q, n_k, commit=True)
    o = F.gdn_recurrent(qkv, xp.to(DEV)[:, Cc:], dev["A_log"], dev["dt_bias"], dev["state"], stash,
                        cu, slots, zero, n_q, n_k, HV, HK, commit=True, vs=vs)
    win = s["hist"][1, :3].float()
    rp = xp.float()
    qr, allx = R.gdn_conv_step(rp[:, :Cc], win, s["conv_w"], n_q, n_k)
    ref, states = R.gdn_recurrent_step(s["state"][1], qr, rp[:, Cc:Cc + HV], rp[:, Cc + HV:],
                                       s["A_log"], s["dt_bias"], n_q, n_k, HV, HK)
    assert torch.allclose(o.cpu(), ref, atol=5e-3, rtol=5e-3)
    assert torch.allclose(dev["state"][1].cpu(), states[-1], atol=5e-3, rtol=5e-3)
    assert torch.equal(dev["hist"][1, :3].cpu().float(), allx[-3:])


def test_gdn_fused_step_equals_the_three_launches_byte_for_byte():
    """conv + recurrence + gated norm + quantisation in one launch, against the separate kernels, over
    four steps with different accepted counts, a padding sequence, and a committing (prefill) step in
    the middle that has to find the current conv window."""
    nseq, W, HV, HK = 3, 5, 6, 2
    s = _gdn_setup(nseq, W, HV=HV, HK=HK, seed=11)
    n_q, n_k, Cc = s["n_q"], s["n_k"], s["C"]
    K = HV * 128
    conv_w, A_log, dt_bias = s["conv_w"].to(DEV), s["A_log"].to(DEV), s["dt_bias"].to(DEV)
    norm_w = (torch.randn(128) * 0.2 + 1.0).to(DEV)
    # reference arm: one window per slot, stash of one slice; fused arm: two windows + word
    hist_a = s["hist"].to(DEV).clone()
    hist_b = F.gdn_hist_alloc(s["nslots"], 3 + W, Cc, DEV)
    hist_b[:, :3 + W] = hist_a
    state_a, state_b = s["state"].to(DEV).clone(), s["state"].to(DEV).clone()
    stash_a = torch.zeros(s["nslots"], W, HV, 1, 260, device=DEV)
    stash_b = torch.zeros_like(stash_a)
    slots = torch.tensor([2, -1, 1], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, W, 2 * W, 3 * W], dtype=torch.int32, device=DEV)
    M = nseq * W
    ld = Cc + K + 2 * HV
    ld = (ld + 7) // 8 * 8

    def both(x, shift):
        sh = torch.tensor(shift, dtype=torch.int32, device=DEV)
        ba = x[:, Cc + K:]
        qkv = F.gdn_conv(x, conv_w, hist_a, cu, slots, sh, n_q, n_k)
        o = F.gdn_recurrent(qkv, ba, A_log, dt_bias, state_a, stash_a, cu, slots, sh, n_q, n_k, HV, HK, vs=1)
        qa_a = F.QuantAct.alloc(M, K, DEV)
        qa_a.q.zero_(); qa_a.scale.zero_()
        F._row(N.ROW_GDN_NORM, F.row_params(M, K, a_f32=o, b=x[:, Cc:], w=norm_w, eps=1e-6, qa=qa_a, ldb=ld))
        qa_b = F.QuantAct.alloc(M, K, DEV)
        qa_b.q.zero_(); qa_b.scale.zero_()
        F.gdn_step(x, x[:, Cc:], ba, conv_w, A_log, dt_bias, norm_w, hist_b, state_b, stash_b, cu, slots, sh,
                   qa_b, n_q, n_k, HV, HK, W)
        torch.cuda.synchronize()
        live = [m for m in range(M) if int(slots[m // W]) >= 0]
        assert torch.equal(qa_a.q[:, live], qa_b.q[:, live])
        assert torch.equal(qa_a.scale[live], qa_b.scale[live])
        assert torch.equal(state_a, state_b) and torch.equal(stash_a, stash_b)

    torch.manual_seed(3)
    for shift in ([0, 0, 0], [3, 0, 1], [5, 0, 2]):
        both(torch.randn(M, ld, device=DEV).to(torch.bfloat16), shift)
    # the fused arm's current window is now window 1 of both live slots
    words = hist_b[:, -1, :2].view(torch.int32).flatten().tolist()
    assert words[1] == 1 and words[2] == 1 and words[0] == 0
    # a committing step (the rows of a prompt chunk) reads the current window and leaves the new one in both
    T = 7
    xp = torch.randn(nseq * T, ld, device=DEV).to(torch.bfloat16)
    cup = torch.tensor([0, T, 2 * T, 3 * T], dtype=torch.int32, device=DEV)
    zero = torch.zeros(nseq, dtype=torch.int32, device=DEV)
    # (bring the reference arm's committed state up to date first: its replay happens in the next launch)
    qa_ = F.gdn_conv(xp, conv_w, hist_a, cup, slots, torch.tensor([1, 0, 4], dtype=torch.int32, device=DEV), n_q, n_k, commit=True)
    qb_ = F.gdn_conv(xp, conv_w, hist_b, cup, slots, torch.tensor([1, 0, 4], dtype=torch.int32, device=DEV), n_q, n_k, commit=True, dual=True)
    torch.cuda.synchronize()
    livep = [m for m in range(nseq * T) if int(slots[m // T]) >= 0]
    assert torch.equal(qa_[livep], qb_[livep])
    for slot in (1, 2):
        assert torch.equal(hist_a[slot, :3], hist_b[slot, :3]) and torch.equal(hist_a[slot, :3], hist_b[slot, 3 + W:6 + W])
    both(torch.randn(M, ld, device=DEV).to(torch.bfloat16), [0, 0, 0])


_LAST_GOT = []


def _attn_case(ctx_lens, rows, splits, nq=12, nkv=2, seed=0, impl=0, tol=3e-2, window=0):
    torch.manual_seed(seed)
    nseq = len(ctx_lens)
    M = sum(rows)
    ld = nq * 256 * 2 + 2 * nkv * 256
    q_off, k_off, v_off = 0, nq * 256 * 2, nq * 256 * 2 + nkv * 256
    qkv = torch.randn(M, ld).to(torch.bfloat16)
    qw, kw = torch.randn(256) * 0.1, torch.randn(256) * 0.1
    max_blocks = max((c + r + 15) // 16 for c, r in zip(ctx_lens, rows))
    nblocks = nseq * max_blocks + 3
    perm = torch.randperm(nblocks)[: nseq * max_blocks].reshape(nseq, max_blocks).to(torch.int32)
    k_hist = [torch.randn(c, nkv, 256) * 0.7 for c in ctx_lens]
    v_hist = [torch.randn(c, nkv, 256) * 0.7 for c in ctx_lens]
    cache = torch.zeros(nblocks, nkv, 2, 16, 256, dtype=torch.uint8)
    cache_f8 = cache.view(torch.float8_e4m3fn)
    for b in range(nseq):
        if ctx_lens[b]:
            t = torch.arange(ctx_lens[b])
            blk = perm[b, t // 16].long()
            cache[blk, :, 0, t % 16] = k_hist[b].to(torch.float8_e4m3fn).view(torch.uint8)
            cache[blk, :, 1, t % 16] = v_hist[b].to(torch.float8_e4m3fn).view(torch.uint8)
    pos = torch.zeros(3, M, dtype=torch.int32)
    slot_map = torch.zeros(M, dtype=torch.int32)
    cu = [0]
    for b in range(nseq):
        for r in range(rows[b]):
            m = cu[-1] + r
            t = ctx_lens[b] + r
            pos[:, m] = t
            slot_map[m] = int(perm[b, t // 16]) * 16 + t % 16
        cu.append(cu[-1] + rows[b])
    cu_t = torch.tensor(cu, dtype=torch.int32)
    kv_len = torch.tensor([c + r for c, r in zip(ctx_lens, rows)], dtype=torch.int32)
    from saber_engine_b200.ops import layouts as L
    cache_d = (L.kv_pages_to_core(cache) if impl == 1 else cache).to(DEV)     # the tcgen05 kernel's page order
    q_out = F.rope_kv(qkv.to(DEV), qw.to(DEV), kw.to(DEV), pos.to(DEV), slot_map.to(DEV), cache_d,
                      nq, nkv, q_off, k_off, v_off, page_layout=impl)
    out = F.attention(q_out, cache_d, perm.to(DEV), cu_t.to(DEV), kv_len.to(DEV), nkv,
                      max(rows), splits=splits, impl=impl, window=window)
    torch.cuda.synchronize()
    F.scratch(DEV).check()
    # reference
    qf = qkv.float()
    q_ref = R.qk_norm_rope(qf[:, :nq * 256].reshape(M, nq, 256), qw, pos)
    k_new = R.qk_norm_rope(qf[:, k_off:k_off + nkv * 256].reshape(M, nkv, 256), kw, pos)
    v_new = qf[:, v_off:].reshape(M, nkv, 256)
    assert torch.allclose(q_out.float().cpu(), R.bf16_round(q_ref), atol=3e-2, rtol=3e-2)
    for b in range(nseq):
        sl = slice(cu[b], cu[b + 1])
        kk = torch.cat([R.fp8_round(k_hist[b]), R.fp8_round(k_new[sl])], 0)
        vv = torch.cat([R.fp8_round(v_hist[b]), R.fp8_round(v_new[sl])], 0)
        ref = R.attention_rows(R.bf16_round(q_ref[sl]), kk, vv, int(kv_len[b]), window=window)
        got = out[sl].float().cpu()
        err = (got - ref).abs().max().item()
        _LAST_GOT.append((got, ref))
        assert err < tol * max(1.0, ref.abs().max().item()), f"seq {b}: max err {err}"


def test_attention_decode_single_and_split():
    _attn_case([100, 37, 513], [5, 5, 5], splits=1)
    _attn_case([100, 37, 513], [5, 5, 5], splits=4, seed=1)
    _attn_case([0], [9], splits=1, seed=2)           # no history: only this step's rows


def test_attention_tcgen05_decode_at_131072_tokens_of_context():
    """One sequence, 131,072 tokens of history in 8,192 scattered pages, a width-8 decode step over 32 key
    segments, against the fp32 restatement."""
    _attn_case([131072], [8], splits=32, impl=1, tol=5e-2, seed=3)


def test_attention_tcgen05_decode_prefill_and_splits():
    """The tcgen05 kernel (fp8 operand legs: Q and the probabilities are e4m3 like the pages) against
    the fp32 restatement."""
    tol = 5e-2          # of the largest output value: the probabilities carry three mantissa bits (half an ulp = 6%)
    _attn_case([100, 37, 513], [5, 5, 5], splits=1, impl=1, tol=tol)
    _attn_case([100, 37, 513], [5, 5, 5], splits=4, seed=1, impl=1, tol=tol)
    _attn_case([0], [9], splits=1, seed=2, impl=1, tol=tol)
    _attn_case([64, 300], [8, 8], splits=2, nq=24, nkv=4, seed=3, impl=1, tol=tol)
    _attn_case([0, 50], [40, 33], splits=1, nq=12, nkv=2, seed=4, impl=1, tol=tol)       # prefill: several query tiles
    _attn_case([700], [1], splits=3, nq=16, nkv=2, seed=5, impl=1, tol=tol)             # GQA 8, one row
    _attn_case([1500, 20], [16, 3], splits=1, nq=6, nkv=2, seed=6, impl=1, tol=tol)     # GQA 3


def test_attention_27b_geometry_and_prefill_rows():
    _attn_case([64, 300], [9, 9], splits=2, nq=24, nkv=4, seed=3)
    _attn_case([0, 50], [40, 33], splits=1, nq=12, nkv=2, seed=4)   # prefill: several q tiles


def test_program_capture_replay_counts_nodes():
    torch.manual_seed(7)
    M, K, Nn = 9, 512, 256
    w = torch.randn(Nn, K) * 0.02
    qw = F.QuantWeight.from_float(w, 4, DEV)
    x = torch.randn(M, K).to(torch.bfloat16).to(DEV)
    nw = torch.zeros(K, device=DEV)
    qa = F.QuantAct.alloc(M, K, DEV)
    out = torch.zeros(M, Nn, dtype=torch.bfloat16, device=DEV)
    prog = N.Program("t")
    prog.row(N.ROW_ADD_RMS, F.row_params(M, K, a=x, w=nw, w_offset=1.0, qa=qa), tag="norm")
    prog.gemm(F.gemm_params(qw, qa, out, F.scratch(DEV), splits=2), tag="gemm")
    prog.keep(x, nw, qa, out, qw)
    prog.run()
    torch.cuda.synchronize()
    eager = out.clone()
    out.zero_()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        assert prog.capture(st) == 2 == prog.declared_launches
        prog.replay(st)
    st.synchronize()
    assert torch.equal(out, eager)
    _, n_ref = R.add_rms(x.cpu(), None, nw.cpu())
    wq, ws = L.quantize_weight_rows(w, 4)
    aq, asc = L.quantize_act_rows(n_ref)
    ref = R.gemm_i8(wq, ws, aq, asc).float()
    assert (out.float().cpu() - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-3


def test_gdn_chunked_prefill_equals_row_by_row_kernel():
    """The 64-row chunked form against the row-by-row kernel (commit mode): same outputs and the
    same final state up to summation order, on two ragged sequences (one not a chunk multiple)."""
    HV, HK = 6, 2
    s = _gdn_setup(2, 4, HV=HV, HK=HK, seed=9)
    n_q, n_k, Cc = s["n_q"], s["n_k"], s["C"]
    lens = [150, 64]
    M = sum(lens)
    torch.manual_seed(10)
    qk = torch.nn.functional.normalize(torch.randn(M, 2 * HK, 128), dim=-1).reshape(M, n_q + n_k)
    qk[:, :n_q] /= 128 ** 0.5
    qkv = torch.cat([qk, torch.randn(M, HV * 128)], 1).to(DEV)
    ba = torch.randn(M, 2 * HV).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0, lens[0], M], dtype=torch.int32, device=DEV)
    slots = torch.tensor([1, 2], dtype=torch.int32, device=DEV)
    sh = torch.zeros(2, dtype=torch.int32, device=DEV)
    A_log, dtb = s["A_log"].to(DEV), s["dt_bias"].to(DEV)
    st_a, st_b = s["state"].to(DEV).clone(), s["state"].to(DEV).clone()
    stash = torch.zeros(3, 4, HV, 2, F.gdn_stash_stride(2), device=DEV)
    want = F.gdn_recurrent(qkv, ba, A_log, dtb, st_a, stash, cu, slots, sh, n_q, n_k, HV, HK, commit=True, vs=2)
    got = F.gdn_chunked(qkv, ba, A_log, dtb, st_b, stash, cu, slots, sh, n_q, n_k, HV, HK, max_rows=max(lens))
    st_c = s["state"].to(DEV).clone()
    rows8 = F.gdn_recurrent(qkv, ba, A_log, dtb, st_c, stash, cu, slots, sh, n_q, n_k, HV, HK, commit=True, prefill_rows=True)
    torch.cuda.synchronize()
    # the eight-threads-per-row prefill form: same rule, another summation order
    assert (rows8 - want).abs().max().item() <= 2e-4 * want.abs().max().item() + 1e-5
    assert (st_a[1:] - st_c[1:]).abs().max().item() <= 2e-4 * st_a.abs().max().item() + 1e-5
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() <= 2e-4 * scale + 1e-5, ((got - want).abs().max().item(), scale)
    assert (st_a[1:] - st_b[1:]).abs().max().item() <= 2e-4 * st_a.abs().max().item() + 1e-5
    assert torch.equal(st_a[0], st_b[0])            # the padding slot is untouched
    # the tensor-core form (tf32 pair products, tcgen05 scan with the state in tensor memory): bf16 operands,
    # fp32 accumulation -- the state copy that feeds a chunk's products is rounded once per chunk
    st_d = s["state"].to(DEV).clone()
    got_tc = F.gdn_chunked(qkv, ba, A_log, dtb, st_d, stash, cu, slots, sh, n_q, n_k, HV, HK, max_rows=max(lens), impl=1)
    torch.cuda.synchronize()
    F.scratch(DEV).check()
    err_o = (got_tc - want).abs().max().item()
    err_s = (st_a[1:] - st_d[1:]).abs().max().item()
    assert err_o <= 1.5e-2 * scale + 1e-4, (err_o, scale)
    assert err_s <= 1.5e-2 * st_a.abs().max().item() + 1e-4, (err_s, st_a.abs().max().item())
    assert torch.equal(st_a[0], st_d[0])
    rms = (got_tc - want).pow(2).mean().sqrt().item() / want.pow(2).mean().sqrt().item()
    assert rms <= 5e-3, rms


def test_gdn_tensor_core_prefill_split_at_a_chunk_boundary_gives_the_same_bytes():
    """The tensor-core chunked form carries the state in tensor memory between chunks and in fp32 memory
    between launches: 256 rows in one launch and as 128 + 128 rows are the same arithmetic, bit for bit
    (what the prefix cache relies on when it resumes at a multiple of 64 rows), and so is a second run."""
    HV, HK = 6, 2
    s = _gdn_setup(2, 4, HV=HV, HK=HK, seed=19)
    n_q, n_k = s["n_q"], s["n_k"]
    M = 256
    torch.manual_seed(20)
    qk = torch.nn.functional.normalize(torch.randn(M, 2 * HK, 128), dim=-1).reshape(M, n_q + n_k)
    qk[:, :n_q] /= 128 ** 0.5
    qkv = torch.cat([qk, torch.randn(M, HV * 128)], 1).to(DEV)
    ba = torch.randn(M, 2 * HV).to(torch.bfloat16).to(DEV)
    slots = torch.tensor([1], dtype=torch.int32, device=DEV)
    sh = torch.zeros(1, dtype=torch.int32, device=DEV)
    A_log, dtb = s["A_log"].to(DEV), s["dt_bias"].to(DEV)
    stash = torch.zeros(3, 4, HV, 2, F.gdn_stash_stride(2), device=DEV)

    def run(pieces):
        st = s["state"].to(DEV).clone()
        outs = []
        for lo, hi in pieces:
            cu = torch.tensor([0, hi - lo], dtype=torch.int32, device=DEV)
            outs.append(F.gdn_chunked(qkv[lo:hi].contiguous(), ba[lo:hi].contiguous(), A_log, dtb, st, stash, cu, slots, sh,
                                      n_q, n_k, HV, HK, max_rows=hi - lo, impl=1))
        torch.cuda.synchronize()
        return torch.cat(outs), st

    o1, s1 = run([(0, 256)])
    o2, s2 = run([(0, 256)])
    o3, s3 = run([(0, 128), (128, 256)])
    F.scratch(DEV).check()
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    assert torch.equal(o1, o3) and torch.equal(s1, s3)


def test_attention_sliding_window_on_the_tensor_core_kernel():
    """A row sees its last `window` keys only: pages below the first row's window are skipped, the rows' own
    lower bounds are masked inside the first tile; decode (with and without splits) and a prefill tile."""
    _attn_case([700, 37, 1500], [5, 5, 5], splits=1, impl=1, window=256, seed=31)
    _attn_case([700, 37, 1500], [4, 4, 4], splits=3, impl=1, window=100, seed=32)      # a window that is no page multiple
    # prefill rows: the window slides inside the tile (128 keys per row: the e4m3 probabilities average over fewer terms)
    _attn_case([900], [200], splits=1, impl=1, window=128, seed=33, nq=6, nkv=1, tol=5e-2)
    _attn_case([50], [6], splits=1, impl=1, window=2048, seed=34)                      # a window longer than the context is no window


def test_attention_packs_several_heads_into_one_tile():
    """Few rows per sequence: 2 heads per 16-row tile at 8 rows, 3 at 5, all 6 at 1 or 2 rows."""
    _attn_case([200, 31], [8, 8], splits=2, nq=24, nkv=4, seed=5)
    _attn_case([77, 300, 16], [1, 1, 1], splits=1, nq=12, nkv=2, seed=6)
    _attn_case([77, 300, 16], [1, 1, 1], splits=3, nq=24, nkv=4, seed=7)
    _attn_case([40, 90, 130], [5, 3, 1], splits=2, nq=12, nkv=2, seed=8)    # ragged: packing stride = widest sequence
    _attn_case([64, 64], [2, 2], splits=1, nq=16, nkv=2, seed=9)            # group of 8 heads, 2 rows: 8 heads per tile


def test_device_draw_equals_the_host_sampler_on_the_same_candidates():
    import ctypes as C
    from saber_engine_b200.ops import native as N
    from saber_engine_b200.serve.engine_api import SamplingParams
    from saber_engine_b200.serve.sampler import sample_candidates
    g = torch.Generator().manual_seed(0)
    rows, K = 96, 64
    vals = torch.sort(torch.randn(rows, K, generator=g) * 3.0, dim=1, descending=True).values.contiguous()
    ids = torch.stack([torch.randperm(5000, generator=g)[:K] for _ in range(rows)]).to(torch.int32)
    u = torch.rand(rows, generator=g)
    settings = [(1.0, 0, 1.0, 0.0), (0.7, 5, 1.0, 0.0), (1.3, 0, 0.8, 0.0), (1.0, 0, 1.0, 0.1), (0.9, 20, 0.9, 0.02), (0.0, 0, 1.0, 0.0)]
    samp = torch.tensor([settings[r % len(settings)] for r in range(rows)], dtype=torch.float32)
    picks = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    d = [t.cuda() for t in (ids, vals, samp, u)]
    N.check(N.lib().saber_sample_seam_launch(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
                                             picks.data_ptr(), rows, N.stream_handle()), "sample_seam")
    got = picks.cpu().tolist()
    agree = 0
    for r in range(rows):
        T, k, p, mp = settings[r % len(settings)]
        if T == 0.0:
            assert got[r] == -7                       # greedy rows keep their pick
            continue
        want, _ = sample_candidates(ids[r].tolist(), vals[r].tolist(), SamplingParams(temperature=T, top_k=k, top_p=p, min_p=mp),
                                    [], [], float(u[r]))
        agree += int(want == got[r])
    assert agree >= 78            # fp32 on the device, double on the host: a draw at a boundary may differ


def test_draft_block_index_tables():
    """Positions, KV slots and attention lengths of the drafter's block rows, against the plain statement."""
    import ctypes as C
    import numpy as np
    from saber_engine_b200.ops import native as N
    nseq, B, max_blocks, page, M = 3, 4, 8, 16, 20
    cu = np.array([0, 5, 5, 20], dtype=np.int32)               # the middle sequence is a padding slot (no rows)
    kv_len = np.array([37, 0, 110], dtype=np.int32)             # sequence 2: block rows 110 .. 113 cross into the page that is not there
    acc = np.array([2, 0, 19], dtype=np.int32)                 # last committed rows: row 2 of sequence 0, the last row of sequence 2
    pos = np.arange(3 * M, dtype=np.int32).reshape(3, M) * 3 + 7
    bt = np.zeros((nseq, max_blocks), dtype=np.int32)
    bt[0, :4] = [5, 9, 2, 11]
    bt[2, :8] = [20, 21, 22, 23, 24, 25, 26, 0]                # the eighth page is not allocated
    dev = lambda a: torch.from_numpy(a).to(DEV)
    t = dict(pos=dev(pos.reshape(-1)), cu=dev(cu), kv=dev(kv_len), acc=dev(acc), bt=dev(bt.reshape(-1)))
    R = nseq * B
    pos_o = torch.full((3 * R,), -7, dtype=torch.int32, device=DEV)
    slot_o = torch.full((R,), -7, dtype=torch.int32, device=DEV)
    len_o = torch.full((nseq,), -7, dtype=torch.int32, device=DEV)
    p = N.DraftIndexParams()
    p.pos, p.cu_rows, p.kv_len, p.acc_row, p.block_table = (t[k].data_ptr() for k in ("pos", "cu", "kv", "acc", "bt"))
    p.pos_out, p.slot_out, p.kv_len_out = pos_o.data_ptr(), slot_o.data_ptr(), len_o.data_ptr()
    p.M, p.nseq, p.block, p.max_blocks, p.page_tokens = M, nseq, B, max_blocks, page
    N.check(N.lib().saber_draft_index_launch(C.byref(p), N.stream_handle()), "draft_index")
    torch.cuda.synchronize()
    want_pos, want_slot, want_len = np.zeros((3, R), np.int32), np.full(R, -1, np.int32), np.zeros(nseq, np.int32)
    for b in range(nseq):
        if cu[b + 1] == cu[b]:
            continue
        at = kv_len[b] - (cu[b + 1] - acc[b])                   # sequence index of the committed row
        want_len[b] = at + 1 + B
        for j in range(B):
            tpos = at + 1 + j
            want_pos[:, b * B + j] = pos[:, acc[b]] + 1 + j
            blk = bt[b, tpos // page] if tpos // page < max_blocks else 0
            want_slot[b * B + j] = blk * page + tpos % page if blk > 0 else -1
    assert np.array_equal(pos_o.cpu().numpy().reshape(3, R), want_pos)
    assert np.array_equal(slot_o.cpu().numpy(), want_slot)
    assert np.array_equal(len_o.cpu().numpy(), want_len)
