"""End-to-end hybrid model on the GPU: native programs vs the plain PyTorch oracle, graph == eager,
speculative decoding == plain greedy decoding, chunked prefill == one-shot prefill."""
import pytest
import torch

from saber_engine_b200.models import config as C
from saber_engine_b200.models.hybrid import HybridModel, SeqStep, run_bucket

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model():
    cfg = C.scaled_hybrid()
    return HybridModel(cfg, device="cuda", max_seqs=4, max_ctx=512, max_width=5, seed=1)


def _blocks(seq_index, n=32):
    return list(range(1 + seq_index * n, 1 + (seq_index + 1) * n))


def _prefill(model, prompt, slot, blocks, chunks=None, eager=False):
    model.reset_slot(slot)
    pos, res = 0, None
    for n in (chunks or [len(prompt)]):
        b = model.build_bucket("prefill", 1, 48)
        res = run_bucket(model, b, [SeqStep(prompt[pos:pos + n], pos, slot, 0, blocks)], eager=eager)
        pos += n
    return res


def _decode(model, prompt, first, drafts, slot, blocks, steps, width, eager=False):
    out = [first]
    shift, pos = 0, len(prompt)
    b = model.build_bucket("decode", 1, width)
    n_steps = 0
    while len(out) < steps:
        rows = [out[-1]] + list(drafts[:width - 1])
        res = run_bucket(model, b, [SeqStep(rows, pos, slot, shift, blocks, uid=7, step_no=n_steps)], eager=eager)
        n = res.n_commit[0]
        out += res.tokens[0]
        pos += n
        shift = n
        drafts = res.drafts[0]
        n_steps += 1
    return out[:steps], n_steps


def test_prefill_logits_match_oracle(model):
    from saber_engine_b200.models.reference_hybrid import forward_full
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, model.cfg.vocab, (40,), generator=g).tolist()
    res = _prefill(model, prompt, 1, _blocks(0))
    b = model.buckets[("prefill", 1, 48)]
    got = b.logits[0, : model.cfg.vocab].float().cpu()
    ref = forward_full(model.cfg, model.w, torch.tensor(prompt))["logits"][-1]
    assert (got - ref).abs().max() < 0.05 * ref.abs().max() + 1e-3
    assert res.tokens[0][0] == int(ref.argmax()) or (ref.max() - ref[res.tokens[0][0]]) < 0.02 * ref.abs().max()


def test_spec_decode_equals_plain_greedy_and_graph_equals_eager(model):
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, model.cfg.vocab, (37,), generator=g).tolist()
    r = _prefill(model, prompt, 1, _blocks(0))
    plain, n_plain = _decode(model, prompt, r.tokens[0][0], [], 1, _blocks(0), 20, 1)
    r2 = _prefill(model, prompt, 2, _blocks(1))
    assert r2.tokens == r.tokens
    spec, n_spec = _decode(model, prompt, r2.tokens[0][0], r2.drafts[0], 2, _blocks(1), 20, 5)
    assert spec == plain
    assert n_spec <= n_plain
    r3 = _prefill(model, prompt, 3, _blocks(2), eager=True)
    eager, _ = _decode(model, prompt, r3.tokens[0][0], r3.drafts[0], 3, _blocks(2), 20, 5, eager=True)
    assert eager == plain


def test_chunked_prefill_equals_one_shot(model):
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, model.cfg.vocab, (45,), generator=g).tolist()
    a = _prefill(model, prompt, 1, _blocks(0))
    b = _prefill(model, prompt, 2, _blocks(1), chunks=[16, 20, 9])
    assert a.tokens == b.tokens


def test_batched_equals_solo(model):
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, model.cfg.vocab, (n,), generator=g).tolist() for n in (20, 33)]
    firsts, solo = [], []
    for j, p in enumerate(prompts):
        r = _prefill(model, p, j + 1, _blocks(j))
        firsts.append(r.tokens[0][0])
        solo.append(_decode(model, p, r.tokens[0][0], [], j + 1, _blocks(j), 8, 1)[0])
    for j, p in enumerate(prompts):
        _prefill(model, p, j + 1, _blocks(j))
    b = model.build_bucket("decode", 2, 1)
    outs = [[f] for f in firsts]
    pos = [len(p) for p in prompts]
    shift = [0, 0]
    for _ in range(7):
        seqs = [SeqStep([outs[j][-1]], pos[j], j + 1, shift[j], _blocks(j)) for j in range(2)]
        res = run_bucket(model, b, seqs)
        for j in range(2):
            outs[j] += res.tokens[j]
            pos[j] += 1
            shift[j] = 1
    assert outs == solo
    assert b.captured and b.program.declared_launches == b.n_launches


def test_fused_launches_equal_one_launch_per_op(model):
    """The fused decode chain (row tails, silu * mul + quant in the gate | up epilogue, weight
    prefetch) commits the same tokens and leaves the same logits as one launch per op, with fewer launches."""
    from saber_engine_b200.models.weights import random_init
    plain = HybridModel(model.cfg, device="cuda", max_seqs=4, max_ctx=512, max_width=5, seed=1, fuse=False)
    assert model.fuse and not plain.fuse
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, model.cfg.vocab, (41,), generator=g).tolist()
    outs = []
    for mdl in (model, plain):
        r = _prefill(mdl, prompt, 1, _blocks(0))
        toks, _ = _decode(mdl, prompt, r.tokens[0][0], r.drafts[0], 1, _blocks(0), 16, 5)
        outs.append((r.tokens, toks, mdl.buckets[("decode", 1, 5)].logits.clone()))
    assert outs[0][0] == outs[1][0] and outs[0][1] == outs[1][1]
    assert torch.equal(outs[0][2], outs[1][2])
    fused_n = model.buckets[("decode", 1, 5)].n_launches
    plain_n = plain.buckets[("decode", 1, 5)].n_launches
    assert fused_n < plain_n, (fused_n, plain_n)


def test_context_of_131072_tokens_prefill_decode_and_prefix_reuse():
    """One sequence of 131,072 tokens through the model in 2048-row chunks (8,192 KV pages per attention
    layer, 32 key segments per decode launch), then decode: speculative == greedy at that depth, and a
    second sequence that re-uses the first 126,976 tokens' pages and a snapshot of the recurrent state,
    prefills the rest in other chunk sizes and must produce the same tokens."""
    cfg = C.scaled_hybrid()
    T, cut = 131072, 131072 - 4096
    model = HybridModel(cfg, device="cuda", max_seqs=2, max_ctx=T + 512, max_width=5, seed=1)
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, cfg.vocab, (T,), generator=g).tolist()
    nblk = (T + 512) // cfg.page_tokens
    blocks_a = list(range(1, 1 + nblk))
    shared = cut // cfg.page_tokens
    blocks_b = blocks_a[:shared] + list(range(1 + nblk, 1 + nblk + (nblk - shared)))
    model.reset_slot(1)
    b2048 = model.build_bucket("prefill", 1, 2048)
    snap, res = None, None
    for pos in range(0, T, 2048):
        if pos == cut:
            torch.cuda.synchronize()
            snap = {i: (model.gdn_state[i][1].clone(), model.gdn_hist[i][1].clone()) for i in model.gdn_state}
        res = run_bucket(model, b2048, [SeqStep(prompt[pos:pos + 2048], pos, 1, 0, blocks_a, blocks_key=("a", 0))])
    first = res.tokens[0][0]

    def decode(slot, blocks, first, drafts, width, steps=8):
        out, shift, pos, n = [first], 0, T, 0
        b = model.build_bucket("decode", 1, width)
        while len(out) < steps:
            rows = [out[-1]] + list(drafts[:width - 1])
            r = run_bucket(model, b, [SeqStep(rows, pos, slot, shift, blocks, uid=3, step_no=n)])
            k = r.n_commit[0]
            out += r.tokens[0]
            pos, shift, drafts, n = pos + k, k, r.drafts[0], n + 1
        return out[:steps]
    # the second sequence first (slot 2): shared pages + restored state, the tail in 512-row chunks
    model.reset_slot(2)
    for i, (st, hist) in snap.items():
        model.gdn_state[i][2].copy_(st)
        model.gdn_hist[i][2].copy_(hist)
    b512 = model.build_bucket("prefill", 1, 512)
    for pos in range(cut, T, 512):
        res_b = run_bucket(model, b512, [SeqStep(prompt[pos:pos + 512], pos, 2, 0, blocks_b, blocks_key=("b", 0))])
    assert res_b.tokens[0][0] == first
    spec_b = decode(2, blocks_b, first, res_b.drafts[0], 5)
    plain_a = decode(1, blocks_a, first, [], 1)
    assert spec_b == plain_a
    model.scratch.check()


def test_a_vocabulary_head_just_over_whole_rounds_of_ctas_runs_its_last_tiles_as_a_split_gemm():
    """150 feature tiles on 148 SMs: 148 tiles fill one round, the two left over run as a GEMM of their own
    split along K -- same logits as the oracle, and the spec-decode invariant holds through both heads."""
    from saber_engine_b200.models.reference_hybrid import forward_full
    cfg = C.scaled_hybrid(name="hybrid-mini-v38400", vocab=150 * 256)
    m = HybridModel(cfg, device="cuda", max_seqs=2, max_ctx=512, max_width=5, seed=4)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    res = _prefill(m, prompt, 1, _blocks(0))
    b = m.buckets[("prefill", 1, 48)]
    tags = b.program.tags()
    assert "lm_head.whole_rounds" in tags and "lm_head.last_tiles" in tags and "draft.head.last_tiles" in tags
    got = b.logits[0, : cfg.vocab].float().cpu()
    ref = forward_full(cfg, m.w, torch.tensor(prompt))["logits"][-1]
    assert (got - ref).abs().max() < 0.05 * ref.abs().max() + 1e-3
    plain, _ = _decode(m, prompt, res.tokens[0][0], [], 1, _blocks(0), 12, 1)
    res2 = _prefill(m, prompt, 2, _blocks(1))
    spec, _ = _decode(m, prompt, res2.tokens[0][0], res2.drafts[0], 2, _blocks(1), 12, 5)
    assert spec == plain
    m.scratch.check()


def test_big_prefill_rungs_on_int8_weight_twins_give_the_same_bytes():
    """Rungs of 256 rows and more multiply with the int8 image of the 4-bit tiles (no widening pass, two token
    tiles per CTA): the same integers and scales, so logits, tokens and drafts are the same bytes."""
    cfg = C.scaled_hybrid()
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, cfg.vocab, (300,), generator=g).tolist()
    outs = []
    for w8 in (True, False):
        m = HybridModel(cfg, device="cuda", max_seqs=2, max_ctx=1024, max_width=5, seed=1, prefill_w8=w8)
        m.reset_slot(1)
        b = m.build_bucket("prefill", 1, 512)
        res = run_bucket(m, b, [SeqStep(prompt, 0, 1, 0, list(range(1, 40)))])
        assert (m.twin_bytes > 0) == w8
        outs.append((res.tokens[0], res.drafts[0], b.logits[0].float().cpu().clone()))
        m.scratch.check()
    assert outs[0][0] == outs[1][0] and outs[0][1] == outs[1][1] and torch.equal(outs[0][2], outs[1][2])


def test_drafter_attention_layers_over_the_context_kv_store_keep_the_invariants():
    """A drafter whose first layer attends over a context-KV store (written from the target's tap row of every
    context position, addressed by the target's block tables) and over its own block rows: drafts change, the
    committed tokens do not (speculative == plain greedy), and graph replay == eager walk."""
    import dataclasses
    base = C.scaled_hybrid()
    cfg = dataclasses.replace(base, name="hybrid-mini-dattn", drafter=dataclasses.replace(base.drafter, attn_layers=1))
    m = HybridModel(cfg, device="cuda", max_seqs=4, max_ctx=512, max_width=5, seed=1)
    ref = HybridModel(base, device="cuda", max_seqs=4, max_ctx=512, max_width=5, seed=1)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    res = _prefill(m, prompt, 1, _blocks(0))
    tags = m.buckets[("prefill", 1, 48)].program.tags()
    assert "draft.L0.attn.core" in tags and "draft.L0.attn.ctx_kv_append" in tags and "draft.block_index" in tags
    res_ref = _prefill(ref, prompt, 1, _blocks(0))
    assert res.tokens[0] == res_ref.tokens[0]                       # the target is the same model
    plain, _ = _decode(m, prompt, res.tokens[0][0], [], 1, _blocks(0), 14, 1)
    res2 = _prefill(m, prompt, 2, _blocks(1))
    spec, n_spec = _decode(m, prompt, res2.tokens[0][0], res2.drafts[0], 2, _blocks(1), 14, 5)
    assert spec == plain
    res3 = _prefill(m, prompt, 3, _blocks(2))
    eager, _ = _decode(m, prompt, res3.tokens[0][0], res3.drafts[0], 3, _blocks(2), 14, 5, eager=True)
    assert eager == plain
    assert int(m.draft_kv[0].abs().sum()) > 0                        # the store has been written
    m.scratch.check()
