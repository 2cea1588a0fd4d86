"""Native block-scaled FP4 GEMM (tcgen05.mma kind::mxf4nvf4 / kind::mxf4, scales in tensor memory)
against the exact fp32 dequantisation of both operands."""
import pytest
import torch

from saber_engine_b200.ops import functional as F
from saber_engine_b200.pack import quant_fp4 as Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(fmt, M, N, K, splits, seed=0):
    torch.manual_seed(seed)
    w = torch.randn(N, K) * 0.05
    w[:, ::7] *= 4.0                                  # block scales that differ a lot inside a row
    x = torch.randn(M, K)
    x[:, 5::16] *= 3.0
    if fmt == 4:
        codes, bs, g = Q.quantize_nvfp4(w)
        qw = F.QuantWeight.from_nvfp4(codes, bs, g, device=DEV)
        wd = Q.dequant_nvfp4(codes, bs, g)
    else:
        codes, e = Q.quantize_mxfp4(w)
        qw = F.QuantWeight.from_mxfp4_native(codes, e, device=DEV)
        wd = Q.dequant_mxfp4(codes, e)
    qa = F.quant_act_fp4(x, fmt, device=DEV)
    vs = 16 if fmt == 4 else 32
    sf = (qa.sf.cpu(), None)
    # exact dequantisation of the activations from what the quantiser kept
    xc = Q.e2m1_decode(qa._codes)
    if fmt == 4:
        b = x.to(torch.bfloat16).float().reshape(M, K // 16, 16)
        bs_x = Q._e4m3_round((b.abs().amax(dim=-1) / 6.0 / qa._g[:, None]).clamp(max=448.0))
        xd = (xc.reshape(M, K // 16, 16) * (bs_x * qa._g[:, None])[..., None]).reshape(M, K)
    else:
        _, e_x = Q.quantize_mxfp4(x.to(torch.bfloat16).float())
        xd = Q.dequant_mxfp4(qa._codes, e_x)
    want = xd.double() @ wd.double().T
    got = F.gemm_i8(qw, qa, splits=splits).float().cpu()
    F.scratch(DEV).check()
    err = (got.double() - want).abs().max().item()
    ref = want.abs().max().item()
    assert got.shape == (M, N)
    assert err <= 6e-3 * ref, (fmt, M, N, K, splits, err, ref)


@pytest.mark.parametrize("fmt", [4, 5])
@pytest.mark.parametrize("M,N,K,splits", [(8, 512, 1024, 1), (64, 304, 2048, 1), (128, 256, 512, 1), (200, 512, 1024, 1),
                                           (40, 512, 2048, 2), (72, 768, 4096, 4)])
def test_fp4_gemm_matches_the_exact_dequantisation(fmt, M, N, K, splits):
    _case(fmt, M, N, K, splits, seed=M + K)


def test_device_row_producer_writes_nvfp4_rows_the_gemm_reads():
    """add + RMSNorm + NVFP4 quantisation on the device (per-token fp32 scale, e4m3 per 16, e2m1 codes in
    the tiled rows, scale atoms) feeding the block-scaled GEMM, against the host restatement."""
    from saber_engine_b200.models.reference_hybrid import _fp4_linear
    from saber_engine_b200.ops import native as N
    from saber_engine_b200.ops import reference as R
    torch.manual_seed(5)
    M, K, Nn = 40, 1024, 512
    w = torch.randn(Nn, K) * 0.05
    codes, bs, g = Q.quantize_nvfp4(w)
    qw = F.QuantWeight.from_nvfp4(codes, bs, g, device=DEV)
    x = (torch.randn(M, K) * 2).to(torch.bfloat16)
    res = (torch.randn(M, K)).to(torch.bfloat16)
    nw = torch.randn(K) * 0.1
    qa = F.QuantAct.alloc(M, K, DEV).as_fp4(4)
    res_d = res.to(DEV).clone()
    F._row(N.ROW_ADD_RMS, F.row_params(M, K, a=x.to(DEV), res=res_d, w=nw.to(DEV), w_offset=1.0, eps=1e-6, qa=qa))
    got = F.gemm_i8(qw, qa).float().cpu()
    F.scratch(DEV).check()
    from saber_engine_b200.ops import layouts as L
    h = R.bf16_round(x.float() + res.float())
    normed = R.bf16_round(h * torch.rsqrt((h * h).mean(dim=1, keepdim=True) + 1e-6) * (1.0 + nw))
    # (1) what the device wrote, dequantised exactly, times the dequantised weight = what the GEMM returned
    c_dev, sf_dev = L.untile_act_fp4(qa.q.cpu(), qa.sf.cpu(), M, 16)
    g_dev = qa.scale[:M].cpu()
    bs_dev = sf_dev.view(torch.float8_e4m3fn).float()
    xd = (Q.e2m1_decode(c_dev).reshape(M, K // 16, 16) * (bs_dev * g_dev[:, None])[..., None]).reshape(M, K)
    want = (xd.double() @ Q.dequant_nvfp4(codes, bs, g).double().T).float()
    assert (got - want).abs().max().item() <= 6e-3 * want.abs().max().item()
    # (2) the device quantiser follows the law: token scale = amax / (6 * 448), block scale = e4m3(block amax / 6 / g),
    # and every value lands within half a code step of its block
    assert torch.allclose(g_dev, normed.abs().amax(dim=1) / (6.0 * 448.0), rtol=2e-2)
    blk = normed.reshape(M, K // 16, 16)
    bs_want = Q._e4m3_round((blk.abs().amax(dim=-1) / 6.0 / g_dev[:, None]).clamp(max=448.0))
    assert (bs_dev == bs_want).float().mean() > 0.98
    step = (bs_dev * g_dev[:, None])[..., None]                 # value of one unit of the e2m1 grid in each block
    err_units = (xd.reshape(M, K // 16, 16) - blk).abs() / step.clamp_min(1e-30)
    assert float(err_units.max()) <= 1.1 and float(err_units.mean()) < 0.3, (float(err_units.max()), float(err_units.mean()))   # the widest e2m1 gap is 2 units
    assert (Q.e2m1_encode(blk / step.clamp_min(1e-30)).reshape(M, K) == c_dev).float().mean() > 0.98
    ref2 = _fp4_linear(normed, qw).float()
    assert (got - ref2).abs().max().item() <= 0.12 * ref2.abs().max().item()           # coarse grid: rounding-level input differences flip codes
    # rows past M stay zero (codes and token scales)
    assert int(qa.q[:, M:].abs().sum()) == 0 and float(qa.scale[M:].abs().sum()) == 0.0


def test_nvfp4_model_steps_match_the_oracle_and_spec_equals_greedy():
    """The hybrid model with native NVFP4 linears (FP4 weights x FP4 activations on the block-scaled
    tensor-core path): prefill logits against the PyTorch oracle, speculative == greedy, graph == eager."""
    import dataclasses
    from saber_engine_b200.models import config as C
    from saber_engine_b200.models.hybrid import HybridModel, SeqStep, run_bucket
    from saber_engine_b200.models.reference_hybrid import forward_full
    cfg = dataclasses.replace(C.scaled_hybrid(), name="hybrid-mini-nvfp4", weight_format="nvfp4")
    model = HybridModel(cfg, device="cuda", max_seqs=4, max_ctx=512, max_width=5, seed=1)
    assert any(getattr(l.mixer_in, "fp4", 0) == 4 for l in model.w.layers)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    blocks = lambda j: list(range(1 + j * 32, 1 + (j + 1) * 32))

    def prefill(slot, j, eager=False):
        model.reset_slot(slot)
        b = model.build_bucket("prefill", 1, 48)
        return run_bucket(model, b, [SeqStep(prompt, 0, slot, 0, blocks(j))], eager=eager)

    def decode(first, drafts, slot, j, steps, width, eager=False):
        out, shift, pos, n_steps = [first], 0, len(prompt), 0
        b = model.build_bucket("decode", 1, width)
        while len(out) < steps:
            rows = [out[-1]] + list(drafts[:width - 1])
            r = run_bucket(model, b, [SeqStep(rows, pos, slot, shift, blocks(j), uid=7, step_no=n_steps)], eager=eager)
            n = r.n_commit[0]
            out += r.tokens[0]
            pos, shift, drafts, n_steps = pos + n, n, r.drafts[0], n_steps + 1
        return out[:steps]
    r = prefill(1, 0)
    got = model.buckets[("prefill", 1, 48)].logits[0, : cfg.vocab].float().cpu()
    ref = forward_full(cfg, model.w, torch.tensor(prompt))["logits"][-1]
    # 4-bit activations: a rounding-level difference between the device and the oracle flips a code, and a code
    # is worth up to a third of its value, so the two agree in direction and size, not to the last digit
    cos = float((got * ref).sum() / (got.norm() * ref.norm()))
    rel = float((got - ref).norm() / ref.norm())
    assert cos > 0.9 and rel < 0.45, (cos, rel)
    plain = decode(r.tokens[0][0], [], 1, 0, 16, 1)
    r2 = prefill(2, 1)
    assert r2.tokens == r.tokens
    assert decode(r2.tokens[0][0], r2.drafts[0], 2, 1, 16, 5) == plain
    r3 = prefill(3, 2, eager=True)
    assert decode(r3.tokens[0][0], r3.drafts[0], 3, 2, 16, 5, eager=True) == plain
