"""SBRPACK1 writer / reader / manifest: round trip, byte offsets, refusals (each with its control)."""
import json
import struct

import numpy as np
import pytest
import torch

from saber_engine_b200.models import config as C
from saber_engine_b200.pack import build as PB
from saber_engine_b200.pack import format as PF


def _small(tmp_path, name="rank0.pack"):
    w = PF.PackWriter(tmp_path / name, 1, 0, {"plan": 1}, {"tier": 1}, build_unix=7)
    w.add("a.weight", np.arange(12, dtype=np.float32).reshape(3, 4), "f32")
    w.add("b.packed", np.arange(5000, dtype=np.uint8), "u8", (100, 100), PF.LAYOUT_W4_TILE256, PF.SHARD_DIM0)
    return w.finish()


def test_header_offsets_and_roundtrip(tmp_path):
    info = _small(tmp_path)
    raw = (tmp_path / "rank0.pack").read_bytes()
    assert raw[:8] == b"SBRPACK1"
    assert struct.unpack_from("<I", raw, 8)[0] == 2 and struct.unpack_from("<I", raw, 12)[0] == 256
    assert struct.unpack_from("<I", raw, 16)[0] == 160 and struct.unpack_from("<I", raw, 20)[0] == 2
    assert struct.unpack_from("<Q", raw, 24)[0] == 256
    assert struct.unpack_from("<Q", raw, 48)[0] % 4096 == 0 and struct.unpack_from("<Q", raw, 56)[0] == len(raw)
    assert struct.unpack_from("<I", raw, 224)[0] == 4 << 20
    r = PF.PackReader(tmp_path / "rank0.pack")
    assert r.order == ["a.weight", "b.packed"]
    a = np.array(r.payload("a.weight")).view(np.float32).reshape(3, 4)
    assert np.array_equal(a, np.arange(12, dtype=np.float32).reshape(3, 4))
    assert r.records["b.packed"].layout_id == PF.LAYOUT_W4_TILE256 and r.records["b.packed"].data_off % 4096 == 0
    assert info["record_count"] == 2


@pytest.mark.parametrize("where,what", [(0, "magic"), (8, "format_version"), (300, "table_sha256"), (-1, "digest")])
def test_reader_refuses_corruption(tmp_path, where, what):
    _small(tmp_path)
    p = tmp_path / "rank0.pack"
    raw = bytearray(p.read_bytes())
    if where == -1:
        where = PF.PackReader(p).records["b.packed"].data_off + 17      # a byte inside that payload
        raw[where] ^= 0xFF
        where = -1
    else:
        raw[where] ^= 0xFF
    p.write_bytes(bytes(raw))
    if where == -1:
        r = PF.PackReader(p)                       # structure is intact, the payload is not
        with pytest.raises(PF.PackError, match="digest"):
            r.payload("b.packed")
        r.payload("a.weight")                      # control: the untouched record still verifies
    else:
        with pytest.raises(PF.PackError, match=what):
            PF.PackReader(p)


def test_reader_refuses_truncation_and_wrong_plan(tmp_path):
    _small(tmp_path)
    p = tmp_path / "rank0.pack"
    PF.PackReader(p, expect_plan_hash=PF.sha256(PF.canonical_json({"plan": 1})), expect_tp=1, expect_rank=0)
    with pytest.raises(PF.PackError, match="plan_hash"):
        PF.PackReader(p, expect_plan_hash=PF.sha256(b"other"))
    with pytest.raises(PF.PackError, match="tp_size"):
        PF.PackReader(p, expect_tp=2)
    p.write_bytes(p.read_bytes()[:-100])
    with pytest.raises(PF.PackError, match="file_bytes"):
        PF.PackReader(p)


def test_model_pack_roundtrip_and_manifest(tmp_path):
    cfg = C.scaled_hybrid(n_layers=4, hidden=256, ffn=512, vocab=512)
    d = PB.write_pack(cfg, tmp_path, tp=1, seed=3)
    assert PF.check_manifest(d) == []
    mw = PB.load_weights(tmp_path, cfg, 1, 0, "cpu")
    from saber_engine_b200.models.weights import random_init
    ref = random_init(cfg, 1, 0, "cpu", 3)
    assert torch.equal(mw.embed, ref.embed) and torch.equal(mw.lm_head.tiles, ref.lm_head.tiles)
    assert mw.layers[0].kind == "gdn" and mw.layers[3].kind == "attn"
    assert torch.equal(mw.layers[0].mixer_in.tiles, ref.layers[0].mixer_in.tiles)
    assert mw.layers[0].down.w4 is False and mw.layers[1].down.w4 is True     # the pack decides W8 vs W4
    assert torch.equal(mw.drafter.head.scale, ref.drafter.head.scale)
    # manifest tamper: a changed record hash is reported
    m = json.loads((d / "manifest.json").read_text())
    m["ranks"][0]["records"][0]["sha256"] = "00" * 32
    (d / "manifest.json").write_text(json.dumps(m))
    assert any("manifest entry differs" in p for p in PF.check_manifest(d))
    with pytest.raises(PF.PackError):
        PB.load_weights(tmp_path, cfg, 1, 0, "cpu")


def test_tp2_pack_shards_and_wrong_config_is_refused(tmp_path):
    cfg = C.scaled_hybrid(n_layers=4, hidden=256, ffn=512, vocab=512)
    d = PB.write_pack(cfg, tmp_path, tp=2, seed=3)
    assert PF.check_manifest(d) == []
    a = PB.load_weights(tmp_path, cfg, 2, 0, "cpu")
    b = PB.load_weights(tmp_path, cfg, 2, 1, "cpu")
    assert a.layers[0].down.K == cfg.ffn_inter // 2 and a.lm_head.N == cfg.vocab // 2
    assert not torch.equal(a.layers[0].down.tiles, b.layers[0].down.tiles)
    assert torch.equal(a.embed, b.embed)
    other = C.scaled_hybrid(n_layers=4, hidden=256, ffn=512, vocab=1024)
    with pytest.raises(PF.PackError, match="plan_hash"):
        PB.load_weights(tmp_path, other, 2, 0, "cpu", verify=False)


def test_mxfp4_and_moe_packs_roundtrip(tmp_path):
    import dataclasses
    from saber_engine_b200.models.weights import random_init
    cfg = dataclasses.replace(C.scaled_hybrid(n_layers=2, hidden=256, ffn=512, vocab=512, drafter=False), weight_format="mxfp4")
    d = PB.write_pack(cfg, tmp_path / "mx", tp=1, seed=4)
    assert PF.check_manifest(d) == []
    mw = PB.load_weights(tmp_path / "mx", cfg, 1, 0, "cpu")
    ref = random_init(cfg, 1, 0, "cpu", 4)
    assert mw.layers[1].gate_up.mx and torch.equal(mw.layers[1].gate_up.tiles, ref.layers[1].gate_up.tiles)
    assert not mw.layers[0].down.mx and not mw.layers[0].down.w4          # the designated W8 linear stays int8
    man = json.loads((d / "manifest.json").read_text())
    assert man["plan"]["descriptor"]["format"].startswith("mxfp4")
    # an iu8 config refuses the MXFP4 pack (plan hash binds the format)
    with pytest.raises(PF.PackError):
        PB.load_weights(tmp_path / "mx", dataclasses.replace(cfg, weight_format="iu8"), 1, 0, "cpu")
    moe = C.scaled_hybrid(n_layers=2, hidden=256, ffn=512, vocab=512, drafter=False, name="mini-moe",
                          moe=C.MoEConfig(n_experts=8, top_k=2, expert_inter=128, shared_inter=128))
    d2 = PB.write_pack(moe, tmp_path / "moe", tp=2, seed=5)
    assert PF.check_manifest(d2) == []
    for rank in range(2):
        got = PB.load_weights(tmp_path / "moe", moe, 2, rank, "cpu")
        want = random_init(moe, 2, rank, "cpu", 5)
        m0, w0 = got.layers[0].moe, want.layers[0].moe
        assert m0["e_lo"] == 4 * rank and m0["e_n"] == 4
        assert torch.equal(m0["gate_up"].tiles, w0["gate_up"].tiles) and torch.equal(m0["down"].scale, w0["down"].scale)
        assert torch.equal(m0["router"].tiles, w0["router"].tiles)
        assert (m0["shared_gate_up"] is None) == (w0["shared_gate_up"] is None)
