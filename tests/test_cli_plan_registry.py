"""Front door: registry, serve planning, launch plan / explain / ledger, autotune laws, CLI."""
import json
import subprocess
import sys

import pytest

from saber_engine_b200.cli.main import main as saber
from saber_engine_b200.plan import launch_plan as LP
from saber_engine_b200.plan.autotune import TuneRecord, TuneTable, choose, make_key
from saber_engine_b200.registry import registry as R


def test_registry_loads_and_plans_tp_by_gpu_count(tmp_path):
    reg = R.load(user_file=tmp_path / "none.toml")
    m = reg.resolve("w4a8")
    assert m.name == "Qwen3.8-27B-W4A8-B200" and sorted(m.tp) == [1, 2, 4, 8]
    assert R.choose_tp(m, None, gpus=8) == 8 and R.choose_tp(m, None, gpus=3) == 2
    assert R.choose_tp(m, None, gpus=0) == 2                      # default_tp when no GPU is visible
    with pytest.raises(R.RegistryError):
        R.choose_tp(m, 3)
    p = R.plan_serve(reg, "27b", tp=4, port=9000, packs=str(tmp_path))
    a = p["argv"]
    assert a[:2] == ["saber", "engine"] and a[a.index("--engine-tp") + 1] == "4"
    assert a[a.index("--engine-decode-widths") + 1] == "1,5,8" and a[a.index("--port") + 1] == "9000"
    assert p["pack_present"] is False


def test_registry_reports_all_problems_at_once(tmp_path):
    bad = tmp_path / "models.toml"
    bad.write_text('schema = 1\n[[model]]\nname = "x y"\n[[model]]\nname = "ok"\nkind = "weird"\nbogus = 1\n'
                   'tokenizer = "t.json"\n[model.tp.3]\npath = "p"\n[[model]]\nname = "w4a8"\n[model.tp.1]\npath="p"\nmax_ctx=1\nmax_seqs=1\n')
    with pytest.raises(R.RegistryError) as ei:
        R.load(user_file=bad)
    text = " | ".join(ei.value.problems)
    for frag in ("letters, digits", "kind must be", "unknown key 'bogus'", "tp.3", "tokenizer must be one of files", "alias 'w4a8'"):
        assert frag in text, frag


def test_user_file_overrides_and_file_mirror_pull(tmp_path):
    from saber_engine_b200.models import config as C
    from saber_engine_b200.pack.build import write_pack
    mirror = tmp_path / "mirror"
    write_pack(C.scaled_hybrid(n_layers=4, hidden=256, ffn=512, vocab=512), mirror / "me" / "mini", tp=1)
    user = tmp_path / "models.toml"
    user.write_text(f'default = "mine"\n[[model]]\nname = "mine"\nrepo = "me/mini"\nendpoint = "file://{mirror}"\n'
                    'config = "hybrid-mini"\n[model.tp.1]\npath = "tp1"\nmax_ctx = 512\nmax_seqs = 2\ndecode_batches = "1,2"\n')
    reg = R.load(user_file=user)
    assert reg.resolve(None).name == "mine"
    out = R.pull(reg, "mine", packs=str(tmp_path / "packs"))
    assert out["verified"] and (tmp_path / "packs" / "me" / "mini" / "tp1" / "manifest.json").exists()
    assert R.plan_serve(reg, None, packs=str(tmp_path / "packs"), gpus=1)["pack_present"]
    assert R.remove(reg, "mine", packs=str(tmp_path / "packs")) and not (tmp_path / "packs" / "me" / "mini" / "tp1").exists()


def test_manifest_unknown_keys_and_plan_hash():
    with pytest.raises(LP.PlanError) as ei:
        LP.Manifest.from_toml('[model]\nmodel="qwen38-27b"\ntp=3\nfoo=1\n[nope]\nx=1\n')
    text = " | ".join(ei.value.problems)
    assert "unknown key 'foo'" in text and "unknown section [nope]" in text
    man = LP.Manifest.from_toml('[model]\nmodel="qwen38-27b"\ntp=2\n[plan]\nallow_untuned=true\n')
    plan = LP.resolve(man)
    assert plan.kv_tokens >= 8 * 262144 and plan.ledger.items["weights"] > 5e9
    again = LP.resolve(man)
    assert plan.plan_hash == again.plan_hash
    other = LP.resolve(LP.Manifest(model="qwen38-27b", tp=4, allow_untuned=True))
    assert other.plan_hash != plan.plan_hash
    text = plan.explain()
    assert "kv_pool (derived)" in text and "mlp.gate_up M=64" in text and "[default]" in text
    with pytest.raises(LP.PlanError, match="no measurement"):
        LP.bind(LP.resolve(LP.Manifest(model="qwen38-27b", tp=2)))          # untuned routes are refused
    with pytest.raises(LP.PlanError, match="KV blocks"):
        LP.resolve(LP.Manifest(model="qwen38-27b", tp=1, budget_mib=30000, allow_untuned=True))


def test_plan_uses_measured_routes():
    man = LP.Manifest(model="qwen38-27b", tp=1, decode_batches=(1, 8), decode_widths=(1, 9), prefill_rows=(128,))
    t = TuneTable()
    base = LP.resolve(LP.Manifest(**{**man.__dict__, "allow_untuned": True}))
    for r in base.routes.values():
        t.put(TuneRecord(r["key"], {"splits": 3, "stages": 4, "name": "s3_st4"}, 10.0))
    plan = LP.bind(LP.resolve(man, table=t))
    assert not plan.missing and all(r["source"] == "autotune" and r["variant"]["splits"] == 3 for r in plan.routes.values())


def test_autotune_choose_laws():
    s = {"ref": [99.0, 10.0, 10.1, 10.0], "fast": [5.0, 9.95, 9.96, 9.95], "slow": [1.0, 20.0, 21.0, 20.0]}
    best, us, second = choose(s, "ref")
    assert best == "ref"                       # within 1%: the reference variant keeps the route
    s["fast"] = [5.0, 8.0, 8.1, 8.0]
    assert choose(s, "ref")[0] == "fast"       # warm-up samples (99, 5, 1) never count
    assert make_key("gemm_i8", N=1, K=2, M=3, w4=1) == "gemm_i8|K=2,M=3,N=1,w4=1"


def test_cli_front_door(tmp_path, capsys):
    assert saber(["models", "list", "--json", "--packs-dir", str(tmp_path)]) == 0
    rows = json.loads(capsys.readouterr().out)
    assert any(r["name"] == "hybrid-mini" for r in rows)
    assert saber(["serve", "--model", "w4a8", "--tp", "2", "--print-argv", "--packs-dir", str(tmp_path)]) == 0
    assert "--engine-tp 2" in capsys.readouterr().out
    assert saber(["serve", "--model", "nope", "--dry-run"]) == 2
    assert saber(["pack", "build", "--model", "hybrid-mini", "--out", str(tmp_path / "p")]) == 0
    assert saber(["pack", "check", "--dir", str(tmp_path / "p" / "tp1")]) == 0
    assert saber(["explain", "--model", "qwen38-27b", "--tp", "8"]) == 0
    assert "tp=8" in capsys.readouterr().out
    r = subprocess.run([sys.executable, "-m", "saber_engine_b200", "probe"], capture_output=True, text=True)
    assert r.returncode == 0 and "native_library" in r.stdout


def test_attention_split_records_are_looked_up_by_shape_and_nearest_context():
    """`attn_tc_decode` records sit beside the GEMM records; a lookup takes the record of the largest tuned
    context not above the asked one, and none when the shape was never measured."""
    from saber_engine_b200.plan.autotune import TuneRecord, TuneTable, make_key
    from saber_engine_b200.plan.tune_attn import OP, lookup
    t = TuneTable("test-device", "build")
    t.put(TuneRecord(make_key(OP, nseq=8, width=8, ctx=4096, nq=24, nkv=4), {"splits": 4, "name": "s4"}, 40.0, 41.0, 7, True))
    t.put(TuneRecord(make_key(OP, nseq=8, width=8, ctx=65536, nq=24, nkv=4), {"splits": 16, "name": "s16"}, 300.0, 320.0, 7, True))
    assert lookup(t, 8, 8, 4096, 24, 4) == 4
    assert lookup(t, 8, 8, 20000, 24, 4) == 4            # between the tuned contexts: the one below
    assert lookup(t, 8, 8, 262144, 24, 4) == 16
    assert lookup(t, 8, 8, 512, 24, 4) is None           # below the smallest tuned context: the rules decide
    assert lookup(t, 4, 8, 4096, 24, 4) is None and lookup(None, 8, 8, 4096, 24, 4) is None
    t2 = TuneTable.load_json(t.to_json()) if hasattr(TuneTable, "load_json") else None
    assert t2 is None or lookup(t2, 8, 8, 4096, 24, 4) == 4
