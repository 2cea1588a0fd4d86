"""Launch rules as data: the packaged table loads, refuses unknown keys with every problem at once,
reproduces the launch decisions of the 27B shapes, and the launchers really read it."""
import copy

import pytest

from saber_engine_b200.rules import Rules, RulesError, default_rules, set_default_rules


def test_packaged_table_resolves_the_27b_routes():
    r = default_rules()
    assert len(r.policy_digest()) == 64
    d = r.resolve_gemm(34816, 5120, 64, "int4")                      # gate_up: 136 tiles fill the SMs
    assert d.grid == (136, 1, 1) and d.variant["splits"] == 1 and d.symbol == "saber::gemm_i8_kernel"
    d = r.resolve_gemm(5120, 17408, 64, "int4")                      # down: 20 tiles x 7 parts = 140 CTAs
    assert d.grid == (20, 1, 7) and d.digest == r.policy_digest()
    assert r.resolve_gemm(16640, 5120, 64, "int4").variant["halves"] == 2      # 65 tiles: two CTAs per packed tile
    assert r.resolve_gemm(16640, 5120, 64, "int8").variant["halves"] == 1      # int8 tiles have no halves
    assert r.resolve_gemm(34816, 5120, 2048, "int4").grid == (136, 16, 1)
    assert r.token_tile(9) == 16 and r.token_tile(72) == 80 and r.token_tile(4096) == 128
    assert r.gemm_splits(20, 1, 6) == 1                               # too few k-blocks to split
    assert r.attn_decode_splits("tc", 8, 4, 6, 8) == 4 and r.attn_decode_splits("tc", 1, 4, 6, 8) == 32
    assert r.attn_decode_splits("tc", 1, 4, 6, 64) == 1               # a prefill-sized tile does not split
    assert r.attn_decode_splits("paged", 8, 4, 6, 8) == 9
    assert r.gdn_form(True, 8) == "recurrent" and r.gdn_form(False, 2048) == "prefill_rows" and r.gdn_form(False, 8) == "recurrent"


def test_unknown_and_missing_keys_are_all_reported():
    doc = copy.deepcopy(default_rules().doc)
    doc["gemm"]["splits"]["max_part"] = 4
    del doc["gdn"]["head_k"]
    doc["colour"] = "red"
    with pytest.raises(RulesError) as ei:
        Rules(doc)
    text = str(ei.value)
    assert "max_part" in text and "head_k" in text and "colour" in text and len(ei.value.problems) == 3


def test_the_launchers_read_the_table_and_the_digest_follows_it():
    from saber_engine_b200.ops.functional import pick_splits
    from saber_engine_b200.plan import launch_plan as LP
    base = default_rules()
    assert pick_splits(20, 1, 136) == 7
    h0 = LP.resolve(LP.Manifest(allow_untuned=True)).plan_hash
    doc = copy.deepcopy(base.doc)
    doc["gemm"]["splits"]["max_parts"] = 4
    try:
        set_default_rules(Rules(doc))
        assert default_rules().policy_digest() != base.policy_digest()
        assert pick_splits(20, 1, 136) == 4
        assert LP.resolve(LP.Manifest(allow_untuned=True)).plan_hash != h0      # another policy, another plan
    finally:
        set_default_rules(None)
    assert pick_splits(20, 1, 136) == 7


def test_prefill_and_tail_thresholds_are_table_entries_and_the_ledger_bills_the_int8_twins():
    from saber_engine_b200.plan import launch_plan as LP
    r = default_rules()
    assert r.doc["prefill"]["sequence_parallel_min_ranks"] == 2 and r.doc["gemm"]["tails"]["row_tail_max_ranks"] == 1
    doc = copy.deepcopy(r.doc)
    del doc["prefill"]["sequence_parallel_min_ranks"]
    with pytest.raises(RulesError) as ei:
        Rules(doc)
    assert "sequence_parallel_min_ranks" in str(ei.value)
    # big prefill rungs multiply with int8 twins of the 4-bit linears: the plan bills them before it sizes the KV pool
    on = LP.resolve(LP.Manifest(allow_untuned=True))
    off = LP.resolve(LP.Manifest(allow_untuned=True, prefill_w8=False))
    assert "weights_prefill_int8_twin" in on.ledger.items and "weights_prefill_int8_twin" not in off.ledger.items
    assert on.plan_hash != off.plan_hash
