"""Resolver of the launch rules: the tables (`rules/*.toml`) say every number a launcher decides
from; this module validates a table (unknown key = error, all problems at once), answers the
launchers' questions, and gives the table's policy digest, which the launch plan hashes.

Parity: `crates/saber-kernels/rules/*.toml` (launch rules as data), `crates/saber-kernels/src/*.rs`
`resolve(op, shape, rules) -> LaunchDescriptor`, the policy digest carried per route.
"""
from __future__ import annotations

import hashlib
import json
import math
import tomllib
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

SCHEMA = {
    "": {"schema_version", "name", "device", "gemm", "prefill", "attn_tc", "attn_paged", "gdn"},
    "prefill": {"sequence_parallel_min_ranks"},
    "device": {"sms", "smem_per_cta", "tmem_columns"},
    "gemm": {"symbol", "tile_n", "tile_k", "threads", "token_tiles", "splits", "halves", "stages", "tails"},
    "gemm.tails": {"row_tail_max_ranks"},
    "gemm.splits": {"waves", "max_parts", "min_kb_per_split", "min_kb", "skip_when_fill_above"},
    "gemm.halves": {"formats", "fill_above", "fill_up_to"},
    "gemm.stages": {"int4", "int8", "mxfp4", "pair"},
    "attn_tc": {"symbol", "threads", "keys_per_tile", "max_rows_per_tile", "split_query_tokens", "decode_splits"},
    "attn_tc.decode_splits": {"fill_target", "ceiling", "floor"},
    "attn_paged": {"symbol", "tile_rows", "tiles_per_cta", "ctas_per_sm", "decode_splits"},
    "attn_paged.decode_splits": {"fill_target", "ceiling", "floor"},
    "gdn": {"head_k", "head_v", "decode_value_slices", "prefill_rows_form_from", "chunk_form_from", "fused_step_max_rows", "fused_step"},
}


class RulesError(Exception):
    def __init__(self, problems):
        super().__init__("; ".join(problems))
        self.problems = list(problems)


@dataclass(frozen=True)
class LaunchDescriptor:
    symbol: str
    grid: tuple
    block: int
    variant: dict
    digest: str               # policy digest of the table that decided this launch


class Rules:
    def __init__(self, doc: dict, source: str = "<memory>"):
        self.doc, self.source = doc, source
        problems = []
        def walk(node, path):
            allowed = SCHEMA.get(path)
            if allowed is None:
                return
            for k, v in node.items():
                if k not in allowed:
                    problems.append(f"[{path or 'top level'}] unknown key {k!r}")
                elif isinstance(v, dict):
                    walk(v, f"{path}.{k}" if path else k)
            for k in allowed - set(node):
                problems.append(f"[{path or 'top level'}] missing key {k!r}")
        walk(doc, "")
        if not problems:
            if doc["schema_version"] != 1:
                problems.append(f"schema_version {doc['schema_version']} is not supported")
            if doc["gdn"]["decode_value_slices"] not in (1, 2, 4):
                problems.append("[gdn] decode_value_slices must be 1, 2 or 4")
            if not 0 < doc["gemm"]["halves"]["fill_above"] < doc["gemm"]["halves"]["fill_up_to"] <= 1:
                problems.append("[gemm.halves] wants 0 < fill_above < fill_up_to <= 1")
        if problems:
            raise RulesError(problems)

    @staticmethod
    def load(path) -> "Rules":
        p = Path(path)
        return Rules(tomllib.loads(p.read_text()), str(p))

    # ---- digest
    def policy_digest(self) -> str:
        return hashlib.sha256(json.dumps(self.doc, sort_keys=True).encode()).hexdigest()

    @property
    def sms(self) -> int:
        return self.doc["device"]["sms"]

    # ---- GEMM
    def token_tile(self, M: int) -> int:
        tiles = self.doc["gemm"]["token_tiles"]
        return next((t for t in tiles if M <= t), tiles[-1])

    def gemm_splits(self, n_tiles: int, m_tiles: int, kb: int) -> int:
        r = self.doc["gemm"]["splits"]
        ctas = n_tiles * m_tiles
        if ctas > self.sms * r["skip_when_fill_above"] or kb < r["min_kb"]:
            return 1
        s = min(self.sms * r["waves"] // ctas, max(1, kb // r["min_kb_per_split"]), r["max_parts"])
        while s > 1 and (s - 1) * math.ceil(kb / s) >= kb:     # no empty part
            s -= 1
        return max(1, s)

    def gemm_halves(self, fmt: str, n_tiles: int, m_tiles: int) -> bool:
        r = self.doc["gemm"]["halves"]
        ctas = n_tiles * m_tiles
        return fmt in r["formats"] and self.sms * r["fill_above"] < ctas <= self.sms * r["fill_up_to"]

    def gemm_stages(self, fmt: str, pair: bool = False) -> int:
        st = self.doc["gemm"]["stages"]
        return st["pair"] if pair else st[fmt]

    def resolve_gemm(self, N_pad: int, K: int, M: int, fmt: str) -> LaunchDescriptor:
        g = self.doc["gemm"]
        nt = self.token_tile(M)
        n_tiles, m_tiles, kb = N_pad // g["tile_n"], -(-M // nt), K // g["tile_k"]
        halves = 2 if self.gemm_halves(fmt, n_tiles, m_tiles) else 1
        splits = 1 if halves == 2 else self.gemm_splits(n_tiles, m_tiles, kb)
        return LaunchDescriptor(g["symbol"], (n_tiles * halves, m_tiles, splits), g["threads"],
                                {"nt": nt, "splits": splits, "halves": halves, "stages": self.gemm_stages(fmt)}, self.policy_digest())

    # ---- attention
    def attn_decode_splits(self, impl: str, nseq: int, n_kv_heads: int, group: int, width: int) -> int:
        if impl == "tc":
            r = self.doc["attn_tc"]
            if width > r["split_query_tokens"] or width * group > r["max_rows_per_tile"]:
                return 1
            law, units = r["decode_splits"], nseq * n_kv_heads
        else:
            r = self.doc["attn_paged"]
            hpt = min(group, r["tile_rows"] // width) if 1 <= width <= r["tile_rows"] // 2 else 1
            tiles = -(-group // hpt)
            law, units = r["decode_splits"], nseq * n_kv_heads * -(-tiles // r["tiles_per_cta"])
        return max(law["floor"], min(law["ceiling"], law["fill_target"] // max(1, units)))

    # ---- Gated DeltaNet
    def gdn_form(self, decode: bool, rows: int) -> str:
        g = self.doc["gdn"]
        if decode:
            return "fused_step" if g["fused_step"] and rows <= g["fused_step_max_rows"] else "recurrent"
        return "prefill_rows" if rows >= g["prefill_rows_form_from"] else "recurrent"


_DEFAULT: Optional[Rules] = None


def default_rules() -> Rules:
    global _DEFAULT
    if _DEFAULT is None:
        _DEFAULT = Rules.load(Path(__file__).with_name("b200.toml"))
    return _DEFAULT


def set_default_rules(rules: Optional[Rules]) -> None:
    """Install another table (a manifest's `rules = "..."`), or None to go back to the packaged one."""
    global _DEFAULT
    _DEFAULT = rules
