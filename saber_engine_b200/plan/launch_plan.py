"""One resolved launch plan: manifest (typed TOML) x device profile x model spec x buckets x autotune
table -> per-(op, shape) kernel variants, a byte ledger that derives the KV pool, and `explain`.

Parity: `crates/saber-plan/src/manifest.rs:1-20` (typed TOML, unknown key = error, all problems at
once), `src/plan.rs:929,1240-1385` (resolve -> bind, refusal when a route has no measurement unless
defaults are explicitly allowed), `src/autotune.rs:28-50` (keys), `crates/saber-cli/src/ledger_law.rs:1-20`
(KV pool = budget - billed - recurrent state - head-room; boot refusal when one max-ctx sequence
does not fit), `crates/saber-cli/src/explain.rs:1-15`.  There are no environment variables on the
engine path: everything is in the plan.
"""
from __future__ import annotations

import hashlib
import json
import tomllib
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Optional

from ..models import config as MC
from ..ops import layouts as L
from .autotune import TuneTable, make_key


class PlanError(Exception):
    def __init__(self, problems):
        super().__init__("; ".join(problems))
        self.problems = list(problems)


@dataclass
class DeviceProfile:
    name: str = "NVIDIA B200"
    sms: int = 148
    hbm_bytes: int = 180 * 10 ** 9
    hbm_gbs: float = 6534.0
    bf16_tflops: float = 1684.0
    nvlink_gbs_per_dir: float = 770.0
    l2_bytes: int = 126 << 20

    @staticmethod
    def measured(path="MEASURED_PEAKS.json") -> "DeviceProfile":
        p = Path(path)
        d = DeviceProfile()
        if p.exists():
            m = json.loads(p.read_text())
            d.hbm_gbs, d.bf16_tflops, d.name = m.get("hbm_gbs", d.hbm_gbs), m.get("bf16_tflops", d.bf16_tflops), m.get("gpu_name", d.name)
        return d


@dataclass
class Manifest:
    model: str = "qwen38-27b"
    pack: Optional[str] = None
    tp: int = 1
    max_ctx: int = 262144
    max_seqs: int = 8
    decode_batches: tuple = (1, 2, 3, 4, 8)
    decode_widths: tuple = (1, 5, 8)
    prefill_rows: tuple = (128, 512, 2048)
    draft_block: int = 8
    budget_mib: int = 160000
    headroom_mib: int = 2048
    prefix_cache_mib: int = 6144
    gdn_state_dtype: str = "f32"
    kv_dtype: str = "fp8_e4m3"
    autotune: Optional[str] = None
    allow_untuned: bool = False
    width_table: str = ""
    prefill_w8: bool = True             # big prefill rungs multiply with an int8 twin of the 4-bit linears (billed below)

    SECTIONS = {"model": ("model", "pack", "tp"), "limits": ("max_ctx", "max_seqs", "budget_mib", "headroom_mib", "prefix_cache_mib"),
                "buckets": ("decode_batches", "decode_widths", "prefill_rows", "draft_block", "width_table"),
                "plan": ("autotune", "allow_untuned", "gdn_state_dtype", "kv_dtype", "prefill_w8")}

    @staticmethod
    def from_toml(text: str) -> "Manifest":
        doc = tomllib.loads(text)
        problems, kw = [], {}
        for sec, body in doc.items():
            if sec not in Manifest.SECTIONS:
                problems.append(f"unknown section [{sec}]")
                continue
            if not isinstance(body, dict):
                problems.append(f"[{sec}] must be a table")
                continue
            for k, v in body.items():
                if k not in Manifest.SECTIONS[sec]:
                    problems.append(f"[{sec}] unknown key {k!r}")
                else:
                    kw[k] = tuple(v) if isinstance(v, list) else v
        m = Manifest(**kw) if not problems else Manifest()
        problems += m.problems()
        if problems:
            raise PlanError(problems)
        return m

    def problems(self) -> list:
        p = []
        if self.tp not in (1, 2, 4, 8):
            p.append(f"tp {self.tp} is not supported (1, 2, 4 or 8)")
        try:
            MC.by_name(self.model)
        except KeyError as exc:
            p.append(str(exc))
        if any(b > self.max_seqs for b in self.decode_batches):
            p.append("a decode batch exceeds max_seqs")
        if self.max_seqs not in self.decode_batches and max(self.decode_batches) < self.max_seqs:
            p.append("no decode batch covers max_seqs")
        if 1 not in self.decode_widths:
            p.append("decode_widths must contain 1")
        if max(self.decode_widths) > self.draft_block + 1:
            p.append("a decode width exceeds draft_block + 1")
        if self.gdn_state_dtype != "f32":
            p.append("gdn_state_dtype must be f32 (the recurrent state of this build is fp32 only)")
        return p


@dataclass
class Ledger:
    """Byte ledger: every arena is billed by name; the KV pool is what is left."""
    budget: int
    items: dict = field(default_factory=dict)

    def bill(self, name: str, nbytes: int) -> None:
        self.items[name] = self.items.get(name, 0) + int(nbytes)

    @property
    def billed(self) -> int:
        return sum(self.items.values())

    @property
    def remaining(self) -> int:
        return self.budget - self.billed

    def table(self) -> list:
        return sorted(self.items.items(), key=lambda kv: -kv[1])


def model_weight_bytes(cfg, tp: int) -> int:
    sh = MC.shard(cfg, tp, 0)
    H = cfg.hidden
    def lin(n, k, bits): return L.round_up(n, L.TILE_N) * k * bits // 8 + L.round_up(n, L.TILE_N) * 4
    per_attn = lin(sh.qkv_n, H, 4) + lin(H, sh.o_k, 4)
    per_gdn = lin(sh.gdn_in_n, H, 4) + lin(H, sh.gdn_out_k, 4)
    if cfg.moe is None:
        mlp = lin(2 * sh.ffn_inter, H, 4) + lin(H, sh.ffn_inter, 4)
    else:
        e = cfg.moe
        mlp = (e.n_experts // tp) * (3 * H * e.expert_inter // 2 + 3 * H * e.expert_inter // 32) + lin(3 * e.shared_inter, H, 4) + e.n_experts * H * 2
    total = cfg.n_attn_layers * (per_attn + mlp) + cfg.n_gdn_layers * (per_gdn + mlp)
    total += cfg.vocab * H * 2 + lin(sh.vocab, H, cfg.lm_head_bits)
    if cfg.drafter:
        d = cfg.drafter
        total += lin(d.hidden, d.n_taps * H, 4) + d.n_layers * (lin(2 * d.inter, d.hidden, 4) + lin(d.hidden, d.inter, 4)) + lin(cfg.vocab, d.hidden, d.head_bits)
    return total


@dataclass
class LaunchPlan:
    manifest: Manifest
    device: DeviceProfile
    routes: dict
    ledger: Ledger
    kv_blocks: int
    kv_tokens: int
    missing: list
    plan_hash: str

    def explain(self) -> str:
        m = self.manifest
        from ..rules import default_rules
        out = [f"plan {self.plan_hash[:16]}  model={m.model} tp={m.tp} device={self.device.name}  "
               f"rules={default_rules().doc['name']}@{default_rules().policy_digest()[:12]}",
               f"  context {m.max_ctx} tokens x {m.max_seqs} sequences; decode batches {list(m.decode_batches)} x widths {list(m.decode_widths)}; prefill rungs {list(m.prefill_rows)}",
               "  ledger (bytes per rank):"]
        for name, b in self.ledger.table():
            out.append(f"    {name:28s} {b / 2 ** 20:12.1f} MiB")
        out.append(f"    {'kv_pool (derived)':28s} {self.kv_blocks * self._block_bytes / 2 ** 20:12.1f} MiB = {self.kv_blocks} blocks = {self.kv_tokens} tokens")
        out.append(f"  routes: {len(self.routes)} ({sum(1 for r in self.routes.values() if r['source'] == 'autotune')} measured, "
                   f"{sum(1 for r in self.routes.values() if r['source'] == 'default')} on declared defaults)")
        for key, r in sorted(self.routes.items()):
            out.append(f"    {key:60s} -> {r['variant']}  [{r['source']}]")
        if self.missing:
            out.append(f"  MISSING measurements ({len(self.missing)}): run `saber tune`, or set allow_untuned = true")
            out += [f"    {k}" for k in self.missing]
        return "\n".join(out)


def resolve(manifest: Manifest, device: Optional[DeviceProfile] = None, table: Optional[TuneTable] = None) -> LaunchPlan:
    problems = manifest.problems()
    if problems:
        raise PlanError(problems)
    device = device or DeviceProfile()
    cfg = MC.by_name(manifest.model)
    tp = manifest.tp
    sh = MC.shard(cfg, tp, 0)
    if table is None and manifest.autotune:
        table = TuneTable.load(manifest.autotune)
    # ---- routes: one per (linear, rows) the buckets can produce
    from .tune_gemm import model_gemm_shapes
    from ..ops.functional import pick_splits
    rows = sorted({b * w for b in manifest.decode_batches for w in manifest.decode_widths} | set(manifest.prefill_rows))
    routes, missing = {}, []
    for name, Nn, K, w4 in model_gemm_shapes(cfg, tp):
        n_pad = L.round_up(Nn, L.TILE_N)
        for M in rows:
            key = make_key("gemm_i8", N=n_pad, K=K, M=M, w4=w4)
            hit = table.records.get(key) if table else None
            if hit is not None:
                routes[f"{name} M={M}"] = {"key": key, "variant": {k: hit.variant.get(k, 1) for k in ("splits", "stages", "halves")}, "source": "autotune"}
            else:
                nt = L.token_tile(M)
                routes[f"{name} M={M}"] = {"key": key, "variant": {"splits": pick_splits(n_pad // L.TILE_N, (M + nt - 1) // nt, K // 128), "stages": 0},
                                           "source": "default"}
                missing.append(key)
    if missing and not manifest.allow_untuned:
        pass   # reported by explain; `bind` refuses
    # ---- ledger
    led = Ledger(manifest.budget_mib << 20)
    led.bill("weights", model_weight_bytes(cfg, tp))
    if manifest.prefill_w8 and cfg.moe is None and getattr(cfg, "weight_format", "iu8") == "iu8" and max(rows) >= 256:
        # (twice the packed linears; the embedding table and the int8 head have no twin: an upper bound)
        led.bill("weights_prefill_int8_twin", 2 * model_weight_bytes(cfg, tp))
    state_b = 4 if manifest.gdn_state_dtype == "f32" else 2
    led.bill("gdn_state_slots", (manifest.max_seqs + 1) * cfg.gdn_state_bytes_per_seq(tp, state_b))
    led.bill("prefix_cache_snapshots", manifest.prefix_cache_mib << 20)
    max_rows = max(rows)
    led.bill("activation_arenas", max_rows * (sh.gdn_in_n * 2 + 2 * sh.ffn_inter * 2 + cfg.hidden * 12 + sh.gdn_conv_c * 4) * 2)
    led.bill("logits", max(manifest.decode_batches) * max(manifest.decode_widths) * sh.vocab * 2 * 2)
    led.bill("splitk_scratch", 256 * 262144 * 4)
    led.bill("headroom", manifest.headroom_mib << 20)
    block_bytes = cfg.kv_bytes_per_token(tp) * cfg.page_tokens
    kv_blocks = max(0, led.remaining // block_bytes) if block_bytes else 0
    need = (manifest.max_ctx + cfg.page_tokens - 1) // cfg.page_tokens + 1
    if block_bytes and kv_blocks < need:
        raise PlanError([f"one {manifest.max_ctx}-token sequence needs {need} KV blocks but the ledger leaves {kv_blocks}: "
                         f"raise budget_mib or lower max_ctx"])
    cap = manifest.max_seqs * need + 1        # never larger than every sequence at full context
    kv_blocks = min(kv_blocks, cap) if block_bytes else 0
    from ..rules import default_rules
    desc = {"manifest": {k: (list(v) if isinstance(v, tuple) else v) for k, v in asdict(manifest).items()},
            "routes": {k: v["variant"] for k, v in routes.items()}, "kv_blocks": kv_blocks,
            "rules": default_rules().policy_digest()}
    plan = LaunchPlan(manifest, device, routes, led, kv_blocks, kv_blocks * cfg.page_tokens, missing,
                      hashlib.sha256(json.dumps(desc, sort_keys=True).encode()).hexdigest())
    plan._block_bytes = block_bytes
    return plan


def bind(plan: LaunchPlan) -> LaunchPlan:
    """Refuse to run on unmeasured routes unless the manifest allows declared defaults."""
    if plan.missing and not plan.manifest.allow_untuned:
        raise PlanError([f"{len(plan.missing)} routes have no measurement (first: {plan.missing[0]}); "
                         "run `saber tune` or set [plan] allow_untuned = true"])
    return plan
