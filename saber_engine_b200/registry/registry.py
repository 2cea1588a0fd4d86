"""Model registry (schema 1): the compiled-in models.toml merged with the user's file; validation
reports ALL problems at once; `plan_serve` composes the fully explicit engine argument list that
`saber serve --model` runs (and `--dry-run` / `--print-argv` print).

Parity: `docs/MODELS.md:20-124`, `crates/saber-cli/src/models/registry.rs:1-8`,
`models/front.rs:1-8` (front door), `models/plan.rs` (argv composition, cf.
`tools/serve_27b.sh:189-194`).  New: TP degrees 1, 2, 4 and 8.
"""
from __future__ import annotations

import os
import re
import shutil
import tomllib
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

VALID_TP = (1, 2, 4, 8)
_NAME = re.compile(r"^[A-Za-z0-9._+\-]+$")


class RegistryError(Exception):
    def __init__(self, problems):
        super().__init__("; ".join(problems))
        self.problems = list(problems)


@dataclass
class TpEntry:
    tp: int
    path: str
    bytes: int = 0
    max_ctx: int = 0
    max_seqs: int = 0
    prefill_rows: str = ""
    decode_batches: str = ""
    decode_widths: str = "1"
    draft_block: int = 8
    budget_mib: int = 0
    legacy_dirs: list = field(default_factory=list)
    tail_args: list = field(default_factory=list)


@dataclass
class ModelEntry:
    name: str
    kind: str = "target"
    aliases: list = field(default_factory=list)
    description: str = ""
    repo: str = ""
    revision: str = "main"
    endpoint: Optional[str] = None
    served_id: str = ""
    drafter: Optional[str] = None
    config: Optional[str] = None
    requires_tag: Optional[str] = None
    license: str = ""
    files: list = field(default_factory=list)
    tokenizer: Optional[str] = None
    chat_template: Optional[str] = None
    engine_args: list = field(default_factory=list)
    default_tp: Optional[int] = None
    tp: dict = field(default_factory=dict)


@dataclass
class Registry:
    models: dict
    default: Optional[str]
    endpoint: str

    def resolve(self, name: Optional[str]) -> ModelEntry:
        key = name or self.default
        if key is None:
            raise RegistryError(["no model named and the registry has no default"])
        for m in self.models.values():
            if key == m.name or key in m.aliases:
                return m
        raise RegistryError([f"unknown model {key!r}; known: {', '.join(sorted(self.models))}"])


def builtin_path() -> Path:
    return Path(__file__).with_name("models.toml")


def user_path() -> Path:
    base = os.environ.get("XDG_CONFIG_HOME") or os.path.join(os.path.expanduser("~"), ".config")
    return Path(base) / "saber" / "models.toml"


def packs_root(override: Optional[str] = None) -> Path:
    if override:
        return Path(override)
    if os.environ.get("SABER_PACKS"):
        return Path(os.environ["SABER_PACKS"])
    base = os.environ.get("XDG_CACHE_HOME") or os.path.join(os.path.expanduser("~"), ".cache")
    return Path(base) / "saber" / "packs"


def _parse(doc: dict, origin: str, problems: list):
    out = {}
    if doc.get("schema", 1) != 1:
        problems.append(f"{origin}: schema {doc.get('schema')} is not supported (this build reads schema 1)")
    for i, raw in enumerate(doc.get("model", [])):
        where = f"{origin}: model[{i}]"
        name = raw.get("name")
        if not isinstance(name, str) or not _NAME.match(name):
            problems.append(f"{where}: name must use letters, digits, - _ . +")
            continue
        known = set(ModelEntry.__dataclass_fields__)
        for k in raw:
            if k not in known:
                problems.append(f"{where} ({name}): unknown key {k!r}")
        m = ModelEntry(**{k: v for k, v in raw.items() if k in known and k != "tp"})
        if m.kind not in ("target", "drafter"):
            problems.append(f"{where} ({name}): kind must be 'target' or 'drafter'")
        for tp_s, t in (raw.get("tp") or {}).items():
            try:
                tp = int(tp_s)
            except ValueError:
                tp = -1
            if tp not in VALID_TP:
                problems.append(f"{where} ({name}): tp.{tp_s} is not one of {VALID_TP}")
                continue
            tk = set(TpEntry.__dataclass_fields__)
            for k in t:
                if k not in tk:
                    problems.append(f"{where} ({name}) tp.{tp}: unknown key {k!r}")
            e = TpEntry(tp=tp, **{k: v for k, v in t.items() if k in tk and k != "tp"})
            if m.kind == "target":
                if e.max_ctx <= 0 or e.max_seqs <= 0:
                    problems.append(f"{where} ({name}) tp.{tp}: max_ctx and max_seqs are required")
                bs = [int(x) for x in e.decode_batches.split(",") if x] if e.decode_batches else []
                if any(b > e.max_seqs for b in bs):
                    problems.append(f"{where} ({name}) tp.{tp}: a decode batch exceeds max_seqs")
            m.tp[tp] = e
        if not m.tp:
            problems.append(f"{where} ({name}): needs at least one [model.tp.N] table")
        if m.tokenizer and m.tokenizer not in m.files:
            problems.append(f"{where} ({name}): tokenizer must be one of files")
        if m.chat_template and m.chat_template not in m.files:
            problems.append(f"{where} ({name}): chat_template must be one of files")
        out[name] = m
    return out


def load(user_file: Optional[Path] = None, builtin: Optional[Path] = None) -> Registry:
    problems: list = []
    base = tomllib.loads((builtin or builtin_path()).read_text())
    models = _parse(base, "models.toml", problems)
    default, endpoint = base.get("default"), base.get("endpoint", "https://huggingface.co")
    uf = user_file if user_file is not None else user_path()
    if uf.exists():
        try:
            udoc = tomllib.loads(uf.read_text())
            models.update(_parse(udoc, str(uf), problems))
            default = udoc.get("default", default)
        except tomllib.TOMLDecodeError as exc:
            problems.append(f"{uf}: {exc}")
    seen = {}
    for m in models.values():
        for a in [m.name] + m.aliases:
            if a in seen and seen[a] != m.name:
                problems.append(f"alias {a!r} is used by both {seen[a]} and {m.name}")
            seen[a] = m.name
    for m in models.values():
        if m.drafter and m.drafter not in seen:
            problems.append(f"{m.name}: drafter {m.drafter!r} is not in the registry")
    if default and default not in seen:
        problems.append(f"default {default!r} is not in the registry")
    if problems:
        raise RegistryError(problems)
    return Registry(models, default, os.environ.get("HF_ENDPOINT", endpoint))


def visible_gpus() -> int:
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def choose_tp(m: ModelEntry, want: Optional[int], gpus: Optional[int] = None) -> int:
    if want is not None:
        if want not in m.tp:
            raise RegistryError([f"{m.name} has no tp {want} pack (available: {sorted(m.tp)})"])
        return want
    gpus = visible_gpus() if gpus is None else gpus
    if gpus == 0:
        return m.default_tp if m.default_tp in m.tp else max(m.tp)
    fit = [t for t in m.tp if t <= gpus]
    if not fit:
        raise RegistryError([f"{m.name} needs at least {min(m.tp)} GPUs, {gpus} visible"])
    return max(fit)


def pack_dir(m: ModelEntry, tp: int, root: Optional[str] = None) -> Path:
    r = packs_root(root)
    for legacy in m.tp[tp].legacy_dirs:
        if (r / legacy).is_dir():
            return r / legacy
    return r / m.repo / m.tp[tp].path


def plan_serve(reg: Registry, model: Optional[str], tp: Optional[int] = None, port: int = 8000,
               packs: Optional[str] = None, extra: Optional[list] = None, gpus: Optional[int] = None) -> dict:
    m = reg.resolve(model)
    if m.kind != "target":
        raise RegistryError([f"{m.name} is a drafter; serve a target"])
    t = choose_tp(m, tp, gpus)
    e = m.tp[t]
    d = pack_dir(m, t, packs)
    argv = ["saber", "engine", "--engine", "real", "--engine-tp", str(t), "--pack", str(d),
            "--engine-config", m.config or m.name, "--engine-max-ctx", str(e.max_ctx),
            "--engine-max-seqs", str(e.max_seqs)]
    if e.prefill_rows:
        argv += ["--engine-prefill-rows", e.prefill_rows]
    if e.decode_batches:
        argv += ["--engine-decode-batches", e.decode_batches]
    argv += ["--engine-decode-widths", e.decode_widths, "--engine-draft-block", str(e.draft_block)]
    if e.budget_mib:
        argv += ["--engine-budget-mib", str(e.budget_mib)]
    argv += list(m.engine_args) + ["--served-model-name", m.served_id or m.name, "--port", str(port)]
    if m.tokenizer:
        argv += ["--tokenizer", str(d.parent / m.tokenizer)]
    if m.chat_template:
        argv += ["--chat-template", str(d.parent / m.chat_template)]
    argv += list(e.tail_args) + list(extra or [])
    return {"model": m.name, "tp": t, "pack_dir": str(d), "pack_present": (d / "manifest.json").exists(),
            "requires_tag": m.requires_tag, "argv": argv}


def pull(reg: Registry, model: Optional[str], tp: Optional[int] = None, packs: Optional[str] = None,
         dry_run: bool = False) -> dict:
    """Fetch a pack from the entry's endpoint. `file://` mirrors are copied; https needs network
    access (curl), which this function reports instead of hiding."""
    m = reg.resolve(model)
    t = choose_tp(m, tp, gpus=0 if tp is None else None)
    dst = pack_dir(m, t, packs)
    endpoint = m.endpoint or reg.endpoint
    src = f"{endpoint.rstrip('/')}/{m.repo}/resolve/{m.revision}/{m.tp[t].path}"
    plan = {"model": m.name, "tp": t, "from": src, "to": str(dst), "bytes": m.tp[t].bytes}
    if dry_run:
        return plan
    if endpoint.startswith("file://"):
        root = Path(endpoint[7:]) / m.repo / m.tp[t].path
        if not root.is_dir():
            raise RegistryError([f"mirror has no {root}"])
        dst.mkdir(parents=True, exist_ok=True)
        for f in root.iterdir():
            shutil.copy2(f, dst / f.name)
        for f in m.files:
            if (root.parent / f).exists():
                shutil.copy2(root.parent / f, dst.parent / f)
        from ..pack import format as PF
        problems = PF.check_manifest(dst)
        if problems:
            raise RegistryError([f"pulled pack is inconsistent: {p}" for p in problems])
        plan["verified"] = True
        return plan
    raise RegistryError([f"pulling from {endpoint} needs network access; use a file:// mirror or copy the pack to {dst}"])


def remove(reg: Registry, model: str, tp: Optional[int] = None, packs: Optional[str] = None, dry_run: bool = False) -> list:
    m = reg.resolve(model)
    gone = []
    for t in ([tp] if tp else sorted(m.tp)):
        d = pack_dir(m, t, packs)
        if d.is_dir():
            gone.append(str(d))
            if not dry_run:
                shutil.rmtree(d)
    return gone
