"""The daily reader: a mirror log and a replay file in, the comparison and the six stop conditions
out.  Per exchange (matched by the mirror's id) it compares the status and whether each side SERVED
the request (2xx, body complete, no error event, no abort finish), the usage counts (prompt_tokens
must be identical: the template is byte-identical), and for greedy requests the ids (token_ids when
the reply carries them, else the decoded text, reasoning and tool calls).  Identity is REPORTED, not
a stop.  The stops, each CLEAR, FIRED (with the evidence) or NOT CHECKED (with what was missing):

  1  a census counter that must read 0 moved during the replay
  2  the recorded side served (2xx) and the replayed side refused or aborted
  3  usage.prompt_tokens differs
  4  the engine exited other than by the window's SIGTERM, logged a CUDA error, or never listened
  5  a GPU power limit other than the expected one, or foreign traffic on the replayed port
  6  the mirror changed what a client received (received and forwarded hashes differ)

Parity: `crates/saber-shadow/src/report.rs:1-22,643-800`.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Optional

from .record import blob_bytes, parse_response, read_lines

# engine and scheduler counters of this build that only move when something went wrong
MUST_BE_ZERO = ("saber:engine_forward_errors_total", "saber:engine_undeclared_shapes_total",
                "saber:engine_kernel_wait_timeouts_total", "saber:sched_fatal_total", "saber:sched_restore_failures_total",
                "saber:sched_park_refusals_total", "saber:engine_argmax_fallbacks_total")


@dataclass
class Verdict:
    status: str                 # CLEAR | FIRED | NOT CHECKED
    detail: str = ""


@dataclass
class Report:
    recorded: int = 0
    replayed: int = 0
    pace: str = ""
    prod_not_served: int = 0
    saber_not_served: int = 0
    status_identical: int = 0
    greedy_compared: int = 0
    greedy_identical: int = 0
    content_identical: int = 0
    usage_compared: int = 0
    finish_table: dict = field(default_factory=dict)
    latency: dict = field(default_factory=dict)
    census_moved: dict = field(default_factory=dict)
    stops: list = field(default_factory=list)

    @property
    def fired(self) -> list:
        return [i + 1 for i, (_, v) in enumerate(self.stops) if v.status == "FIRED"]

    def render(self) -> str:
        out = [f"recorded {self.recorded}, replayed {self.replayed} ({self.pace})",
               f"not served: recorded side {self.prod_not_served}, replayed side {self.saber_not_served}; status identical {self.status_identical}",
               f"greedy: {self.greedy_identical} of {self.greedy_compared} identical; content identical {self.content_identical}; usage compared {self.usage_compared}",
               f"finish reasons (recorded -> replayed): {json.dumps(self.finish_table, sort_keys=True)}",
               f"latency ms (parity is NOT read off these under replay): {json.dumps(self.latency)}"]
        if self.census_moved:
            out.append(f"census moved: {json.dumps(self.census_moved, sort_keys=True)}")
        for i, (name, v) in enumerate(self.stops):
            out.append(f"stop {i + 1}  {v.status:11s} {name}" + (f": {v.detail}" if v.detail else ""))
        return "\n".join(out)


def _pct(v: list) -> dict:
    if not v:
        return {"n": 0}
    v = sorted(v)
    at = lambda q: v[min(len(v) - 1, round(q * (len(v) - 1)))]
    return {"n": len(v), "p50": at(0.5), "p90": at(0.9), "p99": at(0.99)}


def read(log_path: str, replay_path: str, engine_log: Optional[str] = None, power_limits_w: Optional[dict] = None,
         expect_power_w: float = 1000.0, allowed_refusals: tuple = ()) -> Report:
    exchanges = {e["id"]: e for e in read_lines(log_path) if e.get("kind") == "exchange"}
    meta, end, answers = {}, {}, {}
    for line in read_lines(replay_path):
        if line.get("kind") == "replay_meta":
            meta = line
        elif line.get("kind") == "replay_end":
            end = line
        elif line.get("kind") == "answer":
            answers[line["id"]] = line
    r = Report(recorded=len(exchanges), replayed=len(answers), pace=f"{meta.get('pace', '?')} x{meta.get('speed', 1.0)}")
    refused, prompt_differs, not_transparent = [], [], []
    lat_a, lat_b, replayed_prompt, usage_unknown = [], [], 0, 0
    for xid, ex in exchanges.items():
        resp = ex["response"]
        if resp.get("rx_fnv") != resp.get("tx_fnv") and resp.get("complete"):
            not_transparent.append(xid)
        a = parse_response(resp)
        r.prod_not_served += int(not a["served"])
        lat_a.append(resp.get("total_ms", 0))
        ans = answers.get(xid)
        if ans is None:
            continue
        b = parse_response(ans["response"])
        lat_b.append(ans.get("total_ms", 0))
        r.saber_not_served += int(not b["served"])
        r.status_identical += int(a["status"] == b["status"])
        if a["served"] and not b["served"] and xid not in allowed_refusals:
            refused.append(f"{xid} (status {b['status']})")
        if a["usage"] and b["usage"]:
            r.usage_compared += 1
            if a["usage"].get("prompt_tokens") != b["usage"].get("prompt_tokens"):
                prompt_differs.append(f"{xid} ({a['usage'].get('prompt_tokens')} vs {b['usage'].get('prompt_tokens')})")
        if b["usage"]:
            replayed_prompt += int(b["usage"].get("prompt_tokens") or 0)
        else:
            usage_unknown += 1
        key = f"{','.join(a['finish']) or '-'} -> {','.join(b['finish']) or '-'}"
        r.finish_table[key] = r.finish_table.get(key, 0) + 1
        same_text = (a["content"], a["reasoning"], json.dumps(a["tool_calls"], sort_keys=True)) == \
                    (b["content"], b["reasoning"], json.dumps(b["tool_calls"], sort_keys=True))
        if a["served"] and b["served"]:
            r.content_identical += int(same_text)
            try:
                req = json.loads(blob_bytes(ex["request"]))
            except (ValueError, TypeError):
                req = {}
            if float(req.get("temperature", 1.0) or 0.0) < 1e-5:
                r.greedy_compared += 1
                if a["token_ids"] is not None and b["token_ids"] is not None:
                    r.greedy_identical += int(a["token_ids"] == b["token_ids"])
                else:
                    r.greedy_identical += int(same_text)
    r.latency = {"recorded": _pct(lat_a), "replayed": _pct(lat_b)}
    before, after = meta.get("metrics_before"), end.get("metrics_after")
    fam = lambda m, name: next((v for k, v in m.items() if k == name or k.startswith(name + "{")), None)
    # stop 1
    if before is None or after is None:
        s1 = Verdict("NOT CHECKED", "the replay did not scrape the target's /metrics")
    else:
        for k, v in after.items():
            d = v - before.get(k, 0.0)
            if k.startswith("saber:") and d and not any(t in k for t in ("request", "tokens", "seconds", "steps", "bucket")):
                r.census_moved[k] = d
        present = [n for n in MUST_BE_ZERO if fam(after, n) is not None]
        if not present:
            s1 = Verdict("NOT CHECKED", "the target's /metrics carries none of the must-be-zero counters")
        else:
            moved = [f"{n.split(':', 1)[1]} +{fam(after, n) - (fam(before, n) or 0.0):g}" for n in present
                     if fam(after, n) - (fam(before, n) or 0.0) != 0]
            s1 = Verdict("FIRED", "; ".join(moved)) if moved else Verdict("CLEAR")
    # stop 2, 3
    s2 = Verdict("NOT CHECKED", "nothing replayed") if not answers else \
        (Verdict("FIRED", "recorded side served, replayed side did not: " + ", ".join(refused)) if refused else Verdict("CLEAR"))
    s3 = Verdict("NOT CHECKED", "no exchange carried usage on both sides") if not r.usage_compared else \
        (Verdict("FIRED", "prompt_tokens differ: " + ", ".join(prompt_differs)) if prompt_differs else Verdict("CLEAR"))
    # stop 4
    if engine_log is None:
        s4 = Verdict("NOT CHECKED", "no engine log given")
    else:
        bad = []
        if "listening" not in engine_log and "ready" not in engine_log:
            bad.append("no `listening` line")
        if "stopped" not in engine_log:
            bad.append("no `stopped` line (not the window's SIGTERM)")
        bad += [f"`{n}` in the log" for n in ("saber: FATAL", "Traceback", "CUDA error", "illegal memory access", "Xid") if n in engine_log]
        s4 = Verdict("FIRED", "; ".join(bad)) if bad else Verdict("CLEAR")
    # stop 5
    bad, unchecked = [], []
    if not power_limits_w:
        unchecked.append("power limits not read")
    else:
        bad += [f"{gpu} at {w:g} W (want {expect_power_w:g})" for gpu, w in power_limits_w.items() if abs(w - expect_power_w) > 0.5]
    if before is not None and after is not None:
        d = lambda n: (fam(after, n) or 0.0) - (fam(before, n) or 0.0)
        seen = d("saber:request_success_total") + d("saber:request_refused_total")
        if seen > len(answers):
            bad.append(f"the target finished or refused {seen:g} requests and the replay sent {len(answers)}: foreign traffic on the port")
        if usage_unknown == 0 and d("saber:prompt_tokens_total") > replayed_prompt:
            bad.append(f"the target prefilled {d('saber:prompt_tokens_total'):g} prompt tokens and the replay's requests carry {replayed_prompt}: foreign traffic on the port")
    else:
        unchecked.append("foreign traffic not checked (no /metrics scrape)")
    s5 = Verdict("FIRED", "; ".join(bad)) if bad else (Verdict("CLEAR") if not unchecked else
         Verdict("NOT CHECKED", "; ".join(unchecked) + ("" if len(unchecked) == 2 else " (the rest is clear)")))
    # stop 6
    s6 = Verdict("NOT CHECKED", "no exchange recorded") if not exchanges else \
        (Verdict("FIRED", "the mirror changed what a client received: " + ", ".join(not_transparent)) if not_transparent else Verdict("CLEAR"))
    r.stops = [("a census counter that must read 0 moved", s1), ("recorded side served (2xx), replayed side refused or aborted", s2),
               ("usage.prompt_tokens differs", s3), ("the engine exited other than by SIGTERM, a CUDA error, or never listened", s4),
               (f"a power limit other than {expect_power_w:g} W, or foreign traffic on the port", s5),
               ("the mirror changed what a client received", s6)]
    return r
