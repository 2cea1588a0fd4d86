"""Persistent usage history of the console: one SQLite database (WAL), one row per request, rollups
per minute / hour / day kept exactly in step with the rows.

* Rows are keyed by a uid: the proxy's reference for a proxied request (the proxy tags the engine
  request with it, and the engine keeps it in its `/v1/requests` ring), or `e:<engine boot>:<id>` for
  a request that reached the engine directly and was found by the fallback poll.  A proxied request
  is seen by BOTH paths and lands in the same row: the second arrival MERGES into the first (the
  proxy's timings and status, the engine's token counts), so nothing is counted twice.
* Rollups per (bucket, model, key): requests, errors, tokens, sums for the means and log-bucket
  histograms for the quantiles (TTFT, decode tok/s).  Every insert or merge subtracts the row's old
  contribution and adds the new one in the same transaction.  Raw rows are pruned after the
  retention period; rollups are kept, and long-range queries read only them.
* Writes go through ONE writer thread that batches them into a transaction; callers only enqueue.
* No prompt or reply text is stored.

Parity: `crates/saber-console/src/usage.rs:1-22` (rows, merge, rollups in step, writer thread),
`:38-60` (log-bucket histogram layout).
"""
from __future__ import annotations

import json
import math
import queue
import sqlite3
import threading
import time
from dataclasses import asdict, dataclass, field
from typing import Optional

MINUTE_MS, HOUR_MS, DAY_MS = 60_000, 3_600_000, 86_400_000
SRC_PROXY, SRC_ENGINE = 1, 2
GRAINS = (("m", MINUTE_MS), ("h", HOUR_MS), ("d", DAY_MS))


@dataclass(frozen=True)
class LogBuckets:
    """Bucket 0 = (0, base], bucket i = (base r^(i-1), base r^i] with r = 2^(1/per_octave); the last is open."""
    base: float
    per_octave: int
    n: int

    def index(self, x: float) -> int:
        if not x > self.base:
            return 0
        return min(self.n - 1, int(math.ceil(math.log2(x / self.base) * self.per_octave - 1e-9)))

    def upper(self, i: int) -> float:
        return self.base * 2.0 ** (i / self.per_octave)

    def quantile(self, counts: list, q: float) -> Optional[float]:
        total = sum(counts)
        if total <= 0:
            return None
        want, seen = q * total, 0
        for i, c in enumerate(counts):
            seen += c
            if seen >= want and c:
                return self.upper(i)
        return self.upper(self.n - 1)


TTFT_BUCKETS = LogBuckets(1.0, 4, 82)        # ms: 1 ms .. ~18 min
TPS_BUCKETS = LogBuckets(0.1, 4, 72)         # decode tokens / s: 0.1 .. ~22k


@dataclass
class UsageRow:
    uid: str
    ts_ms: int
    model: str = ""
    key: str = ""                   # the credential's label, never the secret
    route: str = ""
    status: int = 0                 # HTTP status; 499 = the client went away first
    prompt_tokens: int = 0
    completion_tokens: int = 0
    ttft_ms: Optional[float] = None
    total_ms: Optional[float] = None
    finish: str = ""
    stream: bool = False
    src: int = SRC_PROXY
    engine_id: str = ""

    @property
    def error(self) -> bool:
        return self.status >= 400 or self.status == 0

    @property
    def decode_tps(self) -> Optional[float]:
        if self.total_ms is None or self.completion_tokens < 2:
            return None
        t = self.total_ms - (self.ttft_ms or 0.0)
        return (self.completion_tokens - 1) * 1000.0 / t if t > 0 else None


def merge_rows(old: UsageRow, new: UsageRow) -> UsageRow:
    """Both views of one request in one row: the proxy's timings and status win, the engine's token
    counts fill what the proxy could not read (a reply without a usage block)."""
    px, en = (old, new) if old.src & SRC_PROXY else (new, old)
    if not (px.src & SRC_PROXY):          # two engine views (a re-poll): the later one wins
        out = UsageRow(**asdict(new))
        out.src = old.src | new.src
        return out
    out = UsageRow(**asdict(px))
    out.src = old.src | new.src
    out.prompt_tokens = px.prompt_tokens or en.prompt_tokens
    out.completion_tokens = px.completion_tokens or en.completion_tokens
    out.finish = px.finish or en.finish
    out.engine_id = px.engine_id or en.engine_id
    out.model = px.model or en.model
    return out


SCHEMA = """
CREATE TABLE IF NOT EXISTS rows (uid TEXT PRIMARY KEY, ts_ms INTEGER, body TEXT);
CREATE INDEX IF NOT EXISTS rows_ts ON rows (ts_ms);
CREATE TABLE IF NOT EXISTS rollup (grain TEXT, bucket INTEGER, model TEXT, key TEXT, requests INTEGER, errors INTEGER,
  prompt_tokens INTEGER, completion_tokens INTEGER, ttft_sum REAL, ttft_n INTEGER, tps_sum REAL, tps_n INTEGER,
  ttft_hist TEXT, tps_hist TEXT, PRIMARY KEY (grain, bucket, model, key));
"""


class UsageStore:
    def __init__(self, path: str, raw_retention_days: int = 30, batch_ms: int = 150):
        self.path, self.retention_days, self.batch_ms = path, raw_retention_days, batch_ms
        self._q: "queue.Queue[Optional[UsageRow]]" = queue.Queue()
        self._db = sqlite3.connect(path, check_same_thread=False)
        self._db.execute("PRAGMA journal_mode=WAL")
        self._db.executescript(SCHEMA)
        self._db.commit()
        self._dblock = threading.Lock()
        self.write_errors = 0
        self._idle = threading.Event()
        self._idle.set()
        self._t = threading.Thread(target=self._writer, name="usage-writer", daemon=True)
        self._t.start()

    # ---- request path: enqueue only
    def record(self, row: UsageRow) -> None:
        self._idle.clear()
        self._q.put(row)

    def flush(self, timeout: float = 5.0) -> bool:
        """Wait until the writer has drained what was queued before the call (tests, shutdown)."""
        return self._idle.wait(timeout)

    def close(self) -> None:
        self._q.put(None)
        self._t.join(timeout=5)
        with self._dblock:
            self._db.close()

    # ---- writer thread
    def _writer(self) -> None:
        while True:
            row = self._q.get()
            if row is None:
                return
            batch = [row]
            deadline = time.monotonic() + self.batch_ms / 1000.0
            stop = False
            while True:
                left = deadline - time.monotonic()
                if left <= 0:
                    break
                try:
                    nxt = self._q.get(timeout=left)
                except queue.Empty:
                    break
                if nxt is None:
                    stop = True
                    break
                batch.append(nxt)
            try:
                with self._dblock:
                    self._apply(batch)
            except sqlite3.Error:
                self.write_errors += 1        # a failure to record never fails a request
            if self._q.empty():
                self._idle.set()
            if stop:
                return

    def _contrib(self, cur, row: UsageRow, sign: int) -> None:
        tps = row.decode_tps
        for grain, ms in GRAINS:
            bucket = row.ts_ms // ms
            got = cur.execute("SELECT requests, errors, prompt_tokens, completion_tokens, ttft_sum, ttft_n, tps_sum, tps_n, "
                              "ttft_hist, tps_hist FROM rollup WHERE grain=? AND bucket=? AND model=? AND key=?",
                              (grain, bucket, row.model, row.key)).fetchone()
            if got is None:
                vals = [0, 0, 0, 0, 0.0, 0, 0.0, 0]
                th, ph = [0] * TTFT_BUCKETS.n, [0] * TPS_BUCKETS.n
            else:
                vals, th, ph = list(got[:8]), json.loads(got[8]), json.loads(got[9])
            vals[0] += sign
            vals[1] += sign * int(row.error)
            vals[2] += sign * row.prompt_tokens
            vals[3] += sign * row.completion_tokens
            if row.ttft_ms is not None:
                vals[4] += sign * row.ttft_ms
                vals[5] += sign
                th[TTFT_BUCKETS.index(row.ttft_ms)] += sign
            if tps is not None:
                vals[6] += sign * tps
                vals[7] += sign
                ph[TPS_BUCKETS.index(tps)] += sign
            cur.execute("INSERT OR REPLACE INTO rollup VALUES (?,?,?,?,?,?,?,?,?,?,?,?,?,?)",
                        (grain, bucket, row.model, row.key, *vals, json.dumps(th), json.dumps(ph)))

    def _apply(self, batch: list) -> None:
        cur = self._db.cursor()
        cur.execute("BEGIN")
        try:
            for row in batch:
                got = cur.execute("SELECT body FROM rows WHERE uid=?", (row.uid,)).fetchone()
                if got is not None:
                    old = UsageRow(**json.loads(got[0]))
                    self._contrib(cur, old, -1)
                    row = merge_rows(old, row)
                self._contrib(cur, row, +1)
                cur.execute("INSERT OR REPLACE INTO rows VALUES (?,?,?)", (row.uid, row.ts_ms, json.dumps(asdict(row))))
            cur.execute("COMMIT")
        except Exception:
            cur.execute("ROLLBACK")
            raise

    # ---- queries (rollups only, except `recent`)
    def prune(self, now_ms: Optional[int] = None) -> int:
        now_ms = int(time.time() * 1000) if now_ms is None else now_ms
        with self._dblock:
            n = self._db.execute("DELETE FROM rows WHERE ts_ms < ?", (now_ms - self.retention_days * DAY_MS,)).rowcount
            self._db.commit()
        return n

    def recent(self, limit: int = 50) -> list:
        with self._dblock:
            got = self._db.execute("SELECT body FROM rows ORDER BY ts_ms DESC LIMIT ?", (limit,)).fetchall()
        return [json.loads(b) for (b,) in got]

    def get(self, uid: str) -> Optional[UsageRow]:
        with self._dblock:
            got = self._db.execute("SELECT body FROM rows WHERE uid=?", (uid,)).fetchone()
        return UsageRow(**json.loads(got[0])) if got else None

    def summary(self, since_ms: int, until_ms: int, grain: str = "h", by: str = "model") -> list:
        """Totals per model (or key) over [since, until): reads the rollup of the given grain."""
        ms = dict(GRAINS)[grain]
        with self._dblock:
            got = self._db.execute("SELECT model, key, requests, errors, prompt_tokens, completion_tokens, ttft_sum, ttft_n, "
                                   "tps_sum, tps_n, ttft_hist, tps_hist FROM rollup WHERE grain=? AND bucket>=? AND bucket<?",
                                   (grain, since_ms // ms, (until_ms + ms - 1) // ms)).fetchall()
        agg: dict = {}
        for r in got:
            k = r[0] if by == "model" else r[1]
            a = agg.setdefault(k, {"requests": 0, "errors": 0, "prompt_tokens": 0, "completion_tokens": 0, "ttft_sum": 0.0,
                                   "ttft_n": 0, "tps_sum": 0.0, "tps_n": 0, "th": [0] * TTFT_BUCKETS.n, "ph": [0] * TPS_BUCKETS.n})
            for name, v in zip(("requests", "errors", "prompt_tokens", "completion_tokens", "ttft_sum", "ttft_n", "tps_sum", "tps_n"), r[2:10]):
                a[name] += v
            a["th"] = [x + y for x, y in zip(a["th"], json.loads(r[10]))]
            a["ph"] = [x + y for x, y in zip(a["ph"], json.loads(r[11]))]
        out = []
        for k, a in sorted(agg.items()):
            out.append({by: k, "requests": a["requests"], "errors": a["errors"], "prompt_tokens": a["prompt_tokens"],
                        "completion_tokens": a["completion_tokens"],
                        "ttft_ms_mean": a["ttft_sum"] / a["ttft_n"] if a["ttft_n"] else None,
                        "ttft_ms_p50": TTFT_BUCKETS.quantile(a["th"], 0.5), "ttft_ms_p99": TTFT_BUCKETS.quantile(a["th"], 0.99),
                        "decode_tps_mean": a["tps_sum"] / a["tps_n"] if a["tps_n"] else None,
                        "decode_tps_p50": TPS_BUCKETS.quantile(a["ph"], 0.5)})
        return out

    def prometheus(self) -> str:
        """Lifetime totals per (model, key) from the day rollup."""
        with self._dblock:
            got = self._db.execute("SELECT model, key, SUM(requests), SUM(errors), SUM(prompt_tokens), SUM(completion_tokens) "
                                   "FROM rollup WHERE grain='d' GROUP BY model, key").fetchall()
        lines = []
        for name, idx in (("requests", 2), ("errors", 3), ("prompt_tokens", 4), ("completion_tokens", 5)):
            lines.append(f"# TYPE saber_console_{name}_total counter")
            for r in got:
                lines.append(f'saber_console_{name}_total{{model="{r[0]}",key="{r[1]}"}} {r[idx]}')
        return "\n".join(lines) + "\n"


def poll_engine_requests(store: UsageStore, ring: list, engine_boot: str, model: str = "") -> int:
    """Fallback for requests that reached the engine directly: one row per FINISHED entry of the
    engine's `/v1/requests` ring.  An entry that carries a console reference merges into the
    proxy's row; a re-poll is a no-op (same uid, same contribution)."""
    n = 0
    for rec in ring:
        if rec.get("status") in (None, "running"):
            continue
        uid = rec.get("client_ref") or f"e:{engine_boot}:{rec['id']}"
        store.record(UsageRow(uid=uid, ts_ms=int(rec.get("created", 0)) * 1000, model=model, route=rec.get("kind", ""),
                              status=200 if rec.get("status") in ("stop", "length", "finished", "tool_calls") else 500,
                              prompt_tokens=rec.get("prompt_tokens", 0), completion_tokens=rec.get("completion_tokens", 0),
                              finish=str(rec.get("status", "")), stream=bool(rec.get("stream")), src=SRC_ENGINE,
                              engine_id=str(rec["id"])))
        n += 1
    return n
