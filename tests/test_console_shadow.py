"""Console (usage store, audit log, keys, `/v1` proxy, admin API) and the shadow tools (mirror, replay,
report) over the serving plane's own mock engine behind the real router, served on the loopback."""
import asyncio
import json
import os
import socket
import stat
import sys
import threading
import time

import pytest
import uvicorn
from starlette.testclient import TestClient

from saber_engine_b200.console.app import Console
from saber_engine_b200.console.audit import Audit
from saber_engine_b200.console.auth import KeyRing, Limiter
from saber_engine_b200.console.supervisor import Supervisor
from saber_engine_b200.console.usage import (SRC_ENGINE, SRC_PROXY, TTFT_BUCKETS, UsageRow, UsageStore,
                                             poll_engine_requests)
from saber_engine_b200.sched.mock import NullExecutor
from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
from saber_engine_b200.serve.server import ServerState, create_app
from saber_engine_b200.serve.tokenizer import ByteCodec
from saber_engine_b200.shadow import report as shadow_report
from saber_engine_b200.shadow.mirror import Mirror
from saber_engine_b200.shadow.record import Fnv, blob_bytes, blob_of, read_lines
from saber_engine_b200.shadow.replay import replay


def _serve(app):
    """Runs an ASGI app on a free loopback port in a thread; returns (base url, stop)."""
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(app, log_level="error", lifespan="on"))
    t = threading.Thread(target=lambda: asyncio.run(server.serve(sockets=[sock])), daemon=True)
    t.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.02)
    assert server.started

    def stop():
        server.should_exit = True
        t.join(timeout=5)
    return f"http://127.0.0.1:{port}", stop


@pytest.fixture()
def engine():
    sched = Scheduler(NullExecutor(seed=2, vocab=300), SchedulerConfig(max_seqs=8, max_ctx=4096, model_name="mock"))
    sched.spawn_step_loop()
    state = ServerState(sched, ByteCodec(300), model_name="mock", api_keys=["sk-engine"])
    url, stop = _serve(create_app(state))
    yield url, state
    stop()
    sched.shutdown()


# ------------------------------------------------------------------------------------ usage / audit / auth
def test_usage_rows_merge_and_rollups_stay_in_step(tmp_path):
    st = UsageStore(str(tmp_path / "u.db"), batch_ms=10)
    t0 = 1_700_000_000_000
    st.record(UsageRow("c1-1", t0, "m", "alice", "/v1/chat/completions", 200, 0, 0, 40.0, 1040.0, "", True, SRC_PROXY))
    st.record(UsageRow("c1-2", t0 + 5, "m", "bob", "/v1/completions", 500, 7, 0, None, 12.0, "", False, SRC_PROXY))
    assert st.flush()
    # the engine's view of the first request arrives later: same uid, merged, not counted twice
    st.record(UsageRow("c1-1", t0 + 900, "m", "", "chat", 200, 100, 51, None, None, "stop", True, SRC_ENGINE, "17"))
    assert st.flush()
    row = st.get("c1-1")
    assert (row.src, row.prompt_tokens, row.completion_tokens, row.ttft_ms, row.key, row.finish) == \
        (SRC_PROXY | SRC_ENGINE, 100, 51, 40.0, "alice", "stop")
    by_key = {r["key"]: r for r in st.summary(t0 - 1000, t0 + 2000, "m", by="key")}
    assert by_key["alice"]["requests"] == 1 and by_key["alice"]["completion_tokens"] == 51 and by_key["alice"]["errors"] == 0
    assert by_key["bob"]["errors"] == 1
    assert abs(by_key["alice"]["decode_tps_mean"] - 50.0) < 1e-6            # 50 tokens after the first in 1000 ms
    lo, hi = TTFT_BUCKETS.upper(TTFT_BUCKETS.index(40.0) - 1), TTFT_BUCKETS.upper(TTFT_BUCKETS.index(40.0))
    assert lo < 40.0 <= hi and by_key["alice"]["ttft_ms_p50"] == hi
    total = st.summary(t0 - 1000, t0 + 2000, "d")
    assert total[0]["requests"] == 2                                         # every grain agrees
    # the engine-poll fallback: a direct request gets its own row, a re-poll changes nothing
    ring = [{"id": 3, "created": t0 // 1000, "prompt_tokens": 5, "completion_tokens": 9, "status": "length", "kind": "completion"},
            {"id": 4, "created": t0 // 1000, "status": "running"},
            {"id": 17, "created": t0 // 1000, "prompt_tokens": 100, "completion_tokens": 51, "status": "stop", "client_ref": "c1-1"}]
    for _ in range(2):
        assert poll_engine_requests(st, ring, "boot9", "m") == 2
        assert st.flush()
    assert st.summary(t0 - 1000, t0 + 2000, "h")[0]["requests"] == 3
    assert st.get("e:boot9:3").completion_tokens == 9
    assert 'saber_console_requests_total{model="m",key="alice"} 1' in st.prometheus()
    assert st.prune(now_ms=t0 + 40 * 86_400_000) == 3 and st.summary(t0 - 1000, t0 + 2000, "d")[0]["requests"] == 3
    st.close()


def test_audit_log_is_owner_only_and_cut_in_half(tmp_path):
    a = Audit(str(tmp_path), max_lines=10)
    for i in range(11):
        a.log("admin", "config.apply", "POST /api/config/apply", 200, "127.0.0.1", f"v{i}")
    assert stat.S_IMODE(os.stat(a.path).st_mode) == 0o600
    tail = a.tail()
    assert 5 <= len(tail) <= 6 and tail[-1]["detail"] == "v10" and "ip" in tail[-1]
    a.log("console", "config.auto_rollback")
    assert a.tail(1)[0]["who"] == "console" and "ip" not in a.tail(1)[0]
    with open(a.path, "a") as f:
        f.write('{"torn')                                                    # a crash in mid-write
    assert a.tail(2)[-1]["who"] == "console"


def test_keys_are_hashed_checked_revoked_and_wrong_ones_lock_the_address_out():
    ring = KeyRing()
    secret = ring.issue("alice")
    assert secret not in json.dumps(ring.to_json()) and ring.check(secret) == "alice" and ring.check(secret + "x") is None
    with pytest.raises(ValueError):
        ring.issue("alice")
    assert KeyRing.from_json(ring.to_json()).check(secret) == "alice"
    assert ring.revoke("alice") and ring.check(secret) is None
    now = [0.0]
    lim = Limiter(max_fails=3, window_s=10, lock_s=30, clock=lambda: now[0])
    for _ in range(3):
        assert not lim.locked("1.2.3.4")
        lim.fail("1.2.3.4")
    assert lim.locked("1.2.3.4") and not lim.locked("5.6.7.8")
    now[0] = 31.0
    assert not lim.locked("1.2.3.4")


# ------------------------------------------------------------------------------------ proxy + admin API
def test_proxy_streams_unchanged_records_usage_and_the_engine_row_merges(engine, tmp_path):
    url, state = engine
    flag = tmp_path / "ready"
    sup = Supervisor(ready_probe=flag.exists, ready_timeout_s=3.0)
    con = Console(sup, str(tmp_path), url, admin_token="adm", engine_bearer="sk-engine",
                  usage=UsageStore(str(tmp_path / "u.db"), batch_ms=10))
    with TestClient(con.app()) as c:
        adm = {"Authorization": "Bearer adm"}
        assert c.get("/api/state").status_code == 401
        key = c.post("/api/keys", json={"label": "alice"}, headers=adm).json()["key"]
        body = {"model": "mock", "prompt": [1, 2, 3, 4, 5], "max_tokens": 12, "temperature": 0, "ignore_eos": True, "stream": True,
                "stream_options": {"include_usage": True}}
        assert c.post("/v1/completions", json=body, headers={"Authorization": "Bearer wrong"}).status_code == 401
        via = c.post("/v1/completions", json=body, headers={"Authorization": f"Bearer {key}"})
        assert via.status_code == 200 and via.headers["content-type"].startswith("text/event-stream")
        import requests
        direct = requests.post(url + "/v1/completions", json=body, headers={"Authorization": "Bearer sk-engine"})
        strip = lambda t: "".join(c["text"] for l in t.splitlines() if l.startswith("data:") and "[DONE]" not in l
                                  for c in json.loads(l[5:])["choices"])
        assert strip(via.text) == strip(direct.text) != ""                    # the same text (steps may cut it differently)
        assert con.usage.flush()
        rows = [r for r in con.usage.recent() if r["key"] == "alice"]
        assert len(rows) == 1 and rows[0]["status"] == 200 and rows[0]["stream"] and rows[0]["ttft_ms"] is not None
        assert rows[0]["completion_tokens"] == 12 and rows[0]["prompt_tokens"] == 5 and rows[0]["finish"] == "length"
        # the engine kept the console's reference: the fallback poll lands in the SAME row
        ring = requests.get(url + "/v1/requests", headers={"Authorization": "Bearer sk-engine"}).json()["data"]
        assert any(r.get("client_ref") == rows[0]["uid"] for r in ring)
        poll_engine_requests(con.usage, ring, "b1", "mock")
        assert con.usage.flush()
        s = {r["key"]: r for r in c.get("/api/usage/summary?hours=1&by=key", headers=adm).json()}
        assert s["alice"]["requests"] == 1 and s[""]["requests"] == 1         # alice once; the direct call once, unlabelled
        # a revoked key is refused; eight wrong keys lock the address out
        assert c.delete("/api/keys/alice", headers=adm).status_code == 200
        assert c.post("/v1/completions", json=body, headers={"Authorization": f"Bearer {key}"}).status_code == 401
        acts = [e["action"] for e in c.get("/api/audit", headers=adm).json()]
        assert acts == ["auth.key.issue", "auth.key.revoke"]
        assert key not in (tmp_path / "audit.jsonl").read_text()
        for _ in range(8):
            c.post("/v1/completions", json=body, headers={"Authorization": "Bearer nope"})
        assert c.post("/v1/completions", json=body, headers={"Authorization": "Bearer nope"}).status_code == 429
    con.usage.close()


def test_admin_api_applies_rolls_back_and_audits(tmp_path):
    flag = tmp_path / "ready"
    good = [sys.executable, "-c", f"import time, pathlib\npathlib.Path(r'{flag}').write_text('ok')\ntime.sleep(60)\n"]
    never = [sys.executable, "-c", "import time; time.sleep(60)"]
    sup = Supervisor(ready_probe=flag.exists, ready_timeout_s=3.0)
    con = Console(sup, str(tmp_path), "http://127.0.0.1:9", usage=UsageStore(str(tmp_path / "u.db")))
    with TestClient(con.app()) as c:
        assert c.post("/api/engine/start").status_code == 409                # nothing has reached ready yet
        assert c.post("/api/config/apply", json={"argv": "x"}).status_code == 400
        assert c.post("/api/config/apply", json={"argv": good, "note": "v1"}).json()["applied"]
        flag.unlink()
        sup.ready_timeout_s = 0.4
        r = c.post("/api/config/apply", json={"argv": never, "note": "v2"})
        assert r.status_code == 502 and not r.json()["applied"]
        sup.ready_timeout_s = 3.0
        assert c.get("/api/state").json()["state"] == "ready"                # auto-rollback to v1
        hist = c.get("/api/config/history").json()
        assert [h["reached_ready"] for h in hist] == [True, False]
        assert c.post("/api/config/rollback", json={"version": 2}).status_code == 404
        flag.unlink()
        assert c.post("/api/config/rollback", json={"version": 1}).json()["applied"]
        assert c.post("/api/engine/stop").json()["state"] == "stopped"
        acts = [(e["who"], e["action"], e.get("status", 0)) for e in c.get("/api/audit").json()]
        assert ("console", "config.auto_rollback", 0) in acts and ("local", "config.apply", 502) in acts
        assert acts[-1] == ("local", "engine.stop", 200)
        assert "config history" in c.get("/").text
        assert c.post("/v1/completions", json={}).status_code == 502         # nothing listens on the engine port
    sup.stop()
    con.usage.close()


# ------------------------------------------------------------------------------------ shadow
def test_mirror_is_transparent_replay_answers_and_the_reader_finds_planted_faults(engine, tmp_path):
    url, _ = engine
    mirror = Mirror(url, str(tmp_path / "log"))
    murl, stop = _serve(mirror.app())
    import requests
    hdr = {"Authorization": "Bearer sk-engine"}
    b1 = {"model": "mock", "prompt": [9, 8, 7], "max_tokens": 8, "temperature": 0, "ignore_eos": True, "stream": True,
          "stream_options": {"include_usage": True}}
    b2 = {"model": "mock", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0, "ignore_eos": True}
    try:
        got1 = requests.post(murl + "/v1/completions", json=b1, headers=hdr)
        want1 = requests.post(url + "/v1/completions", json=b1, headers=hdr)
        got2 = requests.post(murl + "/v1/chat/completions", json=b2, headers=hdr)
        strip = lambda t: "".join(c["text"] for l in t.splitlines() if l.startswith("data:") and "[DONE]" not in l
                                  for c in json.loads(l[5:])["choices"])
        assert got1.status_code == 200 and strip(got1.text) == strip(want1.text) != ""
        assert got2.status_code == 200 and got2.json()["usage"]["completion_tokens"] == 6
        assert requests.get(murl + "/v1/models", headers=hdr).status_code == 200   # forwarded, not recorded
        assert requests.post(murl + "/v1/completions", json=b1).status_code == 401  # the upstream's refusal, unchanged
        assert mirror.flush()
        health = requests.get(murl + "/shadow/health").json()
        assert health["recorded"] == 3 and health["forwarded"] == 4 and health["write_errors"] == 0
    finally:
        stop()
        mirror.close()
    log = mirror.log_path()
    lines = list(read_lines(log))
    ex = [l for l in lines if l["kind"] == "exchange"]
    assert lines[0]["kind"] == "start" and len(ex) == 3
    assert all(e["response"]["rx_fnv"] == e["response"]["tx_fnv"] and e["response"]["complete"] for e in ex)
    f = Fnv()
    f.update(got1.content)
    assert ex[0]["response"]["rx_fnv"] == f.hex() and json.loads(blob_bytes(ex[0]["request"])) == b1
    assert blob_bytes(blob_of(b"\xff\xfe")) == b"\xff\xfe"
    out = str(tmp_path / "replay.jsonl")
    asyncio.run(replay(log, url, out, pace="sequential", bearer="sk-engine"))
    rep = shadow_report.read(log, out, engine_log="listening on 127.0.0.1\nstopped\n", power_limits_w={"gpu0": 1000.0})
    text = rep.render()
    assert rep.replayed == 3 and rep.greedy_compared == 2 and rep.greedy_identical == 2, text
    # the unauthenticated exchange was refused on both sides the same way (the replay sends the key:
    # it is served there, which is not a stop)
    assert rep.fired == [], text
    assert [v.status for _, v in rep.stops][1:] == ["CLEAR"] * 5, text
    # planted faults: a forwarded-bytes hash that differs, a replayed side that did not serve, a CUDA error in the log
    bad_log, bad_out = str(tmp_path / "bad.jsonl"), str(tmp_path / "bad_replay.jsonl")
    with open(bad_log, "w") as fh:
        for l in lines:
            if l["kind"] == "exchange" and l["id"] == ex[1]["id"]:
                l = json.loads(json.dumps(l))
                l["response"]["tx_fnv"] = "0" * 16
            fh.write(json.dumps(l) + "\n")
    with open(bad_out, "w") as fh:
        for l in read_lines(out):
            if l.get("kind") == "answer" and l["id"] == ex[0]["id"]:
                l["response"]["status"] = 503
            fh.write(json.dumps(l) + "\n")
    rep2 = shadow_report.read(bad_log, bad_out, engine_log="listening\nCUDA error: x\n", power_limits_w={"gpu0": 700.0})
    assert rep2.fired == [2, 4, 5, 6], rep2.render()
    pace = asyncio.run(replay(log, url, str(tmp_path / "r2.jsonl"), pace="recorded", speed=50.0, bearer="sk-engine"))
    assert pace["exchanges"] == 3
