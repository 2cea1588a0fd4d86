"""Supervisor over fake engine processes: readiness, auto-rollback of a config that never gets
ready, restart after a crash and after the teardown law's exit 86."""
import sys
import time

from saber_engine_b200.console.supervisor import Supervisor


def _engine(flag, ready_after=0.05, die_after=None, code=0, fatal=False):
    body = f"import sys, time, pathlib\ntime.sleep({ready_after})\npathlib.Path(r'{flag}').write_text('ok')\n"
    if die_after is not None:
        body += f"time.sleep({die_after})\n"
        if fatal:
            body += "print('saber: FATAL rank 1: injected', file=sys.stderr)\n"
        body += f"pathlib.Path(r'{flag}').unlink()\nsys.exit({code})\n"
    else:
        body += "time.sleep(60)\n"
    return [sys.executable, "-c", body]


def test_apply_ready_rollback_and_history(tmp_path):
    flag = tmp_path / "ready"
    sup = Supervisor(ready_probe=flag.exists, ready_timeout_s=3.0, history_path=str(tmp_path / "h.json"))
    assert sup.apply(_engine(flag), note="v1")
    assert sup.state == "ready"
    flag.unlink()
    never = [sys.executable, "-c", "import time; time.sleep(60)"]        # never becomes ready
    sup.ready_timeout_s = 0.5
    assert not sup.apply(never, note="v2")
    sup.ready_timeout_s = 3.0
    assert sup.state == "ready"                                            # rolled back to v1 and ready again
    assert [c.reached_ready for c in sup.history] == [True, False]
    assert "rolled back" in sup.history[1].note and (tmp_path / "h.json").exists()
    sup.drain_and_stop(lambda: True)
    assert sup.state == "stopped"


def test_crash_and_fatal_86_are_restarted(tmp_path):
    flag = tmp_path / "ready"
    sup = Supervisor(ready_probe=flag.exists, ready_timeout_s=3.0, backoff_s=0.01)
    assert sup.apply(_engine(flag, die_after=0.2, code=86, fatal=True))
    seen = set()
    for _ in range(200):
        seen.add(sup.poll())
        if sup.last_fatal and sup.state == "ready":
            break
        time.sleep(0.02)
    assert "injected" in (sup.last_fatal or "")
    assert any(s == "fatal-86" for _, s, _ in sup.events)
    assert sup.state == "ready"                                            # restarted by the supervisor
    sup.stop()
    sup2 = Supervisor(ready_probe=flag.exists, ready_timeout_s=3.0, backoff_s=0.01, max_restarts=1)
    assert sup2.apply(_engine(flag, die_after=0.1, code=3))
    for _ in range(200):
        sup2.poll()
        if any(s == "crashed" for _, s, _ in sup2.events) and sup2.restarts >= 0 and sup2.state in ("ready", "crashed"):
            if len([1 for _, s, _ in sup2.events if s == "crashed"]) >= 1:
                break
        time.sleep(0.02)
    assert any(s == "crashed" for _, s, _ in sup2.events)
    sup2.stop()
