"""Auxiliary subsystems on the CPU: session parking (byte-identical resume, corrupt images refused,
RAM -> drive demotion with the crash law), warm prompts, host trace, step ledger, memory valve,
rank watch with a fake rank process that exits 86."""
import subprocess
import sys
import time

import pytest

from saber_engine_b200.sched.mem_valve import MemValve
from saber_engine_b200.sched.mock import NullExecutor, reference_generation
from saber_engine_b200.sched.park import ParkError, ParkImage, ParkTier
from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
from saber_engine_b200.serve import fatal
from saber_engine_b200.serve.engine_api import EngineRequest, SamplingParams
from saber_engine_b200.utils.host_trace import HostTrace, StartupLedger, StepLedger


def _drain(sub):
    toks = []
    while True:
        ev = sub.events.get_nowait()
        if ev is None:
            return toks, False
        toks += ev.new_token_ids
        if ev.finished:
            return toks, True


def test_park_and_restore_resumes_byte_identically(tmp_path):
    ex = NullExecutor(vocab=997, max_seqs=2)
    sch = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=4096))
    sch.park_tier = ParkTier(ram_budget=1, directory=str(tmp_path))     # force the drive tier
    prompt = list(range(5, 45))
    sub = sch.submit(EngineRequest(prompt, SamplingParams(max_tokens=60, ignore_eos=True)))
    for _ in range(6):
        sch.step()
    got, done = _drain(sub)
    assert not done and len(got) > 0
    other = sch.submit(EngineRequest(list(range(100, 130)), SamplingParams(max_tokens=8, ignore_eos=True)))
    key = sch.park(sub.seq_id)
    assert key in sch.park_tier and sch.park_tier.counters["demoted_to_drive"] >= 0
    sch.run_until_idle()                       # the other request runs while the first is parked
    assert _drain(other)[1]
    assert sch.restore(key) == sub.seq_id
    sch.run_until_idle()
    rest, done = _drain(sub)
    assert done
    assert got + rest == reference_generation(prompt, 60, 997)


def test_corrupt_parked_image_is_refused_before_it_reaches_the_device(tmp_path):
    tier = ParkTier(ram_budget=1 << 30)
    img = ParkImage.build({"kind": "t"}, bytes(range(256)) * 100)
    tier.put("a", img)
    img.payload = img.payload[:100] + b"\x00" + img.payload[101:] if img.payload[100:101] != b"\x00" else img.payload[:100] + b"\x01" + img.payload[101:]
    with pytest.raises(ParkError, match="sha256"):
        tier.take("a")
    assert tier.counters["restore_failures"] == 1
    # truncated file on the drive tier
    t2 = ParkTier(ram_budget=0, directory=str(tmp_path))
    t2.put("b", ParkImage.build({"kind": "t"}, b"x" * 5000))
    t2.put("c", ParkImage.build({"kind": "t"}, b"y" * 5000))       # demotes b
    path = tmp_path / "b.park"
    assert path.exists() and not (tmp_path / ".b.park.tmp").exists()
    path.write_bytes(path.read_bytes()[:-10])
    with pytest.raises(ParkError, match="truncated"):
        t2.take("b")


def test_warm_prompts_fill_the_prefix_cache():
    ex = NullExecutor(vocab=997, max_seqs=2)
    sch = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=8192, prefix_cache_min_tokens=64, prefix_cache_interval=64))
    system = list(range(1, 400))
    assert sch.warm([system]) == 1
    before = sch.prefix.stats.hits
    sub = sch.submit(EngineRequest(system + [7, 8, 9], SamplingParams(max_tokens=4, ignore_eos=True)))
    sch.run_until_idle()
    toks, done = _drain(sub)
    assert done and toks == reference_generation(system + [7, 8, 9], 4, 997)
    assert sch.prefix.stats.hits == before + 1


def test_host_trace_is_free_when_off_and_named_when_on():
    ex = NullExecutor(vocab=997, max_seqs=1)
    sch = Scheduler(ex, SchedulerConfig(max_seqs=1, max_ctx=2048))
    sch.submit(EngineRequest([1, 2, 3], SamplingParams(max_tokens=5, ignore_eos=True)))
    sch.run_until_idle()
    assert sch.trace.steps == []
    sch.trace = HostTrace(True)
    sch.submit(EngineRequest([1, 2, 3], SamplingParams(max_tokens=5, ignore_eos=True)))
    sch.run_until_idle()
    s = sch.trace.summary()
    assert s["steps"] >= 2 and {"Plan", "Launch", "Accept"} <= set(s["mean_us"])
    with pytest.raises(KeyError):
        with sch.trace.phase("NotAPhase"):
            pass
    led = StartupLedger()
    with led.phase("boot"):
        with led.phase("weights"):
            pass
    assert "boot/weights" in led.render()


def test_step_ledger_writes_jsonl(tmp_path):
    path = tmp_path / "steps.jsonl"
    led = StepLedger(str(path))
    for i in range(10):
        led.record("decode", 8, 0.001 * (i + 1), device_ms=float(i))
    led.close()
    assert len(path.read_text().strip().splitlines()) == 10
    assert led.percentiles("device_ms")["p50"] == 5.0


def test_memory_valve_escalates_at_once_and_relaxes_with_hysteresis():
    avail = {"v": 64 << 30}
    v = MemValve(reader=lambda: avail["v"])
    assert v.poll() == "ok"
    avail["v"] = 7 << 30
    assert v.poll() == "park"
    avail["v"] = 9 << 30                    # above the park threshold but inside the hysteresis band
    assert v.poll() == "park"
    avail["v"] = 11 << 30                   # 8 GiB * 1.25 = 10 GiB cleared, demote still holds (< 16 GiB)
    assert v.poll() == "demote"
    avail["v"] = 3 << 30
    assert v.poll() == "refuse" and not v.admits()
    avail["v"] = 64 << 30
    assert v.poll() == "ok"


def test_rank_watch_sees_a_fake_rank_exit_86():
    """Failure detection without a GPU: the failing rank is a CPU-only child process."""
    fatal.reset_for_tests()
    child = subprocess.Popen([sys.executable, "-c",
                              "import sys, time; time.sleep(0.2); print('saber: FATAL rank 1: injected', file=sys.stderr); sys.exit(86)"],
                             stderr=subprocess.PIPE)
    seen = {}
    fatal.RankWatch(child, 1, lambda rank, reason: seen.update(rank=rank, reason=reason))
    for _ in range(100):
        if seen:
            break
        time.sleep(0.05)
    assert seen["rank"] == 1 and "FATAL rank 1: injected" in seen["reason"]
    assert child.returncode == fatal.EXIT_FATAL
    # the serving side turns it into the teardown law
    ex = NullExecutor(vocab=97, max_seqs=1)
    sch = Scheduler(ex, SchedulerConfig(max_seqs=1, max_ctx=512))
    sub = sch.submit(EngineRequest([1, 2, 3], SamplingParams(max_tokens=50, ignore_eos=True)))
    sch.step()
    sch.set_fatal(seen["reason"])
    evs = []
    while (ev := sub.events.get_nowait()) is not None:
        evs.append(ev)
    assert evs[-1].finished and "injected" in evs[-1].error
    fatal.reset_for_tests()


def test_prompt_store_survives_restart_and_obeys_the_crash_law(tmp_path):
    from saber_engine_b200.sched.prompt_store import PromptStore
    system = list(range(1, 700))
    tail = [9, 8, 7]

    def engine():
        ex = NullExecutor(vocab=997, max_seqs=2)
        sch = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=8192, prefix_cache_min_tokens=64, prefix_cache_interval=256))
        sch.prompt_store = PromptStore(str(tmp_path), min_tokens=64)
        return ex, sch

    ex1, s1 = engine()
    sub = s1.submit(EngineRequest(system + tail, SamplingParams(max_tokens=5, ignore_eos=True)))
    s1.run_until_idle()
    want, done = _drain(sub)
    assert done and want == reference_generation(system + tail, 5, 997)
    assert s1.prompt_store.counters["puts"] >= 1
    # a new process: empty prefix cache, the prefix comes back from the drive
    ex2, s2 = engine()
    assert len(s2.prompt_store.records) == s1.prompt_store.counters["puts"]
    sub2 = s2.submit(EngineRequest(system + [5, 5, 5], SamplingParams(max_tokens=5, ignore_eos=True)))
    s2.run_until_idle()
    got, done = _drain(sub2)
    assert done and got == reference_generation(system + [5, 5, 5], 5, 997)
    assert s2.prompt_store.counters["hits"] == 1
    prefilled = sum(rows for kind, _, rows in ex2.launch_log if kind == "prefill")
    assert prefilled < len(system) // 2                    # most of the prompt was not prefilled again
    # crash law: a record whose file is missing or truncated is dropped at boot, a torn index line too
    files = sorted(tmp_path.glob("*.prompt"))
    files[0].write_bytes(files[0].read_bytes()[:-7])
    with open(tmp_path / "index.jsonl", "a") as fh:
        fh.write('{"rec": {"key": "zz", "n_to')
    st = PromptStore(str(tmp_path), min_tokens=64)
    assert st.counters["dropped_at_boot"] >= 2 and files[0].stem not in st.records
    assert not any(p.name.startswith(".") for p in tmp_path.iterdir())      # no temporary files left behind


def test_rank_seams_merge_to_the_seam_of_the_whole_vocabulary():
    import numpy as np
    from saber_engine_b200.runtime.hybrid_executor import merge_rank_seams
    rng = np.random.default_rng(0)
    full = rng.normal(size=(3, 400)).astype(np.float32)
    ids, vals, lse = [], [], []
    for r in range(4):
        sh = full[:, r * 100:(r + 1) * 100]
        o = np.argsort(-sh, axis=1)[:, :8]
        ids.append(o + r * 100)
        vals.append(np.take_along_axis(sh, o, 1))
        lse.append(np.log(np.exp(sh).sum(1)))
    i, v, l = merge_rank_seams(np.stack(ids), np.stack(vals), np.stack(lse))
    want = np.argsort(-full, axis=1)[:, :8]
    assert (i == want).all() and np.allclose(v, np.take_along_axis(full, want, 1))
    assert np.allclose(l, np.log(np.exp(full).sum(1)), atol=1e-5)


def test_index_blob_carries_positions_successors_and_sampling_rows():
    """fill_blob on the CPU (a plain tensor stands in for the pinned blob): three-axis positions,
    next-token table, and the per-head-row sampling tables of decode and prefill buckets."""
    from types import SimpleNamespace

    import numpy as np
    import torch

    from saber_engine_b200.models.hybrid import BlobLayout, SeqStep, fill_blob
    lay = BlobLayout.make(M=16, nseq=2, max_blocks=4)
    dec = SimpleNamespace(layout=lay, blob_host=torch.zeros(lay.words, dtype=torch.int32), kind="decode")
    seqs = [SeqStep([5, 6, 7, 8], 40, 1, 0, [1, 2, 3], rope_delta=-3, sampling=(0.8, 20.0, 0.9, 0.0), uniforms=[0.1, 0.2, 0.3, 0.4]),
            SeqStep([9, 10, 11, 12], 7, 2, 2, [4])]
    fill_blob(dec, seqs, 16)
    a = dec.blob_host.numpy()
    f = a.view(np.float32)
    assert a[lay.pos: lay.pos + 4].tolist() == [37, 38, 39, 40] and a[lay.pos + 4: lay.pos + 8].tolist() == [7, 8, 9, 10]
    assert a[lay.next_ids: lay.next_ids + 8].tolist() == [6, 7, 8, -1, 10, 11, 12, -1]
    assert np.allclose(f[lay.samp: lay.samp + 4], [0.8, 20.0, 0.9, 0.0]) and np.allclose(f[lay.samp + 12: lay.samp + 16], [0.8, 20.0, 0.9, 0.0])
    assert np.allclose(f[lay.samp_u: lay.samp_u + 4], [0.1, 0.2, 0.3, 0.4])
    assert f[lay.samp + 16] == 0.0                         # the greedy sequence's rows keep temperature 0
    assert a[lay.slot_map + 1] == 3 * 16 + (41 % 16)       # KV slots follow the index, not the rotary position
    pre = SimpleNamespace(layout=lay, blob_host=torch.zeros(lay.words, dtype=torch.int32), kind="prefill")
    pos3 = [[0, 1, 2, 2, 2], [0, 1, 2, 2, 3], [0, 1, 2, 3, 2]]
    fill_blob(pre, [SeqStep([1, 2, 3, 4, 5], 0, 1, 0, [1], rope_pos=pos3, next_token=77),
                    SeqStep([6, 7], 0, 2, 0, [2], sampling=(1.0, 0.0, 1.0, 0.0), uniforms=[0.5])], 16)
    a = pre.blob_host.numpy()
    f = a.view(np.float32)
    assert a[lay.pos + 16: lay.pos + 21].tolist() == [0, 1, 2, 2, 3] and a[lay.pos + 32 + 3] == 3
    assert a[lay.next_ids: lay.next_ids + 7].tolist() == [2, 3, 4, 5, 77, 7, -1]
    assert f[lay.samp] == 0.0 and np.allclose(f[lay.samp + 4: lay.samp + 8], [1.0, 0.0, 1.0, 0.0]) and f[lay.samp_u + 1] == 0.5


def test_bounded_host_wait_returns_or_raises_by_its_deadline():
    """A fake of the failing call: an event that completes after a few polls, and one that never does."""
    import time
    from saber_engine_b200.runtime.device_rt import DeviceWaitTimeout, bounded_wait

    class Ev:
        def __init__(self, after):
            self.n, self.after = 0, after

        def query(self):
            self.n += 1
            return self.n > self.after
    assert bounded_wait(Ev(5), 1.0, "a step") < 0.5
    t0 = time.perf_counter()
    with pytest.raises(DeviceWaitTimeout) as ei:
        bounded_wait(Ev(10 ** 12), 0.15, "the decode step", spin_s=0.02)
    assert 0.15 <= time.perf_counter() - t0 < 1.0 and "decode step" in str(ei.value)
