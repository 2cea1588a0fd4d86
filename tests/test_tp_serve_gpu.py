"""Serving on two GPUs through the CLI (skipped on a single-GPU box): rank 0 serves, rank 1 follows."""
import json
import os
import signal
import subprocess
import sys
import time
import urllib.error
import urllib.request

import pytest
import torch

pytestmark = pytest.mark.gpu


def _post(port, path, body):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", json.dumps(body).encode(), {"content-type": "application/json"})
    return json.loads(urllib.request.urlopen(req, timeout=120).read())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_engine_serves_greedy_and_sampled_requests():
    port = 8100 + os.getpid() % 400
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.Popen([sys.executable, "-m", "saber_engine_b200", "engine", "--engine", "real", "--engine-config", "hybrid-mini",
                          "--random-init", "--engine-tp", "2", "--engine-max-ctx", "2048", "--engine-max-seqs", "4",
                          "--engine-decode-batches", "1,2,4", "--engine-prefill-rows", "64,256", "--port", str(port)],
                         env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, start_new_session=True)
    try:
        for _ in range(120):
            try:
                urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2)
                break
            except Exception:
                assert p.poll() is None, "the engine exited before it was ready"
                time.sleep(1)
        else:
            pytest.fail("the engine did not come up")
        body = {"prompt": "hello tensor parallel world", "max_tokens": 10, "temperature": 0}
        a = _post(port, "/v1/completions", body)["choices"][0]["text"]
        b = _post(port, "/v1/completions", body)["choices"][0]["text"]
        assert a == b and a
        s = _post(port, "/v1/completions", {**body, "temperature": 0.9, "seed": 4, "logprobs": 1})["choices"][0]
        assert len(s["logprobs"]["tokens"]) == 10
        # prompt log-probabilities on vocabulary shards: candidates and successor logits merged on the device
        plp = _post(port, "/v1/completions", {**body, "prompt_logprobs": 2})["choices"][0]["prompt_logprobs"]
        assert plp[0] is None and len(plp) > 2
        for e in plp[1:]:
            assert all(v["logprob"] <= 1e-3 and v["logprob"] > -60 for v in e.values())
        assert _post(port, "/v1/completions", body)["choices"][0]["text"] == a      # the engine is still up
    finally:
        os.killpg(p.pid, signal.SIGINT)
        try:
            p.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(p.pid, signal.SIGKILL)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_engine_parks_a_victim_on_both_ranks_and_restores_it():
    """A KV pool too small for two long requests: the running one is parked (every rank exports its own
    shard under the leader's park id), the waiting one runs, the victim comes back and ends with the ids of
    an undisturbed run."""
    import threading
    port = 8500 + os.getpid() % 400
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.Popen([sys.executable, "-m", "saber_engine_b200", "engine", "--engine", "real", "--engine-config", "hybrid-mini",
                          "--random-init", "--engine-tp", "2", "--engine-max-ctx", "2048", "--engine-max-seqs", "4",
                          "--engine-decode-batches", "1,2,4", "--engine-prefill-rows", "64,256", "--engine-kv-blocks", "112",
                          "--engine-park-victims", "--no-prefix-cache", "--port", str(port)],
                         env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, start_new_session=True)
    try:
        for _ in range(120):
            try:
                urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2)
                break
            except Exception:
                assert p.poll() is None, "the engine exited before it was ready"
                time.sleep(1)
        else:
            pytest.fail("the engine did not come up")
        # (111 usable pages of 16 tokens: the first request takes ~97 of them, the second needs ~41)
        a_body = {"prompt": "a long request that will be parked", "max_tokens": 1500, "temperature": 0, "ignore_eos": True}
        b_body = {"prompt": "the request that does not fit beside it", "max_tokens": 600, "temperature": 0, "ignore_eos": True}
        solo = _post(port, "/v1/completions", a_body)["choices"][0]["text"]
        got = {}
        ta = threading.Thread(target=lambda: got.update(a=_post(port, "/v1/completions", a_body)["choices"][0]["text"]))
        ta.start()
        time.sleep(0.1)
        got["b"] = _post(port, "/v1/completions", b_body)["choices"][0]["text"]
        ta.join(timeout=120)
        stats = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/stats", timeout=10).read())
        assert got["a"] == solo and got["b"]
        assert stats["victims_parked"] >= 1 and stats["victims_restored"] >= 1, stats
    finally:
        os.killpg(p.pid, signal.SIGINT)
        try:
            p.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(p.pid, signal.SIGKILL)
