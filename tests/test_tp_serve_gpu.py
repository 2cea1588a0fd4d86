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
        try:                                                    # prompt log-probabilities need the whole vocabulary on one GPU
            _post(port, "/v1/completions", {**body, "prompt_logprobs": 1})
            refused = False
        except urllib.error.HTTPError as e:
            refused = e.code == 400
        assert refused
        assert _post(port, "/v1/completions", body)["choices"][0]["text"] == a      # the engine is still up
    finally:
        os.killpg(p.pid, signal.SIGINT)
        try:
            p.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(p.pid, signal.SIGKILL)
