"""`parallax serve` with an in-box topology (pipeline stages, expert-parallel lanes) as real processes on CPU
over gloo: rank 0 serves the OpenAI API, the other ranks are spawned by the launcher."""

import json
import os
import signal
import subprocess
import sys
import time
import urllib.request

import pytest

from parallax_b200.parallel.launcher import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _post(port: int, body: dict, timeout: float = 120.0) -> dict:
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


@pytest.mark.parametrize("model,topo", [("tiny", ["--pp-size", "2"]),
                                        ("tiny-moe", ["--ep-size", "2", "--enable-dp-attention"])])
def test_serve_with_in_box_topology(model, topo, tmp_path):
    port = free_port()
    log = open(tmp_path / "serve.log", "w")
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    proc = subprocess.Popen([sys.executable, "-m", "parallax_b200.launch", "--model-path", model, "--random-init", "--port",
                             str(port), "--host", "127.0.0.1", "--max-batch-size", "4", "--max-sequence-length", "256",
                             "--log-level", "WARNING"] + topo, cwd=ROOT, env=env, stdout=log, stderr=subprocess.STDOUT,
                            start_new_session=True)
    try:
        deadline = time.time() + 120
        up = False
        while time.time() < deadline and proc.poll() is None:
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/models", timeout=2) as r:
                    up = r.status == 200
                    break
            except OSError:
                time.sleep(0.5)
        assert up, open(tmp_path / "serve.log").read()[-3000:]
        body = {"model": model, "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0}
        a = _post(port, body)
        b = _post(port, body)
        assert a["usage"]["completion_tokens"] >= 1
        assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
        # constrained decoding runs on the rank that samples (the last stage, or every expert-parallel lane)
        schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"]}
        c = _post(port, dict(body, max_tokens=80,
                             response_format={"type": "json_schema", "json_schema": {"name": "x", "schema": schema}}))
        assert isinstance(json.loads(c["choices"][0]["message"]["content"])["ok"], bool)
    finally:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGTERM)      # the server and the ranks it spawned share this process group
            try:
                proc.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(proc.pid, signal.SIGKILL)
        log.close()
