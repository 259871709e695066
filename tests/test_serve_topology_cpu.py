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
# the tests below run up to five model processes at once on tiny models: two threads each is plenty, and it keeps
# them from fighting over the cores (inherited by every child process; torch is already loaded here)
os.environ.setdefault("OMP_NUM_THREADS", "2")


class _StartupError(AssertionError):
    """A server process of the test did not come up (port taken between picking and binding, a slow machine)."""


def _retry_startup(fn):
    """Process-level tests pick free ports before their servers bind them; on the rare collision the test is run
    once more with new ports instead of failing the run."""
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        try:
            return fn(*args, **kwargs)
        except _StartupError:
            tmp = kwargs.get("tmp_path")
            if tmp is not None:
                sub = tmp / "second_try"
                sub.mkdir()
                kwargs["tmp_path"] = sub
            return fn(*args, **kwargs)

    return wrapper


def _post(port: int, body: dict, timeout: float = 120.0) -> dict:
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def _probs(reply: dict) -> list:
    """The reply's fingerprint: the probability of every generated token (the text of a random-init model is mostly
    unprintable, so comparing contents would compare empty strings)."""
    probs = reply["choices"][0]["token_probs"]
    assert len(probs) == reply["usage"]["completion_tokens"] >= 1
    return [float(p) for p in probs]


def _close(a: list, b: list, rel: float = 2e-3) -> bool:
    return len(a) == len(b) and all(abs(x - y) <= rel * max(abs(x), abs(y)) for x, y in zip(a, b))


@pytest.mark.parametrize("model,topo", [("tiny", ["--pp-size", "2"]),
                                        ("tiny-moe", ["--ep-size", "2", "--enable-dp-attention"])])
@_retry_startup
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
        if not up:
            raise _StartupError(open(tmp_path / "serve.log").read()[-3000:])
        body = {"model": model, "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0, "return_probs": True}
        a = _post(port, body)
        b = _post(port, body)
        assert a["usage"]["completion_tokens"] >= 1
        assert _close(_probs(a), _probs(b))      # (the second time the prompt comes from the prefix cache)
        if model == "tiny":
            # online refit of the in-box server: every rank reloads its own layers from the blocks on disk
            import torch
            from safetensors.torch import save_file

            from parallax_b200.engine.engine import Engine
            from parallax_b200.models.config import named_config
            from parallax_b200.utils.weight_refit import calculate_cid
            from tests.test_engine_gpu import _export_weights

            other = Engine(named_config("tiny"), device="cpu", num_blocks=16, page_size=16, max_batch_size=2, seed=7)
            w = _export_weights(other)
            w.pop("lm_head.weight", None)
            f = tmp_path / "all.safetensors"
            save_file({k: v.contiguous() for k, v in w.items()}, str(f))
            cid = calculate_cid(f.read_bytes())
            req = urllib.request.Request(f"http://127.0.0.1:{port}/weight/refit", headers={"Content-Type": "application/json"},
                                         data=json.dumps({"index_map": {k: cid for k in w}, "paths": {cid: str(f)}}).encode())
            assert urllib.request.urlopen(req, timeout=60).status == 200
            c2 = _post(port, body)
            assert not _close(_probs(c2), _probs(a))
            # ... and the reply is the new model's
            from fastapi.testclient import TestClient

            from parallax_b200.engine.service import EngineLoop
            from parallax_b200.frontend.openai_api import create_app
            from parallax_b200.frontend.tokenizer import TokenizerWrapper

            ref_loop = EngineLoop(other)
            ref_loop.start()
            try:
                with TestClient(create_app(ref_loop, TokenizerWrapper.from_pretrained(None, vocab_size=1024), "tiny", 256)) as tc:
                    want = _probs(tc.post("/v1/chat/completions", json=body).json())
            finally:
                ref_loop.stop()
            assert _close(_probs(c2), want), (_probs(c2), want)
        # a burst of clients, half of which hang up mid-stream; the server then still answers as before
        import threading

        errors = []

        def client(i: int) -> None:
            try:
                b = dict(body, max_tokens=20, ignore_eos=True, stream=True,
                         messages=[{"role": "user", "content": f"client number {i} " * (1 + i % 3)}])
                rq = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=json.dumps(b).encode(),
                                            headers={"Content-Type": "application/json"})
                with urllib.request.urlopen(rq, timeout=120) as resp:
                    seen = 0
                    for line in resp:
                        if line.startswith(b"data: "):
                            seen += 1
                            if i % 2 == 0 and seen >= 3:
                                return
            except Exception as e:      # noqa: BLE001
                errors.append(repr(e))

        threads = [threading.Thread(target=client, args=(i,)) for i in range(8)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(150)
        assert not errors and not any(t.is_alive() for t in threads), errors
        after_burst = _post(port, body)
        assert after_burst["usage"]["completion_tokens"] == b["usage"]["completion_tokens"]
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


@_retry_startup
def test_two_nodes_with_manual_layer_ranges_and_no_scheduler(tmp_path):
    """`parallax serve --start-layer/--end-layer --initial-peers`: two processes, each with half of the layers,
    find each other over HTTP; the first one serves the API. Same reply as one process with all layers."""
    from parallax_b200.p2p.static_peers import StaticPeers

    p0, p1, p2 = free_port(), free_port(), free_port()
    env = dict(os.environ, PYTHONPATH=ROOT)
    common = [sys.executable, "-m", "parallax_b200.launch", "--model-path", "tiny", "--random-init", "--host", "127.0.0.1",
              "--max-batch-size", "4", "--max-sequence-length", "256", "--log-level", "WARNING"]
    logs = [open(tmp_path / f"n{i}.log", "w") for i in range(3)]
    procs = [
        subprocess.Popen(common + ["--port", str(p0), "--start-layer", "0", "--end-layer", "2", "--initial-peers",
                                   f"127.0.0.1:{p1}"], cwd=ROOT, env=env, stdout=logs[0], stderr=subprocess.STDOUT),
        subprocess.Popen(common + ["--port", str(p1), "--start-layer", "2", "--end-layer", "4", "--initial-peers",
                                   f"http://127.0.0.1:{p0}"], cwd=ROOT, env=env, stdout=logs[1], stderr=subprocess.STDOUT),
        subprocess.Popen(common + ["--port", str(p2)], cwd=ROOT, env=env, stdout=logs[2], stderr=subprocess.STDOUT),
    ]
    try:
        for port, path in ((p0, "/v1/models"), (p1, "/peer/info"), (p2, "/v1/models")):
            deadline = time.time() + 120
            up = False
            while time.time() < deadline and all(p.poll() is None for p in procs):
                try:
                    with urllib.request.urlopen(f"http://127.0.0.1:{port}{path}", timeout=2) as r:
                        up = r.status == 200
                        break
                except OSError:
                    time.sleep(0.5)
            if not up:
                raise _StartupError("".join(open(tmp_path / f"n{i}.log").read()[-1500:] for i in range(3)))
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 8, "temperature": 0, "return_probs": True}
        split = _post(p0, body)
        whole = _post(p2, body)
        assert split["usage"]["completion_tokens"] == whole["usage"]["completion_tokens"] >= 1
        assert _close(_probs(split), _probs(whole)), (_probs(split), _probs(whole))
        with urllib.request.urlopen(f"http://127.0.0.1:{p1}/peer/info", timeout=5) as r:
            info = json.loads(r.read())
        assert (info["start_layer"], info["end_layer"]) == (2, 4) and f"http://127.0.0.1:{p0}" in info["peers"]
    finally:
        for p in procs:
            if p.poll() is None:
                p.terminate()
        for p in procs:
            try:
                p.wait(15)
            except subprocess.TimeoutExpired:
                p.kill()
        for f in logs:
            f.close()

    # the chain is found through peers of peers, and a gap is reported as "no route yet"
    net = {"http://a/peer/info": {"node_id": "a", "url": "http://a", "start_layer": 0, "end_layer": 3, "peers": ["http://b"]},
           "http://b/peer/info": {"node_id": "b", "url": "http://b", "start_layer": 3, "end_layer": 5, "peers": ["http://c"]},
           "http://c/peer/info": {"node_id": "c", "url": "http://c", "start_layer": 5, "end_layer": 8, "peers": []}}
    me = StaticPeers("a", "http://a", 0, 3, ["http://b"], http_get=lambda u: net[u])
    assert me.route(8) == ["a", "b", "c"] and me.node_addresses()["c"] == "http://c"
    assert me.route(9) is None


@pytest.mark.parametrize("model", ["tiny-hybrid", "tiny+lora"])
@_retry_startup
def test_two_nodes_each_tensor_parallel_over_two_ranks(model, tmp_path):
    """Two pipeline peers without a scheduler, each running its half of the layers tensor-parallel over two
    processes (`--tp-size 2`): rank 0 of a node owns the peer executor and hands every batch to its follower
    through the node's control channel. Same reply as one process with all layers."""
    p0, p1, p2 = free_port(), free_port(), free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    lora_flags, adapter = [], None
    if model.endswith("+lora"):
        # per-request adapters on tensor-parallel nodes: every rank keeps its slice, loads travel as commands
        from parallax_b200.models.config import named_config
        from tests.test_lora_cpu import _make_adapter

        model = model.split("+")[0]
        root = tmp_path if tmp_path.name != "second_try" else tmp_path.parent
        paths = {n: (str(root / n) if (root / n).exists() else _make_adapter(named_config(model), root / n, seed))
                 for seed, n in enumerate(("x", "y"), 1)}
        lora_flags = ["--enable-lora", "--lora-paths"] + [f"{n}={d}" for n, d in paths.items()]
        adapter = "x"
    common = [sys.executable, "-m", "parallax_b200.launch", "--model-path", model, "--random-init", "--host", "127.0.0.1",
              "--max-batch-size", "4", "--max-sequence-length", "256", "--log-level", "WARNING"]
    common = common + lora_flags
    logs = [open(tmp_path / f"n{i}.log", "w") for i in range(3)]
    kw = dict(cwd=ROOT, env=env, stderr=subprocess.STDOUT, start_new_session=True)
    procs = [
        subprocess.Popen(common + ["--port", str(p0), "--start-layer", "0", "--end-layer", "2", "--tp-size", "2",
                                   "--initial-peers", f"127.0.0.1:{p1}"], stdout=logs[0], **kw),
        subprocess.Popen(common + ["--port", str(p1), "--start-layer", "2", "--end-layer", "4", "--tp-size", "2",
                                   "--initial-peers", f"127.0.0.1:{p0}"], stdout=logs[1], **kw),
        subprocess.Popen(common + ["--port", str(p2)], stdout=logs[2], **kw),
    ]
    try:
        for port, path in ((p0, "/v1/models"), (p1, "/peer/info"), (p2, "/v1/models")):
            deadline = time.time() + 150
            up = False
            while time.time() < deadline and all(p.poll() is None for p in procs):
                try:
                    with urllib.request.urlopen(f"http://127.0.0.1:{port}{path}", timeout=2) as r:
                        up = r.status == 200
                        break
                except OSError:
                    time.sleep(0.5)
            if not up:
                raise _StartupError("".join(open(tmp_path / f"n{i}.log").read()[-2000:] for i in range(3)))
        for content, n in (("hello there", 8), ("a much longer prompt " * 6, 5)):
            body = {"model": model, "messages": [{"role": "user", "content": content}], "max_tokens": n, "temperature": 0, "return_probs": True}
            if adapter is not None:
                plain = _probs(_post(p0, body))
                body["lora_path"] = adapter
            split, whole = _post(p0, body), _post(p2, body)
            assert split["usage"]["completion_tokens"] == whole["usage"]["completion_tokens"] >= 1
            assert _close(_probs(split), _probs(whole)), (_probs(split), _probs(whole))
            if adapter is not None:
                assert not _close(_probs(split), plain)        # the adapter changes the reply
    finally:
        for p in procs:
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGTERM)
        for p in procs:
            try:
                p.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
        for f in logs:
            f.close()


@pytest.mark.parametrize("manual", [True, False, "tensor-parallel nodes"])
@_retry_startup
def test_scheduler_and_two_joined_nodes_end_to_end(manual, tmp_path):
    """`parallax run` + two `parallax join` processes + a chat completion through the scheduler: the whole control
    and data path as separate processes. With layer halves assigned by hand the pipeline has two stages (the nodes
    measure the hop between them, the scheduler registers the pipeline once it can price it); left to itself the
    scheduler gives each node the whole (small) model."""
    ps, p0, p1 = free_port(), free_port(), free_port()
    env = dict(os.environ, PYTHONPATH=ROOT)
    logs = [open(tmp_path / f"p{i}.log", "w") for i in range(3)]
    kw = dict(cwd=ROOT, env=env, stderr=subprocess.STDOUT, start_new_session=True)
    node = [sys.executable, "-m", "parallax_b200.launch", "--scheduler-addr", f"127.0.0.1:{ps}", "--random-init",
            "--host", "127.0.0.1", "--max-batch-size", "4", "--max-sequence-length", "256", "--log-level", "WARNING"]
    procs = [subprocess.Popen([sys.executable, "-m", "parallax_b200.backend.app", "--host", "127.0.0.1", "--port", str(ps),
                               "--model-name", "tiny", "--init-nodes-num", "2", "--log-level", "WARNING"], stdout=logs[0], **kw)]
    try:
        deadline = time.time() + 60
        while time.time() < deadline:
            try:
                urllib.request.urlopen(f"http://127.0.0.1:{ps}/cluster/status_json", timeout=2).read()
                break
            except OSError:
                time.sleep(0.3)
        r0, r1 = (["--start-layer", "0", "--end-layer", "2"], ["--start-layer", "2", "--end-layer", "4"]) if manual else ([], [])
        if manual == "tensor-parallel nodes":        # each joined node runs its layers over two ranks
            r0, r1 = r0 + ["--tp-size", "2"], r1 + ["--tp-size", "2"]
        procs.append(subprocess.Popen(node + ["--port", str(p0)] + r0, stdout=logs[1], **kw))
        procs.append(subprocess.Popen(node + ["--port", str(p1)] + r1, stdout=logs[2], **kw))
        status = None
        deadline = time.time() + 150
        while time.time() < deadline and all(p.poll() is None for p in procs):
            with urllib.request.urlopen(f"http://127.0.0.1:{ps}/cluster/status_json", timeout=5) as r:
                status = json.loads(r.read())["data"]
            if status["status"] == "available" and len(status["node_list"]) == 2:
                break
            time.sleep(0.5)
        tails = "".join(open(tmp_path / f"p{i}.log").read()[-1500:] for i in range(3))
        assert status and status["status"] == "available", (status, tails)
        spans = sorted((n["start_layer"], n["end_layer"]) for n in status["node_list"])
        assert spans == ([(0, 2), (2, 4)] if manual else [(0, 4), (0, 4)]), status
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 8, "temperature": 0, "return_probs": True}
        reply = None
        for _ in range(20):          # the first node may still be loading when the cluster turns available
            try:
                reply = _post(ps, body, timeout=60)
                break
            except OSError:
                time.sleep(1.0)
        assert reply is not None and reply["usage"]["completion_tokens"] >= 1, tails
        again = _post(ps, body, timeout=60)
        assert _close(_probs(again), _probs(reply))
        if manual is True:
            # a burst of clients through the scheduler, half of which hang up mid-stream: afterwards neither node holds
            # a request, a shadow request, KV memory or an open stream
            import threading

            def client(i: int) -> None:
                b = dict(body, max_tokens=24, ignore_eos=True, stream=True,
                         messages=[{"role": "user", "content": f"client number {i} " * (1 + i % 3)}])
                rq = urllib.request.Request(f"http://127.0.0.1:{ps}/v1/chat/completions", data=json.dumps(b).encode(),
                                            headers={"Content-Type": "application/json"})
                with urllib.request.urlopen(rq, timeout=120) as resp:
                    seen = 0
                    for line in resp:
                        if line.startswith(b"data: "):
                            seen += 1
                            if i % 2 == 0 and seen >= 3:
                                return                      # leaving closes the connection mid-stream

            threads = [threading.Thread(target=client, args=(i,)) for i in range(8)]
            for t in threads:
                t.start()
            for t in threads:
                t.join(150)
            assert not any(t.is_alive() for t in threads)
            deadline = time.time() + 60
            stats = None
            while time.time() < deadline:
                stats = [json.loads(urllib.request.urlopen(f"http://127.0.0.1:{p}/peer/stats", timeout=5).read()) for p in (p0, p1)]
                if all(st["running"] == st["mirror"] == st["kv_requests"] == st["streams"] == 0 for st in stats):
                    break
                time.sleep(0.5)
            assert all(st["running"] == st["mirror"] == st["kv_requests"] == st["streams"] == 0 for st in stats), stats
        # a JSON-schema request through the scheduler: the last node samples under the schema
        schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"]}
        constrained = _post(ps, dict(body, max_tokens=80, response_format={"type": "json_schema",
                                                                           "json_schema": {"name": "x", "schema": schema}}))
        assert isinstance(json.loads(constrained["choices"][0]["message"]["content"])["ok"], bool)
        # the same through the scheduler as a stream: SSE chunks, a usage chunk, the end marker
        req = urllib.request.Request(f"http://127.0.0.1:{ps}/v1/chat/completions", headers={"Content-Type": "application/json"},
                                     data=json.dumps(dict(body, stream=True)).encode())
        with urllib.request.urlopen(req, timeout=60) as r:
            assert r.headers.get("content-type", "").startswith("text/event-stream")
            lines = [ln.decode() for ln in r.read().split(b"\n") if ln.startswith(b"data: ")]
        assert lines[-1].strip() == "data: [DONE]"
        chunks = [json.loads(ln[6:]) for ln in lines[:-1]]
        usage = [c["usage"] for c in chunks if c.get("usage")]
        assert usage and usage[-1]["completion_tokens"] == reply["usage"]["completion_tokens"]
        assert any(c["choices"] and c["choices"][0].get("finish_reason") for c in chunks)
    finally:
        for p in procs:
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGTERM)
        for p in procs:
            try:
                p.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
        for f in logs:
            f.close()


@_retry_startup
def test_refit_reaches_every_node_of_a_running_cluster(tmp_path):
    """Online weight refit end to end: the scheduler hands a refit request (content-addressed blocks on disk) to
    both nodes of a two-stage pipeline with their heartbeats; afterwards the cluster answers as a model with the
    new weights does."""
    import torch
    from fastapi.testclient import TestClient
    from safetensors.torch import save_file

    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.service import EngineLoop
    from parallax_b200.frontend.openai_api import create_app
    from parallax_b200.frontend.tokenizer import TokenizerWrapper
    from parallax_b200.models.config import named_config
    from parallax_b200.utils.weight_refit import calculate_cid
    from tests.test_engine_gpu import _export_weights

    cfg = named_config("tiny")
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 8, "temperature": 0, "return_probs": True}

    def local_reply(seed):
        torch.manual_seed(0)
        eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, max_total_length=256, seed=seed)
        loop = EngineLoop(eng)
        loop.start()
        try:
            with TestClient(create_app(loop, TokenizerWrapper.from_pretrained(None, vocab_size=cfg.vocab_size), "tiny", 256)) as c:
                return _probs(c.post("/v1/chat/completions", json=body).json()), eng
        finally:
            loop.stop()

    before, _ = local_reply(0)
    after, other = local_reply(7)
    assert not _close(before, after)
    w = _export_weights(other)
    w.pop("lm_head.weight", None)
    names = sorted(w)
    index_map, paths = {}, {}
    for i, group in enumerate((names[0::2], names[1::2])):
        f = tmp_path / f"block{i}.safetensors"
        save_file({k: w[k].contiguous() for k in group}, str(f))
        cid = calculate_cid(f.read_bytes())
        paths[cid] = str(f)
        index_map.update({k: cid for k in group})

    ps, p0, p1 = free_port(), free_port(), free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, PARALLAX_ROUTING_RETRY_DELAY_S="0.5", PARALLAX_FORWARD_RETRY_DELAY_S="0.5",
               PARALLAX_HEARTBEAT_INTERVAL_S="1")
    logs = [open(tmp_path / f"p{i}.log", "w") for i in range(3)]
    kw = dict(cwd=ROOT, env=env, stderr=subprocess.STDOUT, start_new_session=True)
    node = [sys.executable, "-m", "parallax_b200.launch", "--scheduler-addr", f"127.0.0.1:{ps}", "--random-init",
            "--host", "127.0.0.1", "--max-batch-size", "4", "--max-sequence-length", "256", "--log-level", "WARNING",
            "--enable-weight-refit"]
    procs = [subprocess.Popen([sys.executable, "-m", "parallax_b200.backend.app", "--host", "127.0.0.1", "--port", str(ps),
                               "--model-name", "tiny", "--init-nodes-num", "2", "--log-level", "WARNING",
                               "--enable-weight-refit", "true"], stdout=logs[0], **kw)]
    try:
        deadline = time.time() + 60
        while time.time() < deadline:
            try:
                urllib.request.urlopen(f"http://127.0.0.1:{ps}/cluster/status_json", timeout=2).read()
                break
            except OSError:
                time.sleep(0.3)
        procs.append(subprocess.Popen(node + ["--port", str(p0), "--start-layer", "0", "--end-layer", "2"], stdout=logs[1], **kw))
        procs.append(subprocess.Popen(node + ["--port", str(p1), "--start-layer", "2", "--end-layer", "4"], stdout=logs[2], **kw))

        def chat():
            for _ in range(40):
                try:
                    return _probs(_post(ps, body, timeout=60))
                except OSError:
                    time.sleep(1.0)
            raise AssertionError("".join(open(tmp_path / f"p{i}.log").read()[-1500:] for i in range(3)))

        assert _close(chat(), before)
        req = urllib.request.Request(f"http://127.0.0.1:{ps}/weight/refit", headers={"Content-Type": "application/json"},
                                     data=json.dumps({"time_stamp": time.time(), "cid": sorted(paths), "index_map": index_map,
                                                      "paths": paths}).encode())
        assert urllib.request.urlopen(req, timeout=10).status == 200
        got = None
        deadline = time.time() + 60
        while time.time() < deadline:
            got = chat()
            if _close(got, after):
                break
            time.sleep(1.0)
        assert _close(got, after), (got, after, before)
    finally:
        for p in procs:
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGTERM)
        for p in procs:
            try:
                p.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
        for f in logs:
            f.close()


def _wait_status(ps: int, want: str, nodes: int, timeout_s: float = 120.0) -> dict:
    status = None
    deadline = time.time() + timeout_s
    while time.time() < deadline:
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{ps}/cluster/status_json", timeout=5) as r:
                status = json.loads(r.read())["data"]
            if status["status"] == want and len(status["node_list"]) == nodes:
                return status
        except OSError:
            pass
        time.sleep(0.4)
    raise _StartupError(f"cluster did not become {want} with {nodes} node(s): {status}")


def _post_to(url: str, body: dict, timeout: float = 60.0):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.status, json.loads(r.read())
    except urllib.error.HTTPError as e:
        return e.code, json.loads(e.read() or b"{}")


@_retry_startup
def test_router_in_front_of_a_cluster_whose_node_leaves_and_is_replaced(tmp_path):
    """Router -> scheduler -> node as processes. The node is stopped (it says goodbye), the cluster goes back to
    waiting and requests are answered with an error instead of hanging; a new node joins and service resumes,
    through the same router registration."""
    import urllib.error  # noqa: F401  (used by _post_to)

    pr, ps, p0, p1 = free_port(), free_port(), free_port(), free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, PARALLAX_ROUTING_RETRY_DELAY_S="0.5", PARALLAX_FORWARD_RETRY_DELAY_S="0.5",
               PARALLAX_HEARTBEAT_INTERVAL_S="1")
    logs = [open(tmp_path / f"p{i}.log", "w") for i in range(4)]
    kw = dict(cwd=ROOT, env=env, stderr=subprocess.STDOUT, start_new_session=True)
    node = [sys.executable, "-m", "parallax_b200.launch", "--scheduler-addr", f"127.0.0.1:{ps}", "--random-init",
            "--host", "127.0.0.1", "--max-batch-size", "4", "--max-sequence-length", "256", "--log-level", "WARNING"]
    procs = {
        "sched": subprocess.Popen([sys.executable, "-m", "parallax_b200.backend.app", "--host", "127.0.0.1", "--port", str(ps),
                                   "--model-name", "tiny", "--init-nodes-num", "1", "--log-level", "WARNING"], stdout=logs[0], **kw),
        "router": subprocess.Popen([sys.executable, "-m", "parallax_b200.router.app", "--host", "127.0.0.1", "--port", str(pr)],
                                   stdout=logs[1], **kw),
    }
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6, "temperature": 0,
            "return_probs": True}
    try:
        _wait_status(ps, "waiting", 0, 60)
        procs["a"] = subprocess.Popen(node + ["--port", str(p0)], stdout=logs[2], **kw)
        _wait_status(ps, "available", 1)
        for _ in range(100):
            try:
                urllib.request.urlopen(f"http://127.0.0.1:{pr}/health", timeout=2).read()
                break
            except OSError:
                time.sleep(0.2)
        code, reg = _post_to(f"http://127.0.0.1:{pr}/register", {"endpoint": f"http://127.0.0.1:{ps}"})
        assert code == 200 and reg["base_url"].endswith(str(ps)), reg
        first = None
        for _ in range(30):
            code, first = _post_to(f"http://127.0.0.1:{pr}/v1/chat/completions", body)
            if code == 200:
                break
            time.sleep(1.0)
        assert code == 200, first
        fp = _probs(first)
        # the node goes away
        os.killpg(procs["a"].pid, signal.SIGTERM)
        procs["a"].wait(30)
        _wait_status(ps, "waiting", 0, 60)
        t0 = time.time()
        code, err = _post_to(f"http://127.0.0.1:{pr}/v1/chat/completions", body, timeout=200)
        assert code >= 400 and time.time() - t0 < 150, (code, err)         # an error, not a hang
        # a replacement joins
        procs["b"] = subprocess.Popen(node + ["--port", str(p1)], stdout=logs[3], **kw)
        _wait_status(ps, "available", 1)
        again = None
        for _ in range(40):
            code, again = _post_to(f"http://127.0.0.1:{pr}/v1/chat/completions", body)
            if code == 200:
                break
            time.sleep(1.0)
        assert code == 200, again
        assert _close(_probs(again), fp)
    finally:
        for p in procs.values():
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGTERM)
        for p in procs.values():
            try:
                p.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
        for f in logs:
            f.close()


@_retry_startup
def test_switching_the_model_reloads_the_joined_node(tmp_path):
    """`POST /scheduler/init` with another model while a node is serving: the node learns the new allocation from
    its next heartbeat, reloads its executor and serves the new model - the elastic path of a running cluster."""
    ps, p0 = free_port(), free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, PARALLAX_ROUTING_RETRY_DELAY_S="0.5", PARALLAX_FORWARD_RETRY_DELAY_S="0.5",
               PARALLAX_HEARTBEAT_INTERVAL_S="1")
    logs = [open(tmp_path / f"p{i}.log", "w") for i in range(2)]
    kw = dict(cwd=ROOT, env=env, stderr=subprocess.STDOUT, start_new_session=True)
    procs = [subprocess.Popen([sys.executable, "-m", "parallax_b200.backend.app", "--host", "127.0.0.1", "--port", str(ps),
                               "--model-name", "tiny", "--init-nodes-num", "1", "--log-level", "WARNING"], stdout=logs[0], **kw)]
    body = {"messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6, "temperature": 0, "return_probs": True}

    def chat():
        last = None
        for _ in range(40):
            code, last = _post_to(f"http://127.0.0.1:{ps}/v1/chat/completions", body)
            if code == 200:
                return last
            time.sleep(1.0)
        raise AssertionError((last, "".join(open(tmp_path / f"p{i}.log").read()[-1500:] for i in range(2))))

    try:
        _wait_status(ps, "waiting", 0, 60)
        procs.append(subprocess.Popen([sys.executable, "-m", "parallax_b200.launch", "--scheduler-addr", f"127.0.0.1:{ps}",
                                       "--random-init", "--host", "127.0.0.1", "--port", str(p0), "--max-batch-size", "4",
                                       "--max-sequence-length", "256", "--log-level", "INFO"], stdout=logs[1], **kw))
        assert _wait_status(ps, "available", 1)["model_name"] == "tiny"
        dense = _probs(chat())
        code, _r = _post_to(f"http://127.0.0.1:{ps}/scheduler/init", {"model_name": "tiny-moe", "init_nodes_num": 1})
        assert code == 200
        deadline = time.time() + 90
        moe = None
        while time.time() < deadline:
            st = _wait_status(ps, "available", 1, 90)
            if st["model_name"] == "tiny-moe":
                reply = chat()
                moe = _probs(reply)
                if not _close(moe, dense):
                    break
            time.sleep(1.0)
        assert moe is not None and not _close(moe, dense)
        assert "reloading the executor" in open(tmp_path / "p1.log").read()
    finally:
        for p in procs:
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGTERM)
        for p in procs:
            try:
                p.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
        for f in logs:
            f.close()


@_retry_startup
def test_a_peer_that_dies_fails_requests_instead_of_hanging_them(tmp_path):
    """Two peers without a scheduler; the second is killed outright. A request then ends with an error within
    seconds (the first peer cannot deliver the activations), the first peer keeps serving, and once a second peer
    is back on the same address requests complete again."""
    import urllib.error  # noqa: F401

    p0, p1 = free_port(), free_port()
    env = dict(os.environ, PYTHONPATH=ROOT)
    common = [sys.executable, "-m", "parallax_b200.launch", "--model-path", "tiny", "--random-init", "--host", "127.0.0.1",
              "--max-batch-size", "4", "--max-sequence-length", "256", "--log-level", "WARNING"]
    second = common + ["--port", str(p1), "--start-layer", "2", "--end-layer", "4", "--initial-peers", f"127.0.0.1:{p0}"]
    logs = [open(tmp_path / f"n{i}.log", "w") for i in range(3)]
    kw = dict(cwd=ROOT, env=env, stderr=subprocess.STDOUT, start_new_session=True)
    procs = [subprocess.Popen(common + ["--port", str(p0), "--start-layer", "0", "--end-layer", "2", "--initial-peers",
                                        f"127.0.0.1:{p1}"], stdout=logs[0], **kw),
             subprocess.Popen(second, stdout=logs[1], **kw)]
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6, "temperature": 0,
            "return_probs": True}

    def wait_up(port, path):
        deadline = time.time() + 120
        while time.time() < deadline:
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}{path}", timeout=2) as r:
                    if r.status == 200:
                        return
            except OSError:
                time.sleep(0.4)
        raise _StartupError(f"{port}{path} did not come up")

    try:
        wait_up(p0, "/v1/models")
        wait_up(p1, "/peer/info")
        code, ok = _post_to(f"http://127.0.0.1:{p0}/v1/chat/completions", body)
        assert code == 200
        fp = _probs(ok)
        os.killpg(procs[1].pid, signal.SIGKILL)
        procs[1].wait(10)
        t0 = time.time()
        code, err = _post_to(f"http://127.0.0.1:{p0}/v1/chat/completions", body, timeout=120)
        assert code >= 500 and time.time() - t0 < 90, (code, err, time.time() - t0)
        procs.append(subprocess.Popen(second, stdout=logs[2], **kw))
        wait_up(p1, "/peer/info")
        # the new peer does not hold the prefix that the first peer has cached for this prompt: the first attempt may
        # come back aborted (no tokens), which makes the first peer drop its cached prefixes; the retry completes
        again = None
        for _ in range(20):
            code, again = _post_to(f"http://127.0.0.1:{p0}/v1/chat/completions", body)
            if code == 200 and again["usage"]["completion_tokens"] >= 1:
                break
            time.sleep(1.0)
        assert code == 200 and _close(_probs(again), fp), again
    finally:
        for p in procs:
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGTERM)
        for p in procs:
            try:
                p.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
        for f in logs:
            f.close()


@pytest.mark.parametrize("victim", ["last", "first"])
@_retry_startup
def test_a_joined_node_that_dies_is_dropped_and_its_requests_fail_fast(victim, tmp_path):
    """Scheduler + two hand-placed nodes; the second is killed outright (no goodbye). Requests routed through the
    broken pipeline end with an error within seconds, the scheduler drops the silent node after its heartbeat
    time-out and reports the cluster as waiting; when a node takes the vacant layers the cluster serves again."""
    import urllib.error  # noqa: F401

    ps, p0, p1, p2 = free_port(), free_port(), free_port(), free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, PARALLAX_ROUTING_RETRY_DELAY_S="0.5", PARALLAX_FORWARD_RETRY_DELAY_S="0.5",
               PARALLAX_HEARTBEAT_INTERVAL_S="1", PARALLAX_HEARTBEAT_TIMEOUT_S="5")
    logs = [open(tmp_path / f"p{i}.log", "w") for i in range(4)]
    kw = dict(cwd=ROOT, env=env, stderr=subprocess.STDOUT, start_new_session=True)
    node = [sys.executable, "-m", "parallax_b200.launch", "--scheduler-addr", f"127.0.0.1:{ps}", "--random-init",
            "--host", "127.0.0.1", "--max-batch-size", "4", "--max-sequence-length", "256", "--log-level", "WARNING"]
    procs = [subprocess.Popen([sys.executable, "-m", "parallax_b200.backend.app", "--host", "127.0.0.1", "--port", str(ps),
                               "--model-name", "tiny", "--init-nodes-num", "2", "--log-level", "WARNING"], stdout=logs[0], **kw)]
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6, "temperature": 0,
            "return_probs": True}

    def chat_ok(tries=40):
        last = None
        for _ in range(tries):
            code, last = _post_to(f"http://127.0.0.1:{ps}/v1/chat/completions", body)
            if code == 200 and last["usage"]["completion_tokens"] >= 1:
                return last
            time.sleep(1.0)
        raise AssertionError((last, "".join(open(tmp_path / f"p{i}.log").read()[-1200:] for i in range(4))))

    try:
        _wait_status(ps, "waiting", 0, 60)
        procs.append(subprocess.Popen(node + ["--port", str(p0), "--start-layer", "0", "--end-layer", "2"], stdout=logs[1], **kw))
        procs.append(subprocess.Popen(node + ["--port", str(p1), "--start-layer", "2", "--end-layer", "4"], stdout=logs[2], **kw))
        _wait_status(ps, "available", 2)
        fp = _probs(chat_ok())
        k = 2 if victim == "last" else 1            # the node that samples, or the one the scheduler forwards to
        os.killpg(procs[k].pid, signal.SIGKILL)
        procs[k].wait(10)
        t0 = time.time()
        code, err = _post_to(f"http://127.0.0.1:{ps}/v1/chat/completions", body, timeout=150)
        assert code >= 400 and time.time() - t0 < 120, (code, err, time.time() - t0)
        st = _wait_status(ps, "waiting", 1, 60)                  # the silent node is gone from the list
        left = (0, 2) if victim == "last" else (2, 4)
        assert [(n["start_layer"], n["end_layer"]) for n in st["node_list"]] in ([left], [(None, None)])
        vacant = ["--start-layer", "2", "--end-layer", "4"] if victim == "last" else ["--start-layer", "0", "--end-layer", "2"]
        procs.append(subprocess.Popen(node + ["--port", str(p2)] + vacant, stdout=logs[3], **kw))
        _wait_status(ps, "available", 2)
        assert _close(_probs(chat_ok()), fp)
    finally:
        for p in procs:
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGTERM)
        for p in procs:
            try:
                p.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
        for f in logs:
            f.close()


@_retry_startup
def test_in_box_server_ends_when_one_of_its_ranks_dies(tmp_path):
    """`parallax serve --pp-size 2`: when a worker rank is killed the serving process notices (child exit, or the
    rank's heartbeat in the control channel going stale), fails what is in flight and exits with an error status
    instead of hanging - a supervisor can restart it."""
    psutil = pytest.importorskip("psutil")
    port = free_port()
    log = open(tmp_path / "serve.log", "w")
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    proc = subprocess.Popen([sys.executable, "-m", "parallax_b200.launch", "--model-path", "tiny", "--random-init", "--port",
                             str(port), "--host", "127.0.0.1", "--max-batch-size", "4", "--max-sequence-length", "256",
                             "--log-level", "WARNING", "--pp-size", "2"], cwd=ROOT, env=env, stdout=log,
                            stderr=subprocess.STDOUT, start_new_session=True)
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
        if not up:
            raise _StartupError(open(tmp_path / "serve.log").read()[-3000:])
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0}
        assert _post(port, body)["usage"]["completion_tokens"] >= 1
        workers = [c for c in psutil.Process(proc.pid).children(recursive=True) if "parallax_b200.parallel.launcher" in " ".join(c.cmdline())]
        assert len(workers) == 1, [c.cmdline() for c in psutil.Process(proc.pid).children(recursive=True)]
        workers[0].kill()
        code = proc.wait(60)                     # the server goes down by itself ...
        assert code != 0                         # ... and says so
    finally:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGTERM)
            try:
                proc.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(proc.pid, signal.SIGKILL)
        log.close()


@_retry_startup
def test_cli_serve_and_graceful_shutdown(tmp_path):
    """The `parallax` command itself: `serve` (with an in-box pipeline, so that there are worker processes) answers
    requests, and an interrupt takes the whole process tree down without leaving ranks behind."""
    psutil = pytest.importorskip("psutil")
    port = free_port()
    log = open(tmp_path / "cli.log", "w")
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    proc = subprocess.Popen([sys.executable, "-m", "parallax_b200.cli", "serve", "-m", "tiny", "--random-init", "--port", str(port),
                             "--host", "127.0.0.1", "--max-batch-size", "4", "--max-sequence-length", "256", "--pp-size", "2",
                             "--log-level", "WARNING"], cwd=ROOT, env=env, stdout=log, stderr=subprocess.STDOUT,
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
        if not up:
            raise _StartupError(open(tmp_path / "cli.log").read()[-3000:])
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 5, "temperature": 0}
        assert _post(port, body)["usage"]["completion_tokens"] >= 1
        tree = psutil.Process(proc.pid).children(recursive=True)
        assert len(tree) >= 2, [c.cmdline() for c in tree]          # the launcher and at least one worker rank
        proc.send_signal(signal.SIGINT)
        proc.wait(40)
        gone, alive = psutil.wait_procs(tree, timeout=20)
        assert not alive, [c.cmdline() for c in alive]
    finally:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGTERM)
            try:
                proc.wait(20)
            except subprocess.TimeoutExpired:
                os.killpg(proc.pid, signal.SIGKILL)
        else:
            try:
                os.killpg(proc.pid, signal.SIGKILL)      # whatever is left of the group
            except ProcessLookupError:
                pass
        log.close()
