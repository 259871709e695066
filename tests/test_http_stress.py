"""Concurrent HTTP clients, some of which hang up mid-stream: nothing may be left behind in the engine."""

import asyncio
import json
import time

import pytest

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.service import EngineLoop
from parallax_b200.frontend.openai_api import create_app
from parallax_b200.frontend.tokenizer import TokenizerWrapper
from parallax_b200.launch import serve_http
from parallax_b200.models.config import named_config
from parallax_b200.parallel.launcher import free_port


def test_clients_that_hang_up_leave_nothing_behind():
    aiohttp = pytest.importorskip("aiohttp")
    cfg = named_config("tiny")
    eng = Engine(cfg, device="cpu", num_blocks=128, page_size=16, max_batch_size=4, max_total_length=256)
    loop = EngineLoop(eng)
    loop.start()
    tok = TokenizerWrapper.from_pretrained(None, vocab_size=cfg.vocab_size)
    port = free_port()
    server, thread = serve_http(create_app(loop, tok, "tiny", max_model_len=256), "127.0.0.1", port, "warning")
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)

    async def one(session, i: int) -> str:
        body = {"model": "tiny", "prompt": f"request number {i} " * (1 + i % 4), "max_tokens": 40, "temperature": 0,
                "ignore_eos": True, "stream": True}
        async with session.post(f"http://127.0.0.1:{port}/v1/completions", json=body) as resp:
            assert resp.status == 200
            n = 0
            async for line in resp.content:
                if line.startswith(b"data: ") and b"[DONE]" not in line:
                    n += 1
                    if i % 2 == 0 and n >= 2:
                        return "hung up"            # leaving the context closes the connection mid-stream
            return "complete"

    async def run():
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=120)) as session:
            return await asyncio.gather(*(one(session, i) for i in range(12)))

    try:
        results = asyncio.run(run())
        assert results.count("hung up") == 6 and results.count("complete") == 6
        deadline = time.time() + 30
        while time.time() < deadline and (loop.num_inflight or eng.has_work() or eng.cache.reqs):
            time.sleep(0.1)
        assert loop.num_inflight == 0 and not eng.has_work() and not eng.cache.reqs
        # the server still answers
        import urllib.request

        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", headers={"Content-Type": "application/json"},
                                     data=json.dumps({"model": "tiny", "prompt": "after", "max_tokens": 3}).encode())
        with urllib.request.urlopen(req, timeout=30) as r:
            assert json.loads(r.read())["usage"]["completion_tokens"] >= 1
    finally:
        server.should_exit = True
        thread.join(5)
        loop.stop()
