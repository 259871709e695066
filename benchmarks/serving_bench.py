"""Start ``parallax serve`` with random-init weights on this box, drive it with the serving benchmark
client over HTTP, and print the client's report (throughput, TTFT / TPOT / ITL percentiles) as one JSON line.

    python benchmarks/serving_bench.py --model qwen3-8b --num-prompts 1024 --max-concurrency 512 \\
        --input-len 1024 --output-len 256 [--pp-size 2] [--out FILE]

The server is a child process in its own process group; it is stopped through that group's id when the
client is done. This is the end-to-end path a user of the HTTP API sees: tokenisation, request queueing,
continuous batching, streaming of every token as a server-sent event.
"""

from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
import urllib.request

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def wait_ready(url: str, proc: subprocess.Popen, timeout_s: float) -> bool:
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        if proc.poll() is not None:
            return False
        try:
            with urllib.request.urlopen(url, timeout=2) as r:
                if r.status == 200:
                    return True
        except Exception:
            time.sleep(1.0)
    return False


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--port", type=int, default=3037)
    ap.add_argument("--num-prompts", type=int, default=1024)
    ap.add_argument("--max-concurrency", type=int, default=512)
    ap.add_argument("--request-rate", default="inf")
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--pp-size", type=int, default=1)
    ap.add_argument("--tp-size", type=int, default=1)
    ap.add_argument("--startup-timeout", type=float, default=600.0)
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    max_len = args.input_len + args.output_len + 128
    server_cmd = [sys.executable, "-m", "parallax_b200.launch", "--model-path", args.model, "--random-init",
                  "--host", "127.0.0.1", "--port", str(args.port), "--max-batch-size", str(args.max_concurrency),
                  "--max-sequence-length", str(max_len), "--max-num-tokens-per-batch", str(8192 + args.max_concurrency),
                  "--chunked-prefill-size", "4096", "--kv-cache-memory-fraction", "0.85", "--log-level", "WARNING",
                  "--pp-size", str(args.pp_size), "--tp-size", str(args.tp_size)]
    server = subprocess.Popen(server_cmd, env=env, start_new_session=True)
    report = {"server": " ".join(server_cmd[2:])}
    try:
        base = f"http://127.0.0.1:{args.port}"
        if not wait_ready(base + "/v1/models", server, args.startup_timeout):
            report["error"] = "the server did not come up"
        else:
            tmp = args.out + ".client.json" if args.out else os.path.join("/tmp", f"pxl_serving_{os.getpid()}.json")
            client = [sys.executable, os.path.join(ROOT, "benchmarks", "benchmark_serving.py"), "--base-url", base,
                      "--model", args.model, "--dataset", "random", "--random-input-len", str(args.input_len),
                      "--random-output-len", str(args.output_len), "--num-prompts", str(args.num_prompts),
                      "--request-rate", args.request_rate, "--max-concurrency", str(args.max_concurrency),
                      "--ignore-eos", "--byte-tokens", "--save-result", tmp]
            rc = subprocess.run(client, env=env).returncode
            report["client_rc"] = rc
            if os.path.exists(tmp):
                with open(tmp) as f:
                    report["result"] = json.load(f)
    finally:
        try:
            os.killpg(server.pid, signal.SIGTERM)       # the server's own process group
            server.wait(timeout=30)
        except Exception:
            try:
                os.killpg(server.pid, signal.SIGKILL)
            except Exception:
                pass
    line = json.dumps(report)
    print(line, flush=True)
    if args.out:
        with open(args.out, "w") as f:
            f.write(line + "\n")


if __name__ == "__main__":
    main()
