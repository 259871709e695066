"""Serving benchmark client for any OpenAI-compatible endpoint of this framework (node frontend,
cluster backend or router).

    python benchmarks/benchmark_serving.py --base-url http://127.0.0.1:3000 --model qwen3-8b \\
        --dataset random --random-input-len 1024 --random-output-len 256 --num-prompts 1000 --request-rate 16

Requests arrive as a Poisson process (``--request-rate inf`` sends everything at once, optionally
capped by ``--max-concurrency``), responses are streamed, and the report gives request and token
throughput, time to first token, time per output token, inter-token latency, end-to-end latency
(mean / median / p99) and goodput against optional SLOs. Same role as the reference's
``src/backend/benchmark/benchmark_serving.py`` (datasets ``:147-318``, arrivals ``:320``, metrics
``:363-477``) with its own, smaller implementation; datasets here are ``random`` (uniform token ids
decoded by the model's tokenizer, or synthetic words when no tokenizer is given), ``jsonl``
(one ``{"prompt": ..., "max_tokens": ...}`` per line), ``sharegpt`` (a ShareGPT-style conversation
dump: first human turn as prompt, length of the first reply as output budget), ``hf`` (a local parquet /
jsonl copy of a Hugging Face text dataset) and ``wildchat`` (rows with a ``conversation`` list).
"""

from __future__ import annotations

import argparse
import asyncio
import json
import random
import statistics
import time
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class Sample:
    prompt: str
    prompt_len: int
    max_tokens: int


@dataclass
class Result:
    ok: bool = False
    prompt_len: int = 0
    output_tokens: int = 0
    ttft: float = 0.0
    latency: float = 0.0
    itl: list = field(default_factory=list)
    error: str = ""


def make_random_dataset(n: int, in_len: int, out_len: int, range_ratio: float, seed: int, tokenizer=None,
                        prefix_len: int = 0, byte_level: bool = False) -> list[Sample]:
    """``byte_level``: prompts of exactly the asked number of ASCII characters, for servers that run the
    byte-level fallback tokenizer (random-init models): one character is one token there."""
    rng = random.Random(seed)
    vocab = tokenizer.vocab_size if tokenizer is not None else 0
    prefix = [rng.randrange(vocab) for _ in range(prefix_len)] if tokenizer is not None else []
    out = []
    for _ in range(n):
        li = max(1, int(in_len * (1 - range_ratio * rng.random())))
        lo = max(1, int(out_len * (1 - range_ratio * rng.random())))
        if tokenizer is not None:
            ids = prefix + [rng.randrange(vocab) for _ in range(max(li - prefix_len, 1))]
            text = tokenizer.decode(ids)
        elif byte_level:
            text = "".join(rng.choice("abcdefghijklmnopqrstuvwxyz      ") for _ in range(li))
        else:
            text = " ".join(f"w{rng.randrange(50000)}" for _ in range(li))
        out.append(Sample(text, li, lo))
    return out


def _read_records(path: str) -> list[dict]:
    """Rows of a local dataset file: ``.parquet`` (as published on the Hugging Face hub), ``.jsonl`` or ``.json``."""
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq

        return pq.read_table(path).to_pylist()
    with open(path) as f:
        if path.endswith(".jsonl"):
            return [json.loads(line) for line in f if line.strip()]
        data = json.load(f)
    return data if isinstance(data, list) else data.get("data", [])


def load_hf_dataset(path: str, n: int, default_out: int, seed: int, tokenizer=None, text_column: str = "",
                    output_column: str = "") -> list[Sample]:
    """A local copy of a Hugging Face text dataset: the prompt is ``text_column`` (default: the first of
    ``prompt`` / ``question`` / ``instruction`` / ``text`` that the rows have); when ``output_column`` (default
    ``response`` / ``answer`` / ``output``) exists, its length is the output budget. Counterpart of the
    reference's ``hf`` dataset option (``src/backend/benchmark/benchmark_serving.py:210-318``) without the
    download step."""
    rows = _read_records(path)
    rng = random.Random(seed)
    rng.shuffle(rows)

    def pick(row, wanted, candidates):
        if wanted:
            return row.get(wanted)
        return next((row[c] for c in candidates if row.get(c)), None)

    def length(text: str) -> int:
        return len(tokenizer.encode(text)) if tokenizer is not None else max(1, len(text.split()))

    out = []
    for row in rows:
        prompt = pick(row, text_column, ("prompt", "question", "instruction", "text"))
        if not isinstance(prompt, str) or not prompt.strip():
            continue
        reply = pick(row, output_column, ("response", "answer", "output"))
        lo = length(reply) if isinstance(reply, str) and reply else default_out
        out.append(Sample(prompt, length(prompt), max(1, lo)))
        if len(out) >= n:
            break
    return out


def load_wildchat_dataset(path: str, n: int, default_out: int, seed: int, tokenizer=None) -> list[Sample]:
    """WildChat-style rows: ``{"conversation": [{"role": "user", "content": ...}, {"role": "assistant", ...}]}``.
    First user turn = prompt, length of the first assistant turn = output budget."""
    rows = _read_records(path)
    rng = random.Random(seed)
    rng.shuffle(rows)

    def length(text: str) -> int:
        return len(tokenizer.encode(text)) if tokenizer is not None else max(1, len(text.split()))

    out = []
    for row in rows:
        conv = row.get("conversation") or []
        user = next((t.get("content") for t in conv if t.get("role") == "user"), None)
        reply = next((t.get("content") for t in conv if t.get("role") == "assistant"), None)
        if not user:
            continue
        lp = length(user)
        if lp > 4096:
            continue
        out.append(Sample(user, lp, max(1, length(reply)) if reply else default_out))
        if len(out) >= n:
            break
    return out


def load_jsonl_dataset(path: str, n: int, default_out: int) -> list[Sample]:
    out = []
    with open(path) as f:
        for line in f:
            if not line.strip():
                continue
            d = json.loads(line)
            p = d.get("prompt") or d.get("text") or ""
            out.append(Sample(p, max(1, len(p.split())), int(d.get("max_tokens", default_out))))
            if len(out) >= n:
                break
    return out


def load_sharegpt_dataset(path: str, n: int, default_out: int, seed: int, tokenizer=None) -> list[Sample]:
    """ShareGPT-style JSON: a list of ``{"conversations": [{"from": "human", "value": ...}, {"from": "gpt",
    "value": ...}, ...]}``. The first human turn is the prompt and the length of the first reply sets the
    output budget (the reference's ``sample_sharegpt_requests``, ``benchmark_serving.py:147-208``);
    conversations with fewer than two turns or with very short / very long turns are skipped."""
    with open(path) as f:
        data = json.load(f)
    rng = random.Random(seed)
    rng.shuffle(data)

    def length(text: str) -> int:
        return len(tokenizer.encode(text)) if tokenizer is not None else max(1, len(text.split()))

    out = []
    for item in data:
        conv = item.get("conversations") or item.get("conversation") or []
        if len(conv) < 2:
            continue
        prompt, reply = conv[0].get("value", ""), conv[1].get("value", "")
        lp, lr = length(prompt), length(reply)
        if lp < 4 or lr < 4 or lp > 1024 or lp + lr > 2048:
            continue
        out.append(Sample(prompt, lp, lr if lr > 0 else default_out))
        if len(out) >= n:
            break
    return out


async def arrivals(samples: list[Sample], rate: float, burstiness: float, rng: random.Random):
    for s in samples:
        yield s
        if rate != float("inf"):
            # gamma inter-arrival times; burstiness 1 = Poisson process
            await asyncio.sleep(rng.gammavariate(burstiness, 1.0 / (rate * burstiness)))


async def one_request(session, url: str, model: str, s: Sample, chat: bool, ignore_eos: bool, temperature: float) -> Result:
    body = {"model": model, "max_tokens": s.max_tokens, "stream": True, "temperature": temperature,
            "stream_options": {"include_usage": True}}
    if ignore_eos:
        body["ignore_eos"] = True
    if chat:
        body["messages"] = [{"role": "user", "content": s.prompt}]
    else:
        body["prompt"] = s.prompt
    r = Result(prompt_len=s.prompt_len)
    t0 = time.perf_counter()
    last = t0
    try:
        async with session.post(url, json=body) as resp:
            if resp.status != 200:
                r.error = f"HTTP {resp.status}: {(await resp.text())[:200]}"
                return r
            buf = b""
            async for chunk in resp.content.iter_any():
                buf += chunk
                while b"\n\n" in buf:
                    line, buf = buf.split(b"\n\n", 1)
                    line = line.strip()
                    if not line.startswith(b"data:"):
                        continue
                    payload = line[5:].strip()
                    if payload == b"[DONE]":
                        continue
                    d = json.loads(payload)
                    usage = d.get("usage")
                    if usage and usage.get("completion_tokens") is not None:
                        r.output_tokens = int(usage["completion_tokens"])
                        r.prompt_len = int(usage.get("prompt_tokens", r.prompt_len))
                    choices = d.get("choices") or []
                    if not choices:
                        continue
                    c = choices[0]
                    text = (c.get("delta") or {}).get("content") if chat else c.get("text")
                    if text is not None:      # a token may decode to an empty string
                        now = time.perf_counter()
                        if r.ttft == 0.0:
                            r.ttft = now - t0
                        else:
                            r.itl.append(now - last)
                        last = now
            r.latency = time.perf_counter() - t0
            if r.output_tokens == 0:
                r.output_tokens = len(r.itl) + (1 if r.ttft else 0)
            r.ok = r.ttft > 0
            if not r.ok:
                r.error = "no tokens received"
    except Exception as exc:  # connection errors count as failed requests
        r.error = repr(exc)
    return r


def pct(xs: list[float], p: float) -> float:
    if not xs:
        return 0.0
    xs = sorted(xs)
    k = min(len(xs) - 1, max(0, int(round(p / 100.0 * (len(xs) - 1)))))
    return xs[k]


def summarise(results: list[Result], duration: float, slo: dict) -> dict:
    ok = [r for r in results if r.ok]
    tpot = [(r.latency - r.ttft) / (r.output_tokens - 1) for r in ok if r.output_tokens > 1]
    itl = [x for r in ok for x in r.itl]

    def block(name, xs):
        xs_ms = [x * 1e3 for x in xs]
        return {f"mean_{name}_ms": statistics.fmean(xs_ms) if xs_ms else 0.0, f"median_{name}_ms": pct(xs_ms, 50),
                f"p99_{name}_ms": pct(xs_ms, 99)}

    out = {"completed": len(ok), "failed": len(results) - len(ok), "duration_s": duration,
           "total_input_tokens": sum(r.prompt_len for r in ok), "total_output_tokens": sum(r.output_tokens for r in ok),
           "request_throughput": len(ok) / duration if duration else 0.0,
           "output_throughput": sum(r.output_tokens for r in ok) / duration if duration else 0.0,
           "total_token_throughput": sum(r.prompt_len + r.output_tokens for r in ok) / duration if duration else 0.0}
    out.update(block("ttft", [r.ttft for r in ok]))
    out.update(block("tpot", tpot))
    out.update(block("itl", itl))
    out.update(block("e2el", [r.latency for r in ok]))
    if slo:
        good = 0
        for r in ok:
            t = (r.latency - r.ttft) / (r.output_tokens - 1) if r.output_tokens > 1 else 0.0
            if r.ttft * 1e3 <= slo.get("ttft", float("inf")) and t * 1e3 <= slo.get("tpot", float("inf")) \
                    and r.latency * 1e3 <= slo.get("e2el", float("inf")):
                good += 1
        out["request_goodput"] = good / duration if duration else 0.0
    errs = [r.error for r in results if not r.ok]
    if errs:
        out["first_error"] = errs[0]
    return out


async def run(args, samples: list[Sample]) -> dict:
    import aiohttp

    url = args.base_url.rstrip("/") + ("/v1/chat/completions" if args.chat else "/v1/completions")
    rng = random.Random(args.seed)
    sem = asyncio.Semaphore(args.max_concurrency) if args.max_concurrency else None
    timeout = aiohttp.ClientTimeout(total=args.timeout)
    async with aiohttp.ClientSession(timeout=timeout, connector=aiohttp.TCPConnector(limit=0)) as session:
        async def guarded(s):
            if sem is None:
                return await one_request(session, url, args.model, s, args.chat, args.ignore_eos, args.temperature)
            async with sem:
                return await one_request(session, url, args.model, s, args.chat, args.ignore_eos, args.temperature)

        t0 = time.perf_counter()
        tasks = []
        async for s in arrivals(samples, args.request_rate, args.burstiness, rng):
            tasks.append(asyncio.create_task(guarded(s)))
        results = await asyncio.gather(*tasks)
        duration = time.perf_counter() - t0
    slo = {}
    for item in args.goodput or []:
        k, v = item.split(":")
        slo[k] = float(v)
    return summarise(results, duration, slo)


def main(argv: Optional[list[str]] = None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--base-url", default="http://127.0.0.1:3000")
    ap.add_argument("--model", default="default")
    ap.add_argument("--chat", action="store_true", help="use /v1/chat/completions instead of /v1/completions")
    ap.add_argument("--dataset", default="random", choices=["random", "jsonl", "sharegpt", "hf", "wildchat"])
    ap.add_argument("--hf-text-column", default="", help="hf dataset: column that holds the prompt")
    ap.add_argument("--hf-output-column", default="", help="hf dataset: column whose length sets the output budget")
    ap.add_argument("--byte-tokens", action="store_true",
                    help="random dataset: prompts of exactly N characters (servers with the byte-level tokenizer)")
    ap.add_argument("--dataset-path", default="")
    ap.add_argument("--tokenizer", default="", help="local tokenizer directory for the random dataset")
    ap.add_argument("--num-prompts", type=int, default=1000)
    ap.add_argument("--random-input-len", type=int, default=1024)
    ap.add_argument("--random-output-len", type=int, default=128)
    ap.add_argument("--random-range-ratio", type=float, default=0.0)
    ap.add_argument("--random-prefix-len", type=int, default=0)
    ap.add_argument("--request-rate", type=float, default=float("inf"))
    ap.add_argument("--burstiness", type=float, default=1.0)
    ap.add_argument("--max-concurrency", type=int, default=0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--goodput", nargs="*", help="SLOs as ttft:ms tpot:ms e2el:ms")
    ap.add_argument("--timeout", type=float, default=6 * 3600)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--save-result", default="")
    args = ap.parse_args(argv)
    tok = None
    if args.tokenizer:
        from parallax_b200.frontend.tokenizer import TokenizerWrapper

        tok = TokenizerWrapper.from_pretrained(args.tokenizer)
    if args.dataset == "random":
        samples = make_random_dataset(args.num_prompts, args.random_input_len, args.random_output_len,
                                      args.random_range_ratio, args.seed, tok, args.random_prefix_len,
                                      byte_level=args.byte_tokens)
    elif args.dataset == "hf":
        samples = load_hf_dataset(args.dataset_path, args.num_prompts, args.random_output_len, args.seed, tok,
                                  args.hf_text_column, args.hf_output_column)
    elif args.dataset == "wildchat":
        samples = load_wildchat_dataset(args.dataset_path, args.num_prompts, args.random_output_len, args.seed, tok)
    elif args.dataset == "sharegpt":
        samples = load_sharegpt_dataset(args.dataset_path, args.num_prompts, args.random_output_len, args.seed, tok)
    else:
        samples = load_jsonl_dataset(args.dataset_path, args.num_prompts, args.random_output_len)
    report = asyncio.run(run(args, samples))
    print(json.dumps(report, indent=1))
    if args.save_result:
        with open(args.save_result, "w") as f:
            json.dump(report, f, indent=1)
    return report


if __name__ == "__main__":
    main()
