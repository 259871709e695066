"""Offline generation: one prompt through the engine on this machine, with per-step timing.

    python -m parallax_b200.generate --model qwen3-0.6b --random-init --prompt "Hi" --max-tokens 64
    python -m parallax_b200.generate --model /models/Qwen3-8B --prompt "Why is the sky blue?" --topk 40 --temp 0.7

The reference ships the same tool for its own backend (``scripts/generate.py``: load, prefill, decode token by
token, then prompt / generation tokens per second, decode-step percentiles and peak memory). Here the prompt
runs through the serving engine itself (chunked prefill, paged KV, the lookahead off so that a step's wall time is
that step), so what is timed is what the server runs.
"""

from __future__ import annotations

import argparse
import statistics
import time
from typing import Optional


def percentile(values: list, q: float) -> float:
    """Linear interpolation between closest ranks; ``q`` in [0, 100]."""
    if not values:
        return float("nan")
    xs = sorted(values)
    pos = (len(xs) - 1) * q / 100.0
    lo = int(pos)
    hi = min(lo + 1, len(xs) - 1)
    return xs[lo] + (xs[hi] - xs[lo]) * (pos - lo)


def run(model: str, prompt: str, max_tokens: int = 256, topk: int = 1, temp: float = 1.0, random_init: bool = False,
        device: Optional[str] = None, chat: bool = True, out=print) -> dict:
    import torch

    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.frontend.tokenizer import TokenizerWrapper
    from parallax_b200.launch import resolve_model

    args = argparse.Namespace(model_path=model, random_init=random_init, start_layer=None, end_layer=None, use_hfcache=False)
    cfg, loader, name, path = resolve_model(args)
    device = device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    out(f"Loading {name} on {device} ...")
    t0 = time.perf_counter()
    weights = loader.load_weights("cpu", None) if loader is not None else None
    eng = Engine(cfg, device=device, dtype=torch.bfloat16 if device != "cpu" else torch.float32, weights=weights,
                 max_batch_size=1, max_total_length=min(32768, getattr(cfg, "max_position_embeddings", 32768) or 32768),
                 num_blocks=None if device != "cpu" else 512, async_scheduling=False)
    out(f"Loaded in {time.perf_counter() - t0:.1f} s")
    tok = TokenizerWrapper.from_pretrained(path, vocab_size=cfg.vocab_size)
    ids = tok.apply_chat_template([{"role": "user", "content": prompt}]) if chat else tok.encode(prompt)
    greedy = topk == 1 or temp <= 0
    sp = SamplingParams(max_new_tokens=max_tokens, temperature=0.0 if greedy else temp, top_k=0 if greedy else topk)
    if tok.eos_token_ids:
        sp.stop_token_ids = set(tok.eos_token_ids)
    req = Request(input_ids=list(ids), sampling_params=sp, max_total_length=eng.planner.max_total_length)
    eng.add_request(req)

    def sync():
        if device != "cpu":
            torch.cuda.synchronize()

    prefill_s, steps, first_seen = 0.0, [], False
    while eng.has_work():
        sync()
        t = time.perf_counter()
        eng.step()
        sync()
        dt = time.perf_counter() - t
        if not first_seen:
            prefill_s += dt            # prompt slices; the last of them yields the first token
            if req.output_ids:
                first_seen = True
                out(f"Prefill: {prefill_s * 1e3:.2f} ms")
        else:
            steps.append(dt * 1e3)
            out(f"Token {len(req.output_ids)} time: {dt * 1e3:.2f} ms")
    text = tok.decode(req.output_ids)
    out("\nGenerated Content:")
    out(text)
    out("-" * 20)
    res = {"prompt_tokens": req.prompt_len, "generated_tokens": len(req.output_ids), "text": text,
           "prompt_tps": req.prompt_len / prefill_s if prefill_s > 0 else 0.0,
           "generation_tps": len(steps) / (sum(steps) / 1e3) if steps else 0.0, "decode_ms": steps}
    out(f"Prompt: {res['prompt_tokens']} tokens, {res['prompt_tps']:.3f} tokens-per-sec")
    out(f"Generation: {res['generated_tokens']} tokens, {res['generation_tps']:.3f} tokens-per-sec")
    if steps:
        out("Decode step time (ms): " + ", ".join([
            f"min={min(steps):.2f}", f"median={percentile(steps, 50):.2f}", f"max={max(steps):.2f}",
            f"mean={sum(steps) / len(steps):.2f}", f"std={statistics.pstdev(steps):.2f}",
            f"p90={percentile(steps, 90):.2f}", f"p95={percentile(steps, 95):.2f}", f"p99={percentile(steps, 99):.2f}"]))
    else:
        out("Decode step time (ms): n/a")
    if device != "cpu":
        res["peak_memory_gb"] = torch.cuda.max_memory_allocated() / 1024 ** 3
        out(f"Peak memory: {res['peak_memory_gb']:.3f} GB")
    return res


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="Offline generation with per-step timing")
    ap.add_argument("--model", default="qwen3-0.6b", help="checkpoint directory, or a named architecture with --random-init")
    ap.add_argument("--prompt", default="Hi")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--topk", type=int, default=1)
    ap.add_argument("--temp", type=float, default=1.0)
    ap.add_argument("--random-init", action="store_true")
    ap.add_argument("--device", default=None)
    ap.add_argument("--no-chat-template", dest="chat", action="store_false")
    a = ap.parse_args(argv)
    run(a.model, a.prompt, a.max_tokens, a.topk, a.temp, a.random_init, a.device, a.chat)


if __name__ == "__main__":
    main()
