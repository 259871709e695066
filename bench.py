"""Headline benchmark: steady-state serving throughput (output tokens/s) of Qwen3-8B bf16.

Workload (the config named in BASELINE.json): 512 concurrent requests in a closed loop, 1024
input / 256 output uniform-random token ids, 50 % of the requests starting with one of 8
shared random 512-token prefixes (exercises the radix prefix cache), random-init N(0, 0.02)
weights, greedy sampling.

A "step" is one continuous-batching iteration of the engine (`Engine.step()`): every running
request decodes one token while the requests that finished are replaced by new ones whose
prompts are prefilled in the same forward pass. Before timing, the engine is brought to the
closed loop's steady state (untimed): request i starts with ``1024 + g_i`` context tokens and
``256 - g_i`` tokens left to generate, g_i spread uniformly over [0, 256), so that two
requests finish and two are admitted on every step, exactly as after a long run.

Two numbers come out of the same K timed steps:
  * ``value``  — output tokens / device time (CUDA events bracketing each step's GPU work);
  * ``e2e``    — output tokens / wall time through the public API (`Engine.step()`), including
    the per-step host-to-device copy of the packed index tensors from pinned memory and the
    device-to-host read of the sampled token ids.
With N GPUs the model runs as an N-stage pipeline (the layout BASELINE.json names: PP8 at
N=8; ``--parallelism pp2tp4`` selects two stages of four tensor-parallel ranks, ``dp`` N engine
replicas). Rank 0 schedules; ``N+2`` micro-batches are in flight; a step is
one rotation (every running request advances one token). The same 512 requests are served at
every N (strong scaling); times are the max over ranks.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nproc-per-node 8 ... bench.py --gpus 8 --steps 64 --warmup 8
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

METRIC = "output tok/s (Qwen3-8B bf16, 512 concurrent, 1024 in / 256 out, closed loop)"
MODEL = "qwen3-8b"
CONCURRENCY = 512
IN_LEN, OUT_LEN = 1024, 256
N_PREFIXES, PREFIX_LEN, SHARED_FRAC = 8, 512, 0.5


def reference_arm() -> None:
    # The reference could not be installed offline: its build backend (poetry-core) is not in
    # the wheelhouse, and its GPU path needs sglang==0.5.12 / vllm==0.14.0 plus a Rust HTTP
    # frontend, none of which exist in this image.
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference not installable offline: poetry-core build backend, sglang 0.5.12 / "
                       "vllm 0.14.0, lattica and the Rust vllm-rs frontend are absent from the image",
    }))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_workload(rank: int, vocab: int):
    import torch

    g = torch.Generator().manual_seed(1234)
    prefixes = [torch.randint(0, vocab, (PREFIX_LEN,), generator=g).tolist() for _ in range(N_PREFIXES)]
    gr = torch.Generator().manual_seed(99 + rank)

    def new_prompt(length: int = IN_LEN) -> list[int]:
        body = torch.randint(0, vocab, (length,), generator=gr).tolist()
        if float(torch.rand((), generator=gr)) < SHARED_FRAC:
            k = int(torch.randint(0, N_PREFIXES, (), generator=gr))
            body[:PREFIX_LEN] = prefixes[k]
        return body

    return new_prompt


def result_line(args, world, parallelism, tokens, dev_s, wall_s, launches, h2d, d2h, clocks, invalid, extra=None):
    out = {
        "metric": METRIC, "value": round(tokens / dev_s, 1), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_s / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform-random token ids, random-init N(0,0.02) weights",
        "config": {"model": "Qwen3-8B", "global_batch": args.concurrency, "seq_len": IN_LEN + OUT_LEN,
                   "input_len": IN_LEN, "output_len": OUT_LEN,
                   "shared_prefix": "50% of requests share one of 8 x 512 tokens", "parallelism": parallelism,
                   "step": "one continuous-batching iteration over all running requests",
                   "l2": "inputs larger than L2 (16 GB weights + >80 GB KV read per step)",
                   "timing": "CUDA events, max over ranks"},
        "e2e": {"value": round(tokens / wall_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d / args.steps),
                "d2h_bytes_per_step": int(d2h / args.steps), "ms_per_step": round(wall_s / args.steps * 1e3, 3)},
        "gpu_launches": int(launches), "clocks": clocks, "tokens": int(tokens),
    }
    if extra:
        out.update(extra)
    if invalid:
        out["invalid"] = "debug run with a truncated model"
    return out


def run_pipeline(args, cfg, par, world, rank, local_rank, device, invalid) -> None:
    """N GPUs as pipeline stages (optionally x tensor-parallel ranks) behind one scheduler."""
    import re

    import torch
    import torch.distributed as dist

    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.ops import cuda as cu
    from parallax_b200.parallel.dist_engine import DistEngine

    m = re.fullmatch(r"pp(\d+)tp(\d+)", par)
    pp, tp = (int(m.group(1)), int(m.group(2))) if m else ((1, world) if par == "tp" else (world, 1))
    assert pp * tp == world, f"{par} does not fit {world} GPUs"
    conc = args.concurrency
    # a couple of micro-batches more than stages, so that a stage always has one queued while the
    # scheduler on rank 0 commits the tokens of another and plans its next turn
    n_mb = args.micro_batches or (1 if pp == 1 else pp + 2)
    # measured at pp2: slicing prompts finer (1024 / 512 tokens) to even out the micro-batches loses
    # more in kernel efficiency than it gains in balance, so prompts are prefilled in one piece
    chunk = args.prefill_chunk or 4096
    # deep pipelines: a micro-batch that carries whole prompts is several times heavier than the others
    # and every stage behind it runs dry (pp8: stages 50 % busy). A cap on the prompt tokens per
    # micro-batch, about 1.7x the rate at which they arrive (512 requests x ~768 uncached prompt tokens
    # per 256 decode steps, spread over the micro-batches), spreads a prompt over consecutive
    # micro-batches: pp8 20.3 k -> 32.7 k tok/s, stages 88 % busy. At pp2 the stages are already 94 % busy
    # and the finer slices only cost kernel efficiency (15.2 k -> 13.8 k), so no cap there.
    budget = args.prefill_budget
    if budget < 0:
        budget = 0
    elif budget == 0 and pp >= 8:
        arrive = conc * (IN_LEN - SHARED_FRAC * PREFIX_LEN) / OUT_LEN / n_mb
        budget = int(-(-1.66 * arrive // 64) * 64)
    eng = DistEngine(cfg, pp, tp, device, torch.bfloat16, page_size=16, kv_fraction=0.85, max_batch_size=conc,
                     max_num_tokens_per_batch=8192 + conc, micro_batch_ratio=n_mb, max_in_flight=n_mb,
                     chunked_prefill_size=chunk, max_prefill_tokens_per_batch=budget or None,
                     enable_prefix_cache=True, max_total_length=IN_LEN + OUT_LEN + 64, request_timeout_s=None, seed=0)
    if rank != 0:
        eng.serve_forever()
        dist.barrier()
        dist.destroy_process_group()
        return
    new_prompt = make_workload(0, cfg.vocab_size)
    greedy = dict(temperature=0.0, ignore_eos=True)

    def admit(n_out: int, length: int = IN_LEN):
        r = Request(input_ids=new_prompt(length), sampling_params=SamplingParams(max_new_tokens=n_out, **greedy),
                    max_total_length=IN_LEN + OUT_LEN + 64)
        eng.add_request(r)
        return r

    initial = [admit(OUT_LEN - (i * OUT_LEN) // conc, IN_LEN + (i * OUT_LEN) // conc) for i in range(conc)]

    def rotation() -> int:
        """One engine iteration per micro-batch: every running request advances by one token."""
        toks = 0
        for _ in range(n_mb):
            for req, tok in eng.step():
                if tok is not None:
                    toks += 1
                if req.is_finished:
                    admit(OUT_LEN)
        return toks

    while any(r.is_prefill for r in initial):
        rotation()
    for _ in range(max(args.warmup, 0)):
        rotation()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    eng.mark()
    tokens = 0
    for k in eng.host_s:
        eng.host_s[k] = 0.0
    for _ in range(args.steps):
        tokens += rotation()
    torch.cuda.synchronize()
    eng.mark()
    res = eng.elapsed()
    clocks = sampler.stop()
    cu.check_status(device)
    eng.shutdown()
    label = f"pp{pp}" + (f"tp{tp}" if tp > 1 else "")
    print(json.dumps(result_line(args, world, label, tokens, res["device_ms"] / 1e3, res["wall_s"], res["launches"],
                                 res["h2d_bytes"], 4 * tokens, clocks, invalid,
                                 {"prefix_cache": eng.cache.prefix_cache.get_stats() if eng.cache.prefix_cache else None,
                                  "rank0_host_ms_per_step": {k: round(v / args.steps * 1e3, 2) for k, v in eng.host_s.items()},
                                  "micro_batches": n_mb, "prefill_chunk": chunk, "prefill_budget": budget or None,
                                  "gpu_busy_ms_per_step_per_rank": [round(x / args.steps, 2) for x in res.get("busy_ms_per_rank", [])],
                                  "max_micro_batch_rows": max(res.get("max_rows_per_rank", [0]) or [0])})),
          flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--concurrency", type=int, default=CONCURRENCY)
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (marks the run invalid)")
    ap.add_argument("--prefill-chunk", type=int, default=0, help="pipeline modes: prompt tokens per prefill slice")
    ap.add_argument("--prefill-budget", type=int, default=0,
                    help="pipeline modes: prompt tokens per micro-batch over all requests (0 = default for the depth, -1 = no cap)")
    ap.add_argument("--micro-batches", type=int, default=0, help="pipeline modes: micro-batches in flight")
    ap.add_argument("--parallelism", default="auto", help="auto (single GPU, or ppN on N GPUs) | dp | pp | pp<P>tp<T>")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return

    import torch
    import torch.distributed as dist

    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.models.config import named_config
    from parallax_b200.ops import cuda as cu

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            sys.exit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    cfg = named_config(args.model)
    invalid = False
    if args.layers:
        cfg.num_hidden_layers = args.layers
        invalid = True
    par = args.parallelism
    if par == "auto":
        par = "pp" if world > 1 else "dp"
    if par != "dp" and world > 1:
        run_pipeline(args, cfg, par, world, rank, local_rank, device, invalid)
        return
    conc = args.concurrency // world
    eng = Engine(cfg, device=device, page_size=16, kv_fraction=0.88, max_batch_size=conc,
                 max_num_tokens_per_batch=8192 + conc, chunked_prefill_size=4096, enable_prefix_cache=True,
                 max_total_length=IN_LEN + OUT_LEN + 64, request_timeout_s=None, seed=rank)
    new_prompt = make_workload(rank, cfg.vocab_size)
    greedy = dict(temperature=0.0, ignore_eos=True)

    def admit(n_out: int, length: int = IN_LEN) -> None:
        eng.add_request(Request(input_ids=new_prompt(length), sampling_params=SamplingParams(max_new_tokens=n_out, **greedy),
                                max_total_length=IN_LEN + OUT_LEN + 64))

    # ---- untimed: bring the closed loop to its steady state
    initial = []
    for i in range(conc):
        g_i = (i * OUT_LEN) // conc
        r = Request(input_ids=new_prompt(IN_LEN + g_i), sampling_params=SamplingParams(max_new_tokens=OUT_LEN - g_i, **greedy),
                    max_total_length=IN_LEN + OUT_LEN + 64)
        initial.append(r)
        eng.add_request(r)
    while any(r.is_prefill for r in initial):
        for req, _tok in eng.step():
            if req.is_finished:
                admit(OUT_LEN)
    torch.cuda.synchronize()
    cu.check_status(device)

    def one_step(ev=None):
        done = eng.step(events=ev)
        toks = 0
        for req, tok in done:
            if tok is not None:
                toks += 1
            if req.is_finished:
                admit(OUT_LEN)
        return toks

    for _ in range(max(args.warmup, 0)):
        one_step()

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = cu.launch_count
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    tokens = 0
    h2d = d2h = 0
    t0 = time.perf_counter()
    for k in range(args.steps):
        tokens += one_step(events[k])
        h2d += eng.last_step_stats.get("h2d_bytes", 0)
        d2h += eng.last_step_stats.get("d2h_bytes", 0)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    dev_s = sum(a.elapsed_time(b) for a, b in events) / 1e3
    launches = cu.launch_count - launches0
    cu.check_status(device)

    stats = torch.tensor([dev_s, wall_s, float(tokens), float(launches), float(h2d), float(d2h)],
                         dtype=torch.float64, device=device)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        dev_s, wall_s = float(mx[0]), float(mx[1])
        tokens, launches, h2d, d2h = float(sm[2]), float(sm[3]), float(sm[4]), float(sm[5])
    if rank == 0:
        out = result_line(args, world, f"dp{world}" if world > 1 else "single", tokens, dev_s, wall_s, launches, h2d,
                          d2h, clocks, invalid,
                          {"prefix_cache": eng.cache.prefix_cache.get_stats() if eng.cache.prefix_cache else None})
        out["config"]["timing"] = "CUDA events per step, max over ranks"
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
