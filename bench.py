"""Headline benchmark: steady-state serving throughput (output tokens/s) of Qwen3-8B bf16.

Workload (the headline configuration): 512 concurrent requests in a closed loop, 1024
input / 256 output uniform-random token ids, 50 % of the requests starting with one of 8
shared random 512-token prefixes (exercises the radix prefix cache), random-init N(0, 0.02)
weights, greedy sampling.

A "step" is one continuous-batching iteration of the engine (`Engine.step()`): every running
request decodes one token while the requests that finished are replaced by new ones whose
prompts are prefilled in the same forward pass. Before timing, the engine is brought to the
closed loop's steady state (untimed): request i starts with ``in + g_i`` context tokens and
``out - g_i`` tokens left to generate, g_i spread uniformly over [0, out), so that requests
finish and are admitted at the steady rate on every step, exactly as after a long run.

Numbers that come out of the same K timed steps:
  * ``value``  - output tokens / device time (CUDA events bracketing each step's GPU work);
  * ``e2e``    - output tokens / wall time through the public API (`Engine.step()`), including
    the per-step host-to-device copy of the packed index tensors from pinned memory and the
    device-to-host read of the sampled token ids;
  * ``ttft_ms_p50/p99``, ``tpot_ms_p50/p99`` - per request, over the requests that were admitted
    (TTFT) or finished (TPOT) inside the timed region.
With N GPUs the model runs as an N-stage pipeline (PP8 at N=8; ``--parallelism pp2tp4`` selects
two stages of four tensor-parallel ranks, ``dp`` N engine replicas). Rank 0 schedules; a few more
micro-batches than stages are in flight; a step is one rotation (every running request advances one
token). The same requests are served at every N (strong scaling); times are the max over ranks.

``--config`` selects the other named workloads (same JSON schema): ``qwen3-8b-pp2tp4``,
``qwen3-30b-a3b-ep8``, ``deepseek-v3-pp2ep4``, ``qwen3-32b-long-pp2tp4``. ``--impl vllm-stock`` runs the image's stock vLLM
on the headline workload as a labelled context arm (it is NOT the reference arm: ``--impl reference``
reports the reference as unavailable).

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

# name -> model, concurrency, input / output length, shared prefixes (count, length, fraction of requests),
# prefill chunk, default layout on N GPUs
WORKLOADS = {
    "qwen3-8b": dict(model="qwen3-8b", label="Qwen3-8B", conc=512, in_len=1024, out_len=256, prefixes=(8, 512, 0.5),
                     chunk=4096, layout="pp",
                     metric="output tok/s (Qwen3-8B bf16, 512 concurrent, 1024 in / 256 out, closed loop)"),
    "qwen3-8b-pp2tp4": dict(model="qwen3-8b", label="Qwen3-8B", conc=512, in_len=1024, out_len=256,
                            prefixes=(8, 512, 0.5), chunk=4096, layout="pp2tp",
                            metric="output tok/s (Qwen3-8B bf16, 512 concurrent, 1024 in / 256 out, closed loop)"),
    "qwen3-30b-a3b-ep8": dict(model="qwen3-30b-a3b", label="Qwen3-30B-A3B-shaped MoE", conc=1024, in_len=2048,
                              out_len=512, prefixes=None, chunk=4096, layout="ep",
                              metric="output tok/s (Qwen3-30B-A3B-shaped bf16, 1024 concurrent, 2048 in / 512 out, closed loop)"),
    "deepseek-v3-pp2ep4": dict(model="deepseek-v3.2", label="DeepSeek-V3-shaped 671B fp8 (MLA + sparse indexer)", conc=256,
                               in_len=4096, out_len=1024, prefixes=None, chunk=4096, layout="pp2ep",
                               metric="output tok/s (DeepSeek-V3-shaped fp8, 256 concurrent, 4096 in / 1024 out, closed loop)"),
    "qwen3-32b-long-pp2tp4": dict(model="qwen3-32b", label="Qwen3-32B-shaped", conc=64, in_len=32768, out_len=128,
                                  prefixes=None, chunk=8192, layout="pp2tp",
                                  metric="output tok/s (Qwen3-32B-shaped bf16, 64 concurrent, 32768 in / 128 out, 8192-token chunks, closed loop)"),
}


def reference_arm() -> None:
    # The reference cannot be installed without network access: its build backend (poetry-core) is
    # not available offline, and its GPU path needs sglang==0.5.12 / vllm==0.14.0 plus a Rust HTTP
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


def make_workload(wl: dict, rank: int, vocab: int):
    import torch

    g = torch.Generator().manual_seed(1234)
    n_pref, pref_len, frac = wl["prefixes"] or (0, 0, 0.0)
    prefixes = [torch.randint(0, vocab, (pref_len,), generator=g).tolist() for _ in range(n_pref)]
    gr = torch.Generator().manual_seed(99 + rank)

    def new_prompt(length: int) -> list[int]:
        body = torch.randint(0, vocab, (length,), generator=gr).tolist()
        if n_pref and float(torch.rand((), generator=gr)) < frac:
            k = int(torch.randint(0, n_pref, (), generator=gr))
            body[:pref_len] = prefixes[k]
        return body

    return new_prompt


def percentile(xs: list, q: float):
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))]


class LatencyLog:
    """Per-request time to first token and time per output token, from the tokens that came out
    inside the timed region: TTFT of every request admitted in the region whose first token arrived in
    it, TPOT = (time of last token - time of first token in the region) / (tokens in between) of every
    request with at least two tokens in the region."""

    def __init__(self):
        self.t_start = None
        self.ttft: list[float] = []
        self.span: dict = {}      # request id -> [time of first token in the region, time of last, count]

    def start(self) -> None:
        self.t_start = time.time()

    def token(self, req, now: float) -> None:
        if self.t_start is None:
            return
        rec = self.span.get(req.request_id)
        if rec is None:
            self.span[req.request_id] = [now, now, 1]
            if req.arrival_time >= self.t_start:      # admitted in the region: this is its first token
                self.ttft.append((now - req.arrival_time) * 1e3)
        else:
            rec[1] = now
            rec[2] += 1

    def summary(self) -> dict:
        tpot = [(b - a) / (n - 1) * 1e3 for a, b, n in self.span.values() if n > 1]
        r = lambda v: None if v is None else round(v, 2)  # noqa: E731
        return {"ttft_ms_p50": r(percentile(self.ttft, 0.5)), "ttft_ms_p99": r(percentile(self.ttft, 0.99)),
                "tpot_ms_p50": r(percentile(tpot, 0.5)), "tpot_ms_p99": r(percentile(tpot, 0.99)),
                "latency_samples": {"ttft": len(self.ttft), "tpot": len(tpot)}}


def result_line(args, wl, world, parallelism, tokens, dev_s, wall_s, launches, h2d, d2h, clocks, invalid, extra=None):
    pf = wl["prefixes"]
    out = {
        "metric": wl["metric"], "value": round(tokens / dev_s, 1), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_s / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp8 (block-scaled e4m3 weights, bf16 activations)" if "fp8" in wl["label"] else "bf16",
        "data": "synthetic uniform-random token ids, random-init N(0,0.02) weights",
        "config": {"model": wl["label"], "global_batch": args.concurrency, "seq_len": wl["in_len"] + wl["out_len"],
                   "input_len": wl["in_len"], "output_len": wl["out_len"],
                   "shared_prefix": f"{int(pf[2] * 100)}% of requests share one of {pf[0]} x {pf[1]} tokens" if pf else None,
                   "parallelism": parallelism,
                   "step": "one continuous-batching iteration over all running requests",
                   "l2": "inputs larger than L2 (weights and KV read per step are tens of GB)",
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


def pick_layout(wl: dict, par: str, world: int) -> tuple[str, int, int, int]:
    """(label, pp, tp, ep) for a workload on `world` GPUs."""
    import re

    if par == "auto":
        kind = wl["layout"]
        if kind == "pp2tp":
            par = f"pp2tp{world // 2}" if world >= 4 else (f"pp1tp{world}" if world > 1 else "pp1tp1")
        elif kind == "ep":
            par = f"ep{world}"
        elif kind == "pp2ep":
            par = f"pp2ep{world // 2}" if world >= 4 else f"ep{world}"
        else:
            # measured on B200s: two tensor-parallel ranks over the fused GEMM + collective kernels beat a
            # two-stage pipeline (17.9 k vs 15.1 k tok/s); from four GPUs on the pipeline wins (26.1 k vs 22.9 k)
            par = "tp" if world == 2 else f"pp{world}"
    m = re.fullmatch(r"pp(\d+)tp(\d+)", par)
    if m:
        pp, tp, ep = int(m.group(1)), int(m.group(2)), 1
    elif re.fullmatch(r"ep(\d+)", par):
        pp, tp, ep = 1, 1, int(par[2:])
    elif re.fullmatch(r"pp(\d+)ep(\d+)", par):
        m = re.fullmatch(r"pp(\d+)ep(\d+)", par)
        pp, tp, ep = int(m.group(1)), 1, int(m.group(2))
    elif par == "tp":
        pp, tp, ep = 1, world, 1
    else:
        m = re.fullmatch(r"pp(\d+)?", par)
        assert m, f"unknown parallelism {par}"
        pp, tp, ep = (int(m.group(1)) if m.group(1) else world), 1, 1
    assert pp * tp * ep == world, f"{par} does not fit {world} GPUs"
    label = f"pp{pp}" if pp > 1 or (tp == 1 and ep == 1) else ""
    label += f"tp{tp}" if tp > 1 else ""
    label += f"ep{ep}" if ep > 1 else ""
    return label, pp, tp, ep


def run_group(args, wl, cfg, par, world, rank, local_rank, device, invalid) -> None:
    """N GPUs as pipeline stages x tensor- or expert-parallel ranks behind one scheduler on rank 0."""
    import torch
    import torch.distributed as dist

    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.ops import cuda as cu
    from parallax_b200.parallel.dist_engine import DistEngine

    label, pp, tp, ep = pick_layout(wl, par, world)
    conc = args.concurrency
    in_len, out_len = wl["in_len"], wl["out_len"]
    # more micro-batches than stages, so that a stage always has one queued while the scheduler on rank 0
    # commits the tokens of another and plans its next turn; every micro-batch re-reads the stage's weights
    # and runs its GEMMs on fewer rows, so as few extra ones as keep the stages busy (measured: 4 at two
    # stages, where prompts run whole and the micro-batches are uneven; 5 at four stages, whose prompt
    # slices are capped: 26.1 k tok/s against 23.3 k with 6; 10 at eight stages: 32.5 k tok/s against
    # 27.9 k with 9, because one spare micro-batch no longer covers the scheduler's turn-around there)
    n_mb = args.micro_batches or (1 if pp == 1 else {2: 4, 4: 5, 8: 10}.get(pp, pp + 2))
    chunk = args.prefill_chunk or wl["chunk"]
    # deep pipelines: a micro-batch that carries whole prompts is several times heavier than the others
    # and every stage behind it runs dry. A cap on the prompt tokens per micro-batch, about 1.7x the
    # rate at which they arrive (requests x uncached prompt tokens per `out_len` decode steps, spread
    # over the micro-batches), spreads a prompt over consecutive micro-batches; the slices are trimmed so
    # that a micro-batch's rows fill whole 128-row GEMM tiles. Two stages are busy enough without it and
    # finer slices only cost kernel efficiency there.
    budget = args.prefill_budget
    align = 0
    if budget < 0:
        budget = 0
    elif budget == 0 and pp >= 4:
        pf = wl["prefixes"]
        uncached = in_len - (pf[2] * pf[1] if pf else 0)
        arrive = conc * uncached / out_len / n_mb
        budget = int(-(-1.66 * arrive // 64) * 64)
        align = 128
    max_len = in_len + out_len + 64
    kw = dict(page_size=16, kv_fraction=0.85, max_batch_size=conc, max_num_tokens_per_batch=max(8192, chunk) + conc,
              micro_batch_ratio=n_mb, max_in_flight=n_mb, chunked_prefill_size=chunk,
              max_prefill_tokens_per_batch=budget or None, align_rows=align, enable_prefix_cache=bool(wl["prefixes"]),
              max_total_length=max_len, request_timeout_s=None, seed=0)
    if ep > 1:
        kw["ep"] = ep
    eng = DistEngine(cfg, pp, tp, device, torch.bfloat16, **kw)
    if rank != 0:
        eng.serve_forever()
        dist.barrier()
        dist.destroy_process_group()
        return
    new_prompt = make_workload(wl, 0, cfg.vocab_size)
    greedy = dict(temperature=0.0, ignore_eos=True)
    lat = LatencyLog()

    def admit(n_out: int, length: int = in_len):
        r = Request(input_ids=new_prompt(length), sampling_params=SamplingParams(max_new_tokens=n_out, **greedy),
                    max_total_length=max_len)
        eng.add_request(r)
        return r

    initial = [admit(out_len - (i * out_len) // conc, in_len + (i * out_len) // conc) for i in range(conc)]

    def rotation() -> int:
        """One engine iteration per micro-batch: every running request advances by one token."""
        toks = 0
        for _ in range(n_mb):
            now = time.time()
            for req, tok in eng.step():
                if tok is not None:
                    toks += 1
                    lat.token(req, req.last_updated_time or now)
                if req.is_finished:
                    admit(out_len)
        return toks

    # The staggered start above is the steady state only if every initial request waits for the last prompt
    # before it decodes on: prompts first while the loop is being built, the serving policy afterwards.
    for pl in eng.planners:
        pl.scheduler.decode_first = False
    while any(r.is_prefill for r in initial):
        rotation()
    for pl in eng.planners:
        pl.scheduler.decode_first = True
    for _ in range(max(args.warmup, 0)):
        rotation()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    eng.mark()
    lat.start()
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
    pc = eng.cache.prefix_cache.get_stats() if getattr(eng.cache, "prefix_cache", None) else None
    host = {k: round(v / args.steps * 1e3, 2) for k, v in eng.host_s.items()}
    eng.shutdown()
    extra = {"prefix_cache": pc, "rank0_host_ms_per_step": host, "micro_batches": n_mb, "prefill_chunk": chunk,
             "prefill_budget": budget or None, "align_rows": align or None,
             "gpu_busy_ms_per_step_per_rank": [round(x / args.steps, 2) for x in res.get("busy_ms_per_rank", [])],
             "max_micro_batch_rows": max(res.get("max_rows_per_rank", [0]) or [0])}
    extra.update(lat.summary())
    print(json.dumps(result_line(args, wl, world, label, tokens, res["device_ms"] / 1e3, res["wall_s"], res["launches"],
                                 res["h2d_bytes"], 4 * tokens, clocks, invalid, extra)), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def vllm_stock_arm(args, wl) -> None:
    """Context arm: the image's stock vLLM (its own kernels, scheduler and CUDA graphs) on the same
    closed-loop workload, dummy weights of the same architecture. It is a point of comparison for
    what a stock NVIDIA serving stack reaches on this box; it is not the reference implementation."""
    import tempfile

    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")      # step the engine core in this process
    import torch

    from parallax_b200.models.config import named_config

    cfg = named_config(wl["model"])
    hf = dict(cfg.raw or {})
    hf.setdefault("architectures", ["Qwen3ForCausalLM"])
    hf.setdefault("model_type", "qwen3")
    hf.update(torch_dtype="bfloat16", max_position_embeddings=max(40960, wl["in_len"] + wl["out_len"] + 64),
              rms_norm_eps=cfg.rms_norm_eps, hidden_act="silu", attention_bias=False, bos_token_id=0, eos_token_id=1,
              tie_word_embeddings=bool(cfg.tie_word_embeddings))
    d = tempfile.mkdtemp(prefix="pxl_vllm_cfg_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    try:
        from vllm import LLM, SamplingParams
        import vllm
    except Exception as exc:      # noqa: BLE001
        print(json.dumps({"impl": "vllm-stock", "unavailable": f"vllm import failed: {exc}"[:300]}))
        return
    conc, in_len, out_len = args.concurrency, wl["in_len"], wl["out_len"]
    n = args.gpus
    try:
        llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
                  max_model_len=in_len + out_len + 64, max_num_seqs=conc, max_num_batched_tokens=8192 + conc,
                  enable_prefix_caching=bool(wl["prefixes"]), gpu_memory_utilization=0.88, seed=0,
                  pipeline_parallel_size=n if n > 1 else 1, disable_log_stats=True)
    except Exception as exc:      # noqa: BLE001
        print(json.dumps({"impl": "vllm-stock", "unavailable": f"vllm engine start failed: {type(exc).__name__}: {exc}"[:400]}))
        return
    engine = llm.llm_engine
    new_prompt = make_workload(wl, 0, cfg.vocab_size)
    rid = [0]
    arrival, first, last, count = {}, {}, {}, {}

    def admit(n_out: int, length: int = in_len) -> None:
        rid[0] += 1
        sp = SamplingParams(temperature=0.0, max_tokens=n_out, ignore_eos=True, detokenize=False)
        name = f"r{rid[0]}"
        arrival[name] = time.time()
        count[name] = 0
        engine.add_request(name, {"prompt_token_ids": new_prompt(length)}, sp)

    for i in range(conc):
        admit(out_len - (i * out_len) // conc, in_len + (i * out_len) // conc)
    lat_ttft, lat_tpot = [], []
    t_timed = [None]

    def one_step() -> int:
        toks = 0
        now_outs = engine.step()
        now = time.time()
        for o in now_outs:
            name = o.request_id
            n_tok = len(o.outputs[0].token_ids)
            new = n_tok - count.get(name, 0)
            if new > 0:
                toks += new
                count[name] = n_tok
                first.setdefault(name, now)
                last[name] = now
            if o.finished:
                if t_timed[0] is not None and name in first:
                    if arrival[name] >= t_timed[0]:
                        lat_ttft.append((first[name] - arrival[name]) * 1e3)
                    if n_tok > 1 and first[name] >= t_timed[0]:
                        lat_tpot.append((last[name] - first[name]) / (n_tok - 1) * 1e3)
                for dct in (arrival, first, last, count):
                    dct.pop(name, None)
                admit(out_len)
        return toks

    # untimed: all initial prompts prefilled, then the warm-up steps
    seen_first = 0
    t_lim = time.time() + 600
    while seen_first < conc and time.time() < t_lim:
        one_step()
        seen_first = sum(1 for k in first)
        if rid[0] > conc:      # some initial requests already finished and were replaced
            break
    for _ in range(max(args.warmup, 0)):
        one_step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    t_timed[0] = time.time()
    t0 = time.perf_counter()
    tokens = 0
    for _ in range(args.steps):
        tokens += one_step()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    r = lambda v: None if v is None else round(v, 2)  # noqa: E731
    print(json.dumps({
        "impl": f"stock vLLM {vllm.__version__} (context; not the reference arm)", "metric": wl["metric"],
        "value": round(tokens / wall, 1), "unit": "tokens/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(wall / args.steps * 1e3, 3), "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic uniform-random token ids, dummy weights", "timing": "wall clock around engine.step()",
        "config": {"model": wl["label"], "global_batch": conc, "input_len": in_len, "output_len": out_len,
                   "parallelism": f"pp{n}" if n > 1 else "single"},
        "ttft_ms_p50": r(percentile(lat_ttft, 0.5)), "tpot_ms_p50": r(percentile(lat_tpot, 0.5)),
        "ttft_ms_p99": r(percentile(lat_ttft, 0.99)), "tpot_ms_p99": r(percentile(lat_tpot, 0.99)),
        "clocks": clocks, "tokens": int(tokens)}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "vllm-stock"])
    ap.add_argument("--config", default="qwen3-8b", choices=sorted(WORKLOADS))
    ap.add_argument("--concurrency", type=int, default=0, help="0 = the workload's own")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (marks the run invalid)")
    ap.add_argument("--prefill-chunk", type=int, default=0, help="prompt tokens per prefill slice (0 = the workload's own)")
    ap.add_argument("--prefill-budget", type=int, default=0,
                    help="pipeline modes: prompt tokens per micro-batch over all requests (0 = default for the depth, -1 = no cap)")
    ap.add_argument("--micro-batches", type=int, default=0, help="pipeline modes: micro-batches in flight")
    ap.add_argument("--parallelism", default="auto",
                    help="auto (the workload's layout on N GPUs) | dp | pp | pp<P>tp<T> | ep<E> | pp<P>ep<E>")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    wl = WORKLOADS[args.config]
    if not args.concurrency:
        args.concurrency = wl["conc"]
    if args.impl == "vllm-stock":
        vllm_stock_arm(args, wl)
        return

    # every stage hop has its own two-rank communicator, which is what this warning asks for
    os.environ.setdefault("TORCH_NCCL_SHOW_EAGER_INIT_P2P_SERIALIZATION_WARNING", "false")
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # kernels of different ranks wait for one another (NCCL receives, peer-memory flags); loading a
        # kernel for the first time needs the whole context to drain, which a waiting kernel never lets
        # happen in time. Load every kernel when the context is created instead of on first launch.
        os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
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

    cfg = named_config(wl["model"])
    invalid = False
    if args.layers:
        cfg.num_hidden_layers = args.layers
        invalid = True
    par = args.parallelism
    if par != "dp" and world > 1:
        run_group(args, wl, cfg, par, world, rank, local_rank, device, invalid)
        return
    in_len, out_len = wl["in_len"], wl["out_len"]
    max_len = in_len + out_len + 64
    conc = args.concurrency // world
    chunk = args.prefill_chunk or wl["chunk"]
    eng = Engine(cfg, device=device, page_size=16, kv_fraction=0.88, max_batch_size=conc,
                 max_num_tokens_per_batch=max(8192, chunk) + conc, chunked_prefill_size=chunk,
                 enable_prefix_cache=bool(wl["prefixes"]), max_total_length=max_len, request_timeout_s=None, seed=rank)
    new_prompt = make_workload(wl, rank, cfg.vocab_size)
    greedy = dict(temperature=0.0, ignore_eos=True)
    lat = LatencyLog()

    def admit(n_out: int, length: int = in_len):
        r = Request(input_ids=new_prompt(length), sampling_params=SamplingParams(max_new_tokens=n_out, **greedy),
                    max_total_length=max_len)
        eng.add_request(r)
        return r

    # ---- untimed: bring the closed loop to its steady state
    initial = [admit(out_len - (i * out_len) // conc, in_len + (i * out_len) // conc) for i in range(conc)]
    # (prompts first while the loop is being built: the staggered start is the steady state only if every
    # initial request waits for the last prompt before it decodes on; the serving policy afterwards)
    eng.scheduler.decode_first = False
    while any(r.is_prefill for r in initial):
        for req, _tok in eng.step():
            if req.is_finished:
                admit(out_len)
    eng.scheduler.decode_first = True
    torch.cuda.synchronize()
    cu.check_status(device)

    def one_step(ev=None):
        done = eng.step(events=ev)
        toks = 0
        now = time.time()
        for req, tok in done:
            if tok is not None:
                toks += 1
                lat.token(req, req.last_updated_time or now)
            if req.is_finished:
                admit(out_len)
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
    lat.start()
    t0 = time.perf_counter()
    for k in range(args.steps):
        tokens += one_step(events[k])
        h2d += eng.last_step_stats.get("h2d_bytes", 0)
        d2h += eng.last_step_stats.get("d2h_bytes", 0)
    eng.flush()
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
        extra = {"prefix_cache": eng.cache.prefix_cache.get_stats() if eng.cache.prefix_cache else None}
        extra.update(lat.summary())
        out = result_line(args, wl, world, f"dp{world}" if world > 1 else "single", tokens, dev_s, wall_s, launches, h2d,
                          d2h, clocks, invalid, extra)
        out["config"]["timing"] = "CUDA events per step, max over ranks"
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
