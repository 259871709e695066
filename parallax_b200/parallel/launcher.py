"""Process launcher of the multi-GPU engine: one process per GPU on one box.

The calling process becomes rank 0 (scheduler, HTTP frontend, first pipeline stage); ranks
1..N-1 are child processes running :meth:`DistEngine.serve_forever`. Rendezvous is a TCP store
on 127.0.0.1. The reference starts one subprocess per tensor-parallel rank with a pipe for
liveness (``src/parallax/launch.py:230-318``) and lets SGLang or MLX build the process group;
here the same launcher also covers in-box pipeline stages.
"""

from __future__ import annotations

import json
import logging
import os
import socket
import subprocess
import sys
import time
from typing import Optional

logger = logging.getLogger(__name__)

_ENGINE_KEYS = ("page_size", "kv_fraction", "max_batch_size", "max_num_tokens_per_batch", "micro_batch_ratio",
                "chunked_prefill_size", "max_prefill_tokens_per_batch", "enable_prefix_cache", "max_total_length", "request_timeout_s", "num_blocks",
                "seed", "fused", "executor_thread", "align_rows", "max_in_flight", "ep", "kv_cache_dtype", "linear_prefix_slots", "lora")


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def init_process_group(rank: int, world: int, port: int, device_type: str) -> None:
    import datetime

    # Ranks run kernels that wait for each other (NCCL receives, peer-memory flags). CUDA loads a kernel on
    # its first launch and that load waits for the context to drain, which such a waiting kernel may not
    # allow for seconds: load everything when the context is created (must be set before CUDA starts).
    os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")

    import torch
    import torch.distributed as dist

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = str(port)
    if device_type == "cuda":
        torch.cuda.set_device(rank % torch.cuda.device_count())
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank % torch.cuda.device_count()),
                                timeout=datetime.timedelta(seconds=600))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=600))


def build_dist_engine(spec: dict):
    """Build this rank's :class:`DistEngine` from a JSON-able spec (same on every rank)."""
    import torch

    from parallax_b200.models.config import config_from_hf, named_config
    from parallax_b200.parallel.dist_engine import DistEngine, split_layers
    import torch.distributed as dist

    if spec.get("model_path"):
        with open(os.path.join(spec["model_path"], "config.json")) as f:
            cfg = config_from_hf(json.load(f))
    else:
        cfg = named_config(spec["model_name"])
    rank = dist.get_rank()
    device_type = spec.get("device_type", "cuda")
    device = torch.device("cuda", rank % torch.cuda.device_count()) if device_type == "cuda" else torch.device("cpu")
    dtype = getattr(torch, spec.get("dtype", "bfloat16")) if device_type == "cuda" else torch.float32
    pp, tp = spec["pp"], spec["tp"]
    weights = None
    if spec.get("model_path"):
        from parallax_b200.loader.shard_loader import ShardLoader, apply_lora_adapter

        start, end = split_layers(cfg.num_hidden_layers, pp)[rank // (tp * spec.get("ep", 1))]
        weights = ShardLoader(spec["model_path"], start, end).load_weights("cpu", None)
        for lp in spec.get("lora_paths") or []:
            apply_lora_adapter(weights, lp)
    kw = {k: spec[k] for k in _ENGINE_KEYS if k in spec and spec[k] is not None}
    from parallax_b200.frontend.tokenizer import LazyTokenizer

    # constrained decoding turns token ids into text on the rank that samples; loaded there on first use
    kw["tokenizer"] = LazyTokenizer(spec.get("model_path"), cfg.vocab_size)
    return DistEngine(cfg, pp, tp, device, dtype, weights=weights, weights_prefiltered=weights is not None, **kw)


def worker_main() -> None:
    """Entry point of ranks 1..N-1: ``python -m parallax_b200.parallel.launcher '<spec json>'``."""
    spec = json.loads(sys.argv[1])
    logging.basicConfig(level=spec.get("log_level", "INFO"))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    init_process_group(rank, world, int(os.environ["MASTER_PORT"]), spec.get("device_type", "cuda"))
    eng = build_dist_engine(spec)
    try:
        eng.serve_forever()
    finally:
        import torch.distributed as dist

        dist.destroy_process_group()


def spawn_workers(spec: dict, world: int, port: int) -> list[subprocess.Popen]:
    procs = []
    for rank in range(1, world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-m", "parallax_b200.parallel.launcher", json.dumps(spec)],
                                      env=env))
    return procs


def stop_workers(procs: list[subprocess.Popen], timeout: float = 20.0) -> None:
    deadline = time.time() + timeout
    for p in procs:
        try:
            p.wait(max(0.1, deadline - time.time()))
        except subprocess.TimeoutExpired:
            p.terminate()


def launch_dist_engine(spec: dict):
    """Spawn ranks 1..N-1, become rank 0. Returns ``(engine, child processes)``."""
    world = spec["pp"] * spec["tp"] * spec.get("ep", 1)
    port = spec.get("port") or free_port()
    procs = spawn_workers(spec, world, port)
    os.environ.update(RANK="0", WORLD_SIZE=str(world), LOCAL_RANK="0")
    init_process_group(0, world, port, spec.get("device_type", "cuda"))
    return build_dist_engine(spec), procs


def run_multi_gpu(args, cfg, name: str, path: Optional[str]) -> None:
    """``parallax run`` with ``--tp-size`` / ``--pp-size`` > 1 on one box: serve the OpenAI API
    from rank 0 over a :class:`DistEngine`."""
    import torch

    from parallax_b200.engine.service import EngineLoop
    from parallax_b200.frontend.openai_api import create_app
    from parallax_b200.frontend.tokenizer import TokenizerWrapper
    from parallax_b200.launch import serve_http
    from parallax_b200.utils.shared_state import SharedState

    # experts of MoE layers are sharded over the stage's tensor-parallel group, so an expert-parallel
    # size simply asks for a group of that many ranks; with --enable-dp-attention the expert-parallel
    # ranks instead each run attention on their own requests and meet only in the MoE layers
    ep_size = getattr(args, "ep_size", 1)
    dp_lanes = ep_size if (getattr(args, "enable_dp_attention", False) and ep_size > 1 and cfg.is_moe) else 1
    tp_size = args.tp_size if dp_lanes > 1 else max(args.tp_size, ep_size)
    device_type = "cuda" if torch.cuda.is_available() else "cpu"
    spec = dict(model_path=path, model_name=name.split("/")[-1], pp=args.pp_size, tp=tp_size, ep=dp_lanes,
                device_type=device_type,
                dtype=args.dtype if args.dtype in ("bfloat16", "float16") else "bfloat16",
                page_size=args.kv_block_size, kv_fraction=args.kv_cache_memory_fraction,
                kv_cache_dtype=getattr(args, "kv_cache_dtype", None),
                max_batch_size=args.max_batch_size, max_num_tokens_per_batch=args.max_num_tokens_per_batch,
                micro_batch_ratio=args.micro_batch_ratio, chunked_prefill_size=args.chunked_prefill_size,
                max_prefill_tokens_per_batch=getattr(args, "max_prefill_tokens_per_batch", 0) or None,
                enable_prefix_cache=args.enable_prefix_cache, max_total_length=args.max_sequence_length,
                request_timeout_s=args.request_timeout_s, num_blocks=None if device_type == "cuda" else 1024,
                lora_paths=(args.lora_paths or []) if args.enable_lora else [], log_level=args.log_level)
    if getattr(args, "enable_return_routed_experts", False):
        logger.warning("--enable-return-routed-experts is served by the single-process engine only; ignored here")
    from parallax_b200.launch import _lora_spec

    per_request = _lora_spec(args)
    if per_request is not None:
        # named adapters are served per request; a single unnamed one is merged into the weights at load
        spec["lora"], spec["lora_paths"] = per_request, []
    engine, procs = launch_dist_engine(spec)
    state = SharedState.create(in_process=True)
    state.set_layer_allocation(name, 0, cfg.num_hidden_layers, tp_size, changed=False)
    loop = EngineLoop(engine, shared_state=state)
    loop.start()
    tok = TokenizerWrapper.from_pretrained(path, vocab_size=cfg.vocab_size)
    app = create_app(loop, tok, name, max_model_len=args.max_sequence_length)
    state.set_status("available")
    logger.info("serving %s on http://%s:%d with pp=%d tp=%d dp-attention lanes=%d", name, args.host, args.port,
                args.pp_size, tp_size, dp_lanes)
    _server, thread = serve_http(app, args.host, args.port, args.log_level)
    try:
        while thread.is_alive():
            if any(p.poll() is not None for p in procs):
                raise RuntimeError("a worker rank exited; shutting the engine down")
            time.sleep(0.5)
    finally:
        loop.stop()
        engine.shutdown()
        stop_workers(procs)


if __name__ == "__main__":
    worker_main()
