"""Node launcher (``parallax serve`` / ``parallax join``).

Standalone mode (``--model-path`` without ``--scheduler-addr``): load the whole model (or
``[--start-layer, --end-layer)``), start the engine loop and the OpenAI-compatible frontend on
``--port``. Scheduler mode (``--scheduler-addr``): join the cluster, wait up to 300 s for a
layer allocation, serve it, heartbeat every 10 s and rebuild the executor whenever the
scheduler moves this node to a different layer range. Mirrors the control flow of
``src/parallax/launch.py:89-309`` with in-process threads instead of helper processes.

Multi-GPU inside the box: ``--pp-size/--tp-size/--ep-size`` start one process per GPU through
``torch.distributed`` (see :mod:`parallax_b200.parallel.launcher`).
"""

from __future__ import annotations

import logging
import os
import threading
import time
from typing import Optional

from parallax_b200.args import parse_args
from parallax_b200.utils.logging_config import set_log_level
from parallax_b200.utils.shared_state import SharedState

logger = logging.getLogger(__name__)

_DTYPES = {"float16": "float16", "bfloat16": "bfloat16", "float32": "float32"}


def resolve_model(args):
    """(ModelConfig, weights-or-None, display name, local path or None)."""
    import torch  # noqa: F401

    from parallax_b200.models.config import named_config

    name = args.model_path or "tiny"
    if args.random_init or not (os.path.isdir(name) or "/" in name):
        try:
            return named_config(name.split("/")[-1]), None, name, None
        except KeyError:
            if args.random_init:
                raise
    from parallax_b200.loader.shard_loader import ShardLoader

    loader = ShardLoader(name, args.start_layer, args.end_layer, args.use_hfcache)
    return loader.config, loader, name, str(loader.model_path)


def build_engine(args, cfg, loader, start: int, end: int, shared_state=None):
    import torch

    from parallax_b200.engine.engine import Engine

    device = "cuda:0" if torch.cuda.is_available() else "cpu"
    dtype = getattr(torch, _DTYPES[args.dtype]) if device != "cpu" else torch.float32
    weights = None
    if loader is not None:
        weights = loader.load_weights("cpu", None)
        from parallax_b200.loader.shard_loader import apply_lora_adapter

        # a single adapter without a name is folded into the weights; named adapters ("name=path") are
        # kept apart and chosen per request
        for lp in (args.lora_paths or []) if args.enable_lora else []:
            if "=" not in lp and len(args.lora_paths) == 1:
                apply_lora_adapter(weights, lp)
    if (start, end) != (0, cfg.num_hidden_layers):
        raise ValueError("a partial layer range is served by a pipeline peer; use scheduler mode")
    return Engine(cfg, device=device, dtype=dtype, page_size=args.kv_block_size,
                  kv_fraction=args.kv_cache_memory_fraction, max_batch_size=args.max_batch_size,
                  max_num_tokens_per_batch=args.max_num_tokens_per_batch, micro_batch_ratio=args.micro_batch_ratio,
                  chunked_prefill_size=args.chunked_prefill_size, enable_prefix_cache=args.enable_prefix_cache,
                  max_total_length=args.max_sequence_length, request_timeout_s=args.request_timeout_s,
                  weights=weights, shared_state=shared_state,
                  num_blocks=None if device != "cpu" else 1024, lora=_lora_spec(args),
                  kv_cache_dtype=getattr(args, "kv_cache_dtype", None),
                  return_routed_experts=bool(getattr(args, "enable_return_routed_experts", False)))


def _lora_spec(args):
    """Per-request adapters: on with --enable-lora unless the only adapter given is unnamed (merged instead)."""
    if not getattr(args, "enable_lora", False):
        return None
    paths = args.lora_paths or []
    if len(paths) == 1 and "=" not in paths[0]:
        return None
    from parallax_b200.loader.lora import parse_lora_paths

    return {"max_loaded": args.max_loaded_loras or max(args.max_loras_per_batch, len(paths), 2),
            "max_rank": args.max_lora_rank or 64, "paths": parse_lora_paths(paths)}


def serve_http(app, host: str, port: int, log_level: str = "info"):
    import uvicorn

    config = uvicorn.Config(app, host=host, port=port, log_level=log_level.lower())
    server = uvicorn.Server(config)
    t = threading.Thread(target=server.run, name="HttpFrontend", daemon=True)
    t.start()
    return server, t


def run_standalone(args) -> None:
    from parallax_b200.engine.service import EngineLoop
    from parallax_b200.frontend.openai_api import create_app
    from parallax_b200.frontend.tokenizer import TokenizerWrapper

    state = SharedState.create(in_process=True)
    cfg, loader, name, path = resolve_model(args)
    start = 0 if args.start_layer is None else args.start_layer
    end = cfg.num_hidden_layers if args.end_layer is None else args.end_layer
    state.set_layer_allocation(name, start, end, args.tp_size, changed=False)
    if (start, end) != (0, cfg.num_hidden_layers):
        run_static_peer(args, state, name, start, end)     # one peer of a pipeline (tensor-parallel with --tp-size)
        return
    if args.pp_size * args.tp_size * args.ep_size > 1:
        from parallax_b200.parallel.launcher import run_multi_gpu

        run_multi_gpu(args, cfg, name, path)
        return
    engine = build_engine(args, cfg, loader, start, end, state)
    tok = TokenizerWrapper.from_pretrained(path, vocab_size=cfg.vocab_size)
    engine.tokenizer = tok           # requests with a JSON schema check candidate tokens by their text
    loop = EngineLoop(engine, shared_state=state)
    loop.start()
    app = create_app(loop, tok, name, max_model_len=args.max_sequence_length)
    if args.engine_core_input_addr and args.engine_core_output_addr:
        from parallax_b200.frontend.engine_core_server import EngineCoreServer

        core = EngineCoreServer(loop, args.engine_core_input_addr, args.engine_core_output_addr,
                                max_model_len=args.max_sequence_length, dtype=args.dtype,
                                block_size=args.kv_block_size, num_gpu_blocks=engine.cache.num_blocks)
        core.start()
        logger.info("engine-core protocol: requests from %s, outputs to %s", args.engine_core_input_addr,
                    args.engine_core_output_addr)
    state.set_status("available")
    logger.info("serving %s on http://%s:%d (layers [%d, %d))", name, args.host, args.port, start, end)
    server, thread = serve_http(app, args.host, args.port, args.log_level)
    try:
        while thread.is_alive():
            time.sleep(0.5)
    except KeyboardInterrupt:
        pass
    finally:
        server.should_exit = True
        loop.stop()


def run_static_peer(args, state: SharedState, name: str, start: int, end: int) -> None:
    """``parallax serve --start-layer a --end-layer b --initial-peers <other nodes>``: one stage of a pipeline
    whose nodes find each other without a scheduler (the first node serves the API and routes by layer range)."""
    from parallax_b200.p2p.node_runtime import NodeRuntime
    from parallax_b200.p2p.static_peers import StaticAgent, StaticPeers

    host = "127.0.0.1" if args.host in ("localhost", "0.0.0.0") else args.host
    url = args.announce_maddrs[0] if args.announce_maddrs else f"http://{host}:{args.port}"
    if "://" not in url:
        url = "http://" + url
    peers = StaticPeers(f"{host}:{args.port}", url, start, end, list(args.initial_peers or []))
    runtime = NodeRuntime(args, StaticAgent(peers), state, name, start, end)
    state.set_status("available")
    logger.info("serving layers [%d, %d) of %s on %s; peers: %s", start, end, name, url, peers.seeds or "none yet")
    try:
        while runtime.thread.is_alive():
            time.sleep(0.5)
    except KeyboardInterrupt:
        pass
    finally:
        runtime.shutdown()


def wait_for_allocation(state: SharedState, timeout_s: float = 300.0, poll_s: float = 0.2) -> Optional[dict]:
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        info = state.get_model_info()
        if info["block_start_index"] is not None and info["block_end_index"] is not None:
            return info
        time.sleep(poll_s)
    return None


def run_scheduler_mode(args) -> None:
    """Join a cluster and serve whatever layer range the scheduler assigns (reloading on change)."""
    from parallax_b200.p2p.node_runtime import NodeRuntime
    from parallax_b200.p2p.server import NodeAgent, SchedulerClient

    state = SharedState.create(in_process=True)
    host = "127.0.0.1" if args.host in ("localhost", "0.0.0.0") else args.host
    agent = NodeAgent(SchedulerClient(args.scheduler_addr), state, http_addr=f"http://{host}:{args.port}",
                      max_batch_size=args.max_batch_size, max_sequence_length=args.max_sequence_length,
                      param_mem_ratio=args.param_mem_ratio, kvcache_mem_ratio=args.kvcache_mem_ratio,
                      start_layer=args.start_layer, end_layer=args.end_layer)
    state.set_status("joining")
    agent.join()
    info = wait_for_allocation(state, 300.0)
    if info is None:
        raise SystemExit("no layer allocation received from the scheduler within 300 s")
    agent.start()
    own_model_path = args.model_path      # None: serve whatever model the scheduler names, also after it changes
    try:
        while True:
            info = state.get_model_info()
            args.model_path = own_model_path or info["model_name"]
            runtime = NodeRuntime(args, agent, state, info["model_name"], info["block_start_index"],
                                  info["block_end_index"])
            agent.on_refit = runtime.apply_refit
            state.update(_layer_allocation_changed=False)
            state.set_status("available")
            from parallax_b200.utils.banner import display_parallax_join

            display_parallax_join(info["model_name"], info["block_start_index"], info["block_end_index"])
            runtime.serve_until_allocation_changes()
            runtime.shutdown()
            logger.info("layer allocation changed; reloading the executor")
    except KeyboardInterrupt:
        pass
    finally:
        agent.stop()


def main(argv=None) -> None:
    args = parse_args(argv)
    set_log_level("DEBUG" if args.verbose else args.log_level)
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    if args.scheduler_addr:
        from parallax_b200.utils.version_check import check_latest_release

        check_latest_release()
        run_scheduler_mode(args)
    else:
        run_standalone(args)


if __name__ == "__main__":
    main()
