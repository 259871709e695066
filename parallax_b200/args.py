"""Command-line flags of a serving node (``parallax serve`` / ``parallax join``).

Flag names and defaults are the public interface of the reference
(``src/parallax/server/server_args.py:16-388``) and are kept verbatim, including the
backend-selection flags that only exist for compatibility (this engine has exactly one GPU
backend; ``--attention-backend``, ``--moe-runner-backend``, ``--gpu-backend`` are accepted
and ignored). In-box topology flags are added: ``--pp-size``, ``--ep-size``.
"""

from __future__ import annotations

import argparse
from typing import Optional, Sequence


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="parallax_b200 serving node")
    # HTTP
    p.add_argument("--host", type=str, default="localhost", help="Host of the HTTP server.")
    p.add_argument("--port", type=int, default=3000, help="Port of the HTTP server")
    p.add_argument("--node-chat-port", type=int, default=3002, help="Port of the node chat HTTP server")
    # cluster / control channel
    p.add_argument("--initial-peers", nargs="+", default=[], help="List of initial peers")
    p.add_argument("--scheduler-addr", type=str, default=None, help="Scheduler address (host:port)")
    p.add_argument("--relay-servers", nargs="+", default=[], help="List of relay peers")
    p.add_argument("--tcp-port", type=int, default=0, help="Port of the node's control channel")
    p.add_argument("--udp-port", type=int, default=0, help="Unused; accepted for compatibility")
    p.add_argument("--announce-maddrs", nargs="+", default=[], help="Addresses to announce")
    p.add_argument("--dht-prefix", type=str, default="gradient", help="Prefix for registry keys")
    p.add_argument("--notify-url", type=str, default=None, help="URL to notify when a batch was forwarded")
    # model
    p.add_argument("--model-path", type=str, default=None, help="HF repo name or local checkpoint directory")
    p.add_argument("--max-sequence-length", type=int, default=32768, help="Maximum prompt + output length")
    p.add_argument("--param-mem-ratio", type=float, default=0.65, help="Memory share reserved for parameters")
    p.add_argument("--kvcache-mem-ratio", type=float, default=0.25, help="Memory share reserved for the KV cache")
    p.add_argument("--start-layer", type=int, default=None, help="First decoder layer of this shard (inclusive)")
    p.add_argument("--end-layer", type=int, default=None, help="Ending layer index for this shard (exclusive)")
    p.add_argument("--dtype", type=str, default="bfloat16", choices=["float16", "bfloat16", "float32"])
    # KV cache
    p.add_argument("--kv-cache-memory-fraction", type=float, default=0.8,
                   help="Fraction of the free device memory given to the KV cache")
    p.add_argument("--kv-block-size", type=int, default=16, help="Block size for KV cache management")
    p.add_argument("--kv-cache-dtype", type=str, default="auto", choices=["auto", "bf16", "fp8_e4m3"],
                   help="Storage type of the K / V pages of softmax-attention layers (auto: the model's dtype)")
    p.add_argument("--disable-prefix-cache", dest="enable_prefix_cache", action="store_false", default=True,
                   help="Disable the radix prefix cache")
    p.add_argument("--chunked-prefill-size", type=int, default=1024, help="Max prompt tokens per prefill chunk (0: off)")
    p.add_argument("--max-prefill-tokens-per-batch", type=int, default=0,
                   help="Prompt tokens one (micro-)batch carries over all requests; evens out the micro-batches "
                        "of an in-box pipeline (0: only the token budget limits them)")
    # batching
    p.add_argument("--max-batch-size", type=int, default=8, help="Maximum number of in-flight requests")
    p.add_argument("--max-num-tokens-per-batch", type=int, default=16384, help="Token budget of one forward pass")
    p.add_argument("--prefill-priority", type=int, default=0, choices=[0, 1])
    p.add_argument("--micro-batch-ratio", type=int, default=1, help="micro batch = max batch / ratio")
    p.add_argument("--scheduler-wait-ms", type=int, default=500, help="Scheduler wait time in milliseconds")
    p.add_argument("--request-timeout-s", type=int, default=600, help="Per-request timeout")
    # online weight refit
    p.add_argument("--enable-weight-refit", action="store_true", help="Enable runtime weight refit")
    p.add_argument("--weight-refit-mode", type=str, default="disk", help="'cpu' or 'disk'")
    # accepted for compatibility with the reference's multi-backend CLI
    p.add_argument("--attention-backend", type=str, default="flashinfer",
                   choices=["torch_native", "flashinfer", "triton", "fa3"])
    p.add_argument("--enable-dp-attention", action="store_true")
    p.add_argument("--moe-runner-backend", type=str, default="auto",
                   choices=["auto", "triton", "triton_kernel", "flashinfer_trtllm", "flashinfer_cutlass",
                            "flashinfer_mxfp4"])
    # LoRA
    p.add_argument("--enable-lora", action="store_true", help="Enable LoRA adapter support")
    p.add_argument("--max-lora-rank", type=int, default=None)
    p.add_argument("--lora-target-modules", nargs="*", type=str, default=None)
    p.add_argument("--lora-paths", nargs="*", type=str, default=None)
    p.add_argument("--max-loras-per-batch", type=int, default=2)
    p.add_argument("--max-loaded-loras", type=int, default=None)
    p.add_argument("--lora-eviction-policy", choices=["lru", "fifo"], default="lru")
    p.add_argument("--lora-backend", choices=["triton", "csgmv"], default="triton")
    p.add_argument("--max-lora-chunk-size", choices=[16, 32, 64, 128], type=int, default=16)
    p.add_argument("--fully-sharded-loras", action="store_true")
    p.add_argument("--enable-return-routed-experts", action="store_true",
                   help="Return the experts every token was routed to with non-streaming replies (rollout replay; "
                        "single-process engine, MoE models)")
    # parallelism
    p.add_argument("--tp-size", type=int, default=1, help="Tensor parallel size")
    p.add_argument("--dp-size", type=int, default=1, help="Data parallel size")
    p.add_argument("--pp-size", type=int, default=1, help="Pipeline stages inside this box (one GPU group each)")
    p.add_argument("--ep-size", type=int, default=1, help="Expert parallel size inside a stage")
    p.add_argument("--nccl-port", type=int, default=None, help="Rendezvous port of the in-box process group")
    # misc
    p.add_argument("--log-level", type=str, default="INFO", choices=["DEBUG", "INFO", "WARNING", "ERROR"])
    p.add_argument("--verbose", action="store_true", help="Enable verbose logging")
    p.add_argument("--gpu-backend", type=str, default="sglang", choices=["sglang", "vllm", "native"],
                   help="Accepted for compatibility; the sm_100a engine is always used")
    p.add_argument("--use-hfcache", action="store_true", default=False)
    p.add_argument("--random-init", action="store_true", help="Random N(0, 0.02) weights instead of a checkpoint")
    # engine-core wire protocol: serve an external frontend (e.g. vLLM's Rust HTTP frontend) over ZMQ
    p.add_argument("--engine-core-input-addr", type=str, default=None,
                   help="ZMQ endpoint of the frontend's request ROUTER (the engine connects a DEALER)")
    p.add_argument("--engine-core-output-addr", type=str, default=None,
                   help="ZMQ endpoint of the frontend's output PULL (the engine connects a PUSH)")
    return p


def parse_args(argv: Optional[Sequence[str]] = None) -> argparse.Namespace:
    args = build_parser().parse_args(argv)
    validate_args(args)
    return args


def validate_args(args: argparse.Namespace) -> None:
    if args.start_layer is not None and args.start_layer < 0:
        raise ValueError("start_layer must be non-negative")
    if args.end_layer is not None and args.end_layer <= (args.start_layer or 0):
        raise ValueError("end_layer must be greater than start_layer")
    if not 0.0 <= args.kv_cache_memory_fraction <= 1.0:
        raise ValueError("kv_cache_memory_fraction must be between 0.0 and 1.0")
    if getattr(args, "max_batch_size", None) is not None and args.max_batch_size <= 0:
        raise ValueError("max_batch_size must be positive")
    msl = getattr(args, "max_sequence_length", None)
    if msl is not None and msl <= 0:
        raise ValueError("max_sequence_len must be positive")
    if msl is None and getattr(args, "max_batch_size", None) is None:
        raise ValueError("max_sequence_len or max_batch_size must be provided")
    if args.max_num_tokens_per_batch <= 0:
        raise ValueError("max_num_tokens_per_batch must be positive")
    if args.kv_block_size <= 0:
        raise ValueError("kv_block_size must be positive")
    cps = getattr(args, "chunked_prefill_size", None)
    if cps is not None:
        if cps < 0:
            raise ValueError("chunked_prefill_size must be non-negative")
        if cps == 0:
            args.chunked_prefill_size = None
        elif cps % args.kv_block_size:
            # chunks end on block boundaries so that every chunk can be published to the prefix cache
            args.chunked_prefill_size = max(args.kv_block_size, cps - cps % args.kv_block_size)
    if args.micro_batch_ratio <= 0:
        raise ValueError("micro_batch_ratio must be positive")
    if args.scheduler_wait_ms < 0:
        raise ValueError("scheduler_wait_ms must be non-negative")
    if getattr(args, "request_timeout_s", None) is not None and args.request_timeout_s <= 0:
        raise ValueError("request_timeout_s must be positive")
    if args.enable_weight_refit and args.weight_refit_mode not in ("cpu", "disk"):
        raise ValueError("Unrecognized refit mode. Choose 'cpu' or 'disk'")
    if args.dtype not in ("float16", "bfloat16", "float32"):
        raise ValueError(f"Unsupported dtype: {args.dtype}")
    for name in ("tp_size", "dp_size", "pp_size", "ep_size"):
        if getattr(args, name, 1) <= 0:
            raise ValueError(f"{name} must be positive")
