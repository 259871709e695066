"""Static knowledge of the cluster backend: supported models, sizes, join command.

Counterpart of ``src/backend/server/static_config.py:11-262`` without the Apple (MLX)
model-name mapping, which has no meaning on B200.
"""

from __future__ import annotations

import logging
import math
from typing import Optional

from parallax_b200.scheduling.model_info import ModelInfo

logger = logging.getLogger(__name__)

MODELS = [
    "Qwen/Qwen3-0.6B", "Qwen/Qwen3-1.7B", "Qwen/Qwen3-4B", "Qwen/Qwen3-8B", "Qwen/Qwen3-14B", "Qwen/Qwen3-32B",
    "Qwen/Qwen3-8B-FP8", "Qwen/Qwen3-32B-FP8", "Qwen/Qwen3-30B-A3B", "Qwen/Qwen3-235B-A22B-Instruct-2507-FP8",
    "Qwen/Qwen2.5-0.5B-Instruct", "Qwen/Qwen2.5-7B-Instruct", "Qwen/Qwen2.5-32B-Instruct",
    "Qwen/Qwen2.5-72B-Instruct", "Qwen/Qwen3-Next-80B-A3B-Instruct", "Qwen/Qwen3.5-35B-A3B",
    "deepseek-ai/DeepSeek-V3", "deepseek-ai/DeepSeek-V3.1", "deepseek-ai/DeepSeek-R1", "deepseek-ai/DeepSeek-V3.2",
    "moonshotai/Kimi-K2-Instruct", "openai/gpt-oss-20b", "openai/gpt-oss-120b", "zai-org/GLM-4.6",
    "zai-org/GLM-4.5-Air", "MiniMaxAI/MiniMax-M2", "MiniMaxAI/MiniMax-M3", "stepfun-ai/Step-3.5-Flash",
    "nvidia/Llama-3.1-8B-Instruct-FP8", "nvidia/Llama-3.3-70B-Instruct-FP8",
]

NODE_JOIN_COMMAND_LOCAL_NETWORK = "parallax join"
NODE_JOIN_COMMAND_PUBLIC_NETWORK = "parallax join -s {scheduler_addr} "

# shapes of the benchmark models, usable without a checkpoint on disk
_BUILTIN = {"Qwen/Qwen3-0.6B": "qwen3-0.6b", "Qwen/Qwen3-8B": "qwen3-8b", "Qwen/Qwen3-32B": "qwen3-32b",
            "Qwen/Qwen3-30B-A3B": "qwen3-30b-a3b", "deepseek-ai/DeepSeek-V3": "deepseek-v3",
            "deepseek-ai/DeepSeek-V3.2": "deepseek-v3.2"}


def get_param_bytes_per_element(config: dict, model_name: str = "") -> float:
    q = config.get("quantization_config") or config.get("quantization")
    method = config.get("quant_method")
    if method is None and q is not None:
        method = q.get("quant_method") or q.get("mode")
    if q is not None and q.get("bits") is not None:
        return q["bits"] / 8
    if method is None:
        return 2
    if method == "fp8":
        return 1
    if method in ("mxfp4", "int4", "awq", "gptq", "compressed-tensors"):
        return 0.5
    logger.warning("model %s: quant method %s unknown; assuming 1 byte per parameter", model_name, method)
    return 1


def model_info_from_config(config: dict, model_name: str) -> ModelInfo:
    experts = config.get("num_local_experts") or config.get("num_experts") or config.get("n_routed_experts")
    kvh = config.get("num_key_value_heads") or config.get("num_attention_groups") or 0
    pb = get_param_bytes_per_element(config, model_name)
    return ModelInfo(
        model_name=model_name, head_size=config.get("head_dim") or 128,
        qk_nope_head_dim=config.get("qk_nope_head_dim"), qk_rope_head_dim=config.get("qk_rope_head_dim"),
        v_head_dim=config.get("v_head_dim"), hidden_dim=config.get("hidden_size", 0),
        intermediate_dim=config.get("intermediate_size", 0), num_attention_heads=config.get("num_attention_heads", 0),
        num_kv_heads=kvh, vocab_size=config.get("vocab_size", 0), num_layers=config.get("num_hidden_layers", 0),
        ffn_num_projections=3, param_bytes_per_element=pb, mlx_param_bytes_per_element=pb,
        cache_bytes_per_element=2, embedding_bytes_per_element=2, num_local_experts=experts,
        num_experts_per_tok=config.get("num_experts_per_tok"), moe_intermediate_dim=config.get("moe_intermediate_size"),
        tie_embedding=bool(config.get("tie_word_embeddings", False)))


def get_model_info(model_name: str, use_hfcache: bool = False) -> ModelInfo:
    from parallax_b200.utils.model_download import load_config_only

    try:
        return model_info_from_config(load_config_only(model_name, local_files_only=use_hfcache), model_name)
    except Exception:
        from parallax_b200.models.config import named_config

        if model_name in _BUILTIN:
            return model_info_from_config(named_config(_BUILTIN[model_name]).raw, model_name)
        try:      # a named architecture (what `--random-init` serves), e.g. "qwen3-8b" or "tiny"
            return model_info_from_config(named_config(model_name.split("/")[-1]).raw, model_name)
        except KeyError:
            pass
        raise


_cache: Optional[dict] = None


def init_model_info_dict_cache(use_hfcache: bool = False) -> None:
    global _cache
    if _cache is not None:
        return
    _cache = {}
    for name in MODELS:
        try:
            _cache[name] = get_model_info(name, use_hfcache)
        except Exception as e:
            logger.debug("no config for %s: %s", name, e)
            _cache[name] = None


def get_model_info_dict_cache() -> dict:
    return _cache or {}


def estimate_vram_gb_required(model_info: Optional[ModelInfo], param_mem_ratio: float = 0.65) -> float:
    if model_info is None:
        return 0
    total = model_info.embedding_io_bytes + model_info.num_layers * model_info.decoder_layer_io_bytes(roofline=False)
    return total / 1024 ** 3 / param_mem_ratio


def get_model_list() -> list[dict]:
    info = get_model_info_dict_cache()
    return [{"name": n, "vram_gb": math.ceil(estimate_vram_gb_required(info.get(n)))} for n in MODELS]


def get_node_join_command(scheduler_addr: Optional[str], is_local_network: bool) -> Optional[dict]:
    if not scheduler_addr:
        return None
    tpl = NODE_JOIN_COMMAND_LOCAL_NETWORK if is_local_network else NODE_JOIN_COMMAND_PUBLIC_NETWORK
    return {"command": tpl.format(scheduler_addr=scheduler_addr)}
