"""Architecture registry: HF ``architectures[0]`` -> stage class.

The reference keeps one ``EntryClass`` per model file and looks it up by architecture name
(``src/parallax/server/shard_loader.py:79-112``, aliases ``:40-44``). Here one generic GQA
decoder covers the Llama/Qwen-style families through configuration flags, and dedicated
stage classes cover MLA/DSA (DeepSeek) and hybrid linear-attention models.
"""

from __future__ import annotations


from parallax_b200.models.config import ModelConfig

_REGISTRY: dict[str, str] = {
    # generic GQA decoder
    "LlamaForCausalLM": "decoder",
    "Qwen2ForCausalLM": "decoder",
    "Qwen3ForCausalLM": "decoder",
    "Qwen3MoeForCausalLM": "decoder",
    "Glm4MoeForCausalLM": "decoder",
    "MiniMaxM2ForCausalLM": "decoder",
    "GptOssForCausalLM": "decoder",
    "Step3p5ForCausalLM": "decoder",
    "MistralForCausalLM": "decoder",
    # MLA / DSA
    "DeepseekV3ForCausalLM": "deepseek",
    "DeepseekV32ForCausalLM": "deepseek",
    "GlmMoeDsaForCausalLM": "deepseek",
    "KimiK2ForCausalLM": "deepseek",
    # hybrid gated-delta-net
    "Qwen3NextForCausalLM": "hybrid",
    "Qwen3_5ForConditionalGeneration": "hybrid",
    "Qwen3_5MoeForConditionalGeneration": "hybrid",
    # block-sparse (MSA)
    "MiniMaxM3SparseForCausalLM": "msa",
}


def supported_architectures() -> list[str]:
    return sorted(_REGISTRY)


def family_of(arch: str) -> str:
    try:
        return _REGISTRY[arch]
    except KeyError as e:
        raise ValueError(f"unsupported architecture {arch!r}; supported: {supported_architectures()}") from e


def build_stage(cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype, max_positions=None,
                tp_rank: int = 0, tp_size: int = 1, tp_group=None, comm=None, ep_rank: int = 0, ep_size: int = 1,
                ep_comm=None, ep_local_init: bool = False):
    stage = _build_stage(cfg, start_layer, end_layer, device, dtype, max_positions, tp_rank, tp_size, tp_group, comm)
    if ep_size > 1:
        # experts over a group of their own (data-parallel attention): GQA decoders and the MLA families; the
        # other families split their experts over the tensor-parallel group of the stage
        own_group = family_of(cfg.architecture) in ("decoder", "deepseek")
        if not cfg.is_moe or not hasattr(stage, "set_expert_parallel") or not (own_group or tp_size > 1):
            raise ValueError(f"expert parallelism is not available for {cfg.architecture}")
        stage.set_expert_parallel(ep_rank, ep_size, ep_comm, ep_local_init)
    return stage


def _build_stage(cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype, max_positions, tp_rank, tp_size,
                 tp_group, comm):
    fam = family_of(cfg.architecture)
    if tp_size > 1 and fam != "decoder":
        from parallax_b200.models import tp_families

        cls = {"deepseek": tp_families.TPDeepseekStage, "hybrid": tp_families.TPHybridStage,
               "msa": tp_families.TPMSAStage}[fam]
        return cls(cfg, start_layer, end_layer, device, dtype, max_positions=max_positions, tp_rank=tp_rank,
                   tp_size=tp_size, tp_group=tp_group, comm=comm)
    if fam == "decoder":
        if tp_size > 1:
            from parallax_b200.models.decoder_tp import TPDecoderStage

            return TPDecoderStage(cfg, start_layer, end_layer, device, dtype, max_positions=max_positions,
                                  tp_rank=tp_rank, tp_size=tp_size, tp_group=tp_group, comm=comm)
        from parallax_b200.models.decoder import DecoderStage

        return DecoderStage(cfg, start_layer, end_layer, device, dtype, max_positions=max_positions)
    if fam == "deepseek":
        from parallax_b200.models.deepseek import DeepseekStage

        return DeepseekStage(cfg, start_layer, end_layer, device, dtype, max_positions=max_positions)
    if fam == "hybrid":
        from parallax_b200.models.hybrid import HybridStage

        return HybridStage(cfg, start_layer, end_layer, device, dtype, max_positions=max_positions)
    if fam == "msa":
        from parallax_b200.models.msa import MSAStage

        return MSAStage(cfg, start_layer, end_layer, device, dtype, max_positions=max_positions)
    raise ValueError(fam)
