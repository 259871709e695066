"""Random HF-named state dicts for the tiny test architectures (what a checkpoint of that family contains)."""

import torch

from parallax_b200.models.config import LINEAR, MSA_ATTENTION


def _gen(seed):
    g = torch.Generator().manual_seed(seed)
    return lambda *shape, scale=0.05: torch.randn(*shape, generator=g) * scale


def _mlp(sd, cfg, p, gi, rnd):
    H = cfg.hidden_size
    if cfg.layer_is_moe(gi):
        I = cfg.moe_intermediate_size
        sd[p + "mlp.gate.weight"] = rnd(cfg.num_experts, H)
        if cfg.architecture.startswith("Deepseek"):
            sd[p + "mlp.gate.e_score_correction_bias"] = rnd(cfg.num_experts)
            Is = I * int((cfg.raw or {}).get("n_shared_experts") or 0)
            if Is:
                for n, shape in (("gate_proj", (Is, H)), ("up_proj", (Is, H)), ("down_proj", (H, Is))):
                    sd[p + f"mlp.shared_experts.{n}.weight"] = rnd(*shape)
        for e in range(cfg.num_experts):
            sd[p + f"mlp.experts.{e}.gate_proj.weight"] = rnd(I, H)
            sd[p + f"mlp.experts.{e}.up_proj.weight"] = rnd(I, H)
            sd[p + f"mlp.experts.{e}.down_proj.weight"] = rnd(H, I)
    else:
        I = cfg.intermediate_size
        sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"] = rnd(I, H), rnd(I, H)
        sd[p + "mlp.down_proj.weight"] = rnd(H, I)


def hf_state_dict(cfg, family: str, seed: int = 0) -> dict:
    rnd = _gen(seed)
    H, D, Hq, Hkv = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    sd = {"model.embed_tokens.weight": rnd(cfg.vocab_size, H), "model.norm.weight": 1 + rnd(H)}
    if not cfg.tie_word_embeddings:
        sd["lm_head.weight"] = rnd(cfg.vocab_size, H)
    for gi in range(cfg.num_hidden_layers):
        p = f"model.layers.{gi}."
        a = p + "self_attn."
        sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"] = 1 + rnd(H), 1 + rnd(H)
        if family == "deepseek":
            ql, L, R = cfg.q_lora_rank, cfg.kv_lora_rank, cfg.qk_rope_head_dim
            nope, V = cfg.qk_nope_head_dim, cfg.v_head_dim
            sd[a + "q_a_proj.weight"], sd[a + "q_a_layernorm.weight"] = rnd(ql, H), 1 + rnd(ql)
            sd[a + "q_b_proj.weight"] = rnd(Hq * (nope + R), ql)
            sd[a + "kv_a_proj_with_mqa.weight"], sd[a + "kv_a_layernorm.weight"] = rnd(L + R, H), 1 + rnd(L)
            sd[a + "kv_b_proj.weight"] = rnd(Hq * (nope + V), L)
            sd[a + "o_proj.weight"] = rnd(H, Hq * V)
            if cfg.index_topk > 0:
                Hi, Di = cfg.index_n_heads, cfg.index_head_dim
                i = a + "indexer."
                sd[i + "wq_b.weight"], sd[i + "wk.weight"] = rnd(Hi * Di, ql), rnd(Di, H)
                sd[i + "k_norm.weight"], sd[i + "k_norm.bias"] = 1 + rnd(Di), rnd(Di)
                sd[i + "weights_proj.weight"] = rnd(Hi, H)
        elif family == "hybrid" and cfg.layer_kind(gi) == LINEAR:
            Hk, Hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
            Dk, Dv, Kc = cfg.linear_key_head_dim, cfg.linear_value_head_dim, cfg.linear_conv_kernel_dim
            la = p + "linear_attn."
            sd[la + "in_proj_qkv.weight"] = rnd(2 * Hk * Dk + Hv * Dv, H)
            sd[la + "in_proj_z.weight"] = rnd(Hv * Dv, H)
            sd[la + "in_proj_b.weight"], sd[la + "in_proj_a.weight"] = rnd(Hv, H), rnd(Hv, H)
            sd[la + "conv1d.weight"] = rnd(2 * Hk * Dk + Hv * Dv, 1, Kc, scale=0.3)
            sd[la + "A_log"], sd[la + "dt_bias"] = rnd(Hv, scale=0.5), rnd(Hv, scale=0.5)
            sd[la + "norm.weight"], sd[la + "out_proj.weight"] = 1 + rnd(Dv), rnd(H, Hv * Dv)
        else:
            gated = family == "hybrid"
            sd[a + "q_proj.weight"] = rnd(Hq * D * (2 if gated else 1), H)
            sd[a + "k_proj.weight"], sd[a + "v_proj.weight"] = rnd(Hkv * D, H), rnd(Hkv * D, H)
            sd[a + "o_proj.weight"] = rnd(H, Hq * D)
            if cfg.qk_norm or gated:
                sd[a + "q_norm.weight"], sd[a + "k_norm.weight"] = 1 + rnd(D), 1 + rnd(D)
            if family == "msa" and cfg.layer_kind(gi) == MSA_ATTENTION:
                sp = (cfg.raw or {})["sparse_attention_config"]
                Hi, Di = sp["sparse_num_index_heads"], sp["sparse_index_dim"]
                sd[a + "index_q_proj.weight"], sd[a + "index_k_proj.weight"] = rnd(Hi * Di, H, scale=0.1), rnd(Di, H, scale=0.1)
                sd[a + "index_q_norm.weight"], sd[a + "index_k_norm.weight"] = rnd(Di), rnd(Di)
        _mlp(sd, cfg, p, gi, rnd)
    return sd
