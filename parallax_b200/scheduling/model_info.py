"""Shape / cost model of a transformer used by the cluster scheduler.

All decoder layers are assumed to cost the same. The estimates feed layer allocation
(parameter bytes per layer, KV bytes per token) and the roofline latency model (FLOPs and
bytes per layer for a request shape). Formulas follow
``src/scheduling/model_info.py:86-193`` of the reference so that allocations agree.
"""

from __future__ import annotations

from typing import Optional


class ModelInfo:
    def __init__(
        self,
        model_name: str = "",
        head_size: int = 128,
        hidden_dim: int = 4096,
        intermediate_dim: int = 12288,
        num_attention_heads: int = 32,
        num_kv_heads: int = 8,
        vocab_size: int = 151936,
        num_layers: int = 36,
        ffn_num_projections: int = 3,
        num_local_experts: Optional[int] = None,
        num_experts_per_tok: Optional[int] = None,
        moe_intermediate_dim: Optional[int] = None,
        tie_embedding: bool = False,
        param_bytes_per_element: float = 1,
        cache_bytes_per_element: int = 1,
        embedding_bytes_per_element: int = 1,
        qk_nope_head_dim: Optional[int] = None,
        qk_rope_head_dim: Optional[int] = None,
        v_head_dim: Optional[int] = None,
        mlx_model_name: str = "",
        mlx_param_bytes_per_element: float = 1,
        **extra,
    ):
        self.model_name = model_name
        self.mlx_model_name = mlx_model_name or model_name
        self.head_size = head_size
        self.hidden_dim = hidden_dim
        self.intermediate_dim = intermediate_dim
        self.num_attention_heads = num_attention_heads
        self.num_kv_heads = num_kv_heads
        self.vocab_size = vocab_size
        self.num_layers = num_layers
        self.ffn_num_projections = ffn_num_projections
        self.num_local_experts = num_local_experts
        self.num_experts_per_tok = num_experts_per_tok
        self.moe_intermediate_dim = moe_intermediate_dim
        self.tie_embedding = tie_embedding
        self.param_bytes_per_element = param_bytes_per_element
        self.mlx_param_bytes_per_element = mlx_param_bytes_per_element
        self.cache_bytes_per_element = cache_bytes_per_element
        self.embedding_bytes_per_element = embedding_bytes_per_element
        self.qk_nope_head_dim = qk_nope_head_dim
        self.qk_rope_head_dim = qk_rope_head_dim
        self.v_head_dim = v_head_dim
        for k, v in extra.items():
            setattr(self, k, v)
        if qk_nope_head_dim is not None and qk_rope_head_dim is not None:
            self.head_size_k = qk_nope_head_dim + qk_rope_head_dim
        else:
            self.head_size_k = head_size
        self.head_size_v = v_head_dim if v_head_dim is not None else head_size

    # ---- dims
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_size

    @property
    def k_dim(self) -> int:
        return self.num_kv_heads * self.head_size_k

    @property
    def v_dim(self) -> int:
        return self.num_kv_heads * self.head_size_v

    @property
    def mlx_bit_factor(self) -> float:
        return self.mlx_param_bytes_per_element / self.param_bytes_per_element

    # ---- memory
    @property
    def embedding_io_bytes(self) -> int:
        return self.embedding_bytes_per_element * self.vocab_size * self.hidden_dim

    @property
    def per_token_per_layer_kv_size(self) -> int:
        return self.cache_bytes_per_element * (self.k_dim + self.v_dim)

    def per_layer_kv_cache_size(self, *, batch_size: int = 1, source_seq_len: int = 256) -> int:
        return self.per_token_per_layer_kv_size * batch_size * source_seq_len

    def expected_num_activated_experts(self, *, batch_size: int = 1, target_seq_len: int = 1) -> Optional[int]:
        """E * (1 - (1 - k/E)^tokens): experts touched by a batch under uniform routing."""
        if self.num_local_experts is None or self.num_experts_per_tok is None:
            return None
        tokens = batch_size * target_seq_len
        e, k = self.num_local_experts, self.num_experts_per_tok
        return int(e * (1 - (1 - k / e) ** tokens))

    # ---- compute
    def decoder_layer_flops(self, *, batch_size: int = 1, target_seq_len: int = 1, source_seq_len: int = 256) -> int:
        t, h = target_seq_len, self.hidden_dim
        proj = 2 * 2 * t * h * h + 2 * t * h * (self.k_dim + self.v_dim)
        attn = 2 * h * t * source_seq_len * 2
        ffn = 2 * self.ffn_num_projections * t * h * self.intermediate_dim
        experts = self.expected_num_activated_experts(batch_size=batch_size, target_seq_len=target_seq_len)
        if experts is not None:
            ffn *= experts
        return batch_size * (proj + attn + ffn)

    def decoder_layer_io_bytes(self, roofline: Optional[bool] = None, *, batch_size: int = 1,
                               target_seq_len: int = 1, source_seq_len: int = 256) -> int:
        """Bytes per decoder layer: parameters (all experts) when sizing memory; parameters of
        the experts actually touched plus the KV cache read when ``roofline`` is set."""
        pb = self.param_bytes_per_element
        attn = pb * self.hidden_dim * self.q_dim * 2 + pb * self.hidden_dim * (self.k_dim + self.v_dim)
        inter = self.moe_intermediate_dim if self.moe_intermediate_dim is not None else self.intermediate_dim
        ffn = pb * self.ffn_num_projections * self.hidden_dim * inter
        kv = 0
        if roofline:
            experts = self.expected_num_activated_experts(batch_size=batch_size, target_seq_len=target_seq_len)
            if experts is not None:
                ffn *= experts
            kv = self.per_layer_kv_cache_size(batch_size=batch_size, source_seq_len=source_seq_len)
        elif self.num_local_experts is not None:
            ffn *= self.num_local_experts
        return round(ffn + kv + attn)

    def lm_head_flops(self, target_seq_len: int = 1) -> int:
        return 2 * target_seq_len * self.hidden_dim * self.vocab_size

    @classmethod
    def from_model_config(cls, cfg, model_name: str = "", param_bytes: float = 2, cache_bytes: int = 2) -> "ModelInfo":
        """Build from a :class:`parallax_b200.models.config.ModelConfig`."""
        return cls(
            model_name=model_name or cfg.architecture, head_size=cfg.head_dim, hidden_dim=cfg.hidden_size,
            intermediate_dim=cfg.intermediate_size, num_attention_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads, vocab_size=cfg.vocab_size, num_layers=cfg.num_hidden_layers,
            num_local_experts=cfg.num_experts or None, num_experts_per_tok=cfg.num_experts_per_tok or None,
            moe_intermediate_dim=cfg.moe_intermediate_size or None, tie_embedding=cfg.tie_word_embeddings,
            param_bytes_per_element=param_bytes, cache_bytes_per_element=cache_bytes,
            embedding_bytes_per_element=2,
            qk_nope_head_dim=cfg.qk_nope_head_dim or None, qk_rope_head_dim=cfg.qk_rope_head_dim or None,
            v_head_dim=cfg.v_head_dim or None,
        )
