"""Qwen2-MoE (``Qwen2MoeForCausalLM``): configuration, layer plan and tensor names.

The reference reaches this architecture only through GGUF metadata
(model/ModelConfig.cajeta:190-191, expert keys :261-296, ``norm_topk_prob`` default
false :286-291, tie rule :318) and binds experts by ggml names
(model/MoeFfn.cajeta:454-519).  Reading the Hugging Face ``config.json`` keys, the
per-layer choice of feed-forward (``decoder_sparse_step``, ``mlp_only_layers``) and the
per-layer window (``use_sliding_window``, ``sliding_window``, ``max_window_layers``) are
this engine's own:

* layer ``l`` has the sparse mixture iff ``l`` is not in ``mlp_only_layers``,
  ``num_experts > 0`` and ``(l + 1) % decoder_sparse_step == 0``; otherwise a dense
  SwiGLU MLP of ``intermediate_size``;
* layer ``l`` attends over a window iff ``use_sliding_window`` and
  ``l >= max_window_layers``; the window counts the current token (keys
  ``[p + 1 - w, p]``, model/PagedKvCache.cajeta:382-388).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Tuple

from ..config.base import ConfigError, ConfigReader, ModelConfig, register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

ARCHITECTURE = "Qwen2MoeForCausalLM"


@dataclass(frozen=True)
class Qwen2MoeConfig(ModelConfig):
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    hidden_act: str
    use_sliding_window: bool
    sliding_window: int
    max_window_layers: int
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int
    norm_topk_prob: bool
    decoder_sparse_step: int
    mlp_only_layers: Tuple[int, ...]
    eos_token_ids: Tuple[int, ...]

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "Qwen2MoeConfig":
        arch = r.raw["architectures"][0]
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", heads, minimum=1)
        if heads % kv_heads != 0:
            raise ConfigError(f"{r.source}: num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        head_dim = r.optional_integer("head_dim")
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(f"{r.source}: hidden_size {hidden} is not a multiple of num_attention_heads {heads} and 'head_dim' is absent")
            head_dim = hidden // heads
        if head_dim < 2 or head_dim % 2 != 0:
            raise ConfigError(f"{r.source}: head_dim must be even and >= 2, found {head_dim}")
        act = r.string("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{r.source}: hidden_act '{act}' is not supported; supported: silu")
        if r.raw.get("rope_scaling") is not None:
            raise ConfigError(f"{r.source}: rope_scaling {r.raw['rope_scaling']!r} is not supported; supported: null")
        layers = r.integer("num_hidden_layers", minimum=1)
        experts = r.integer("num_experts", 0, minimum=0)
        top_k = r.integer("num_experts_per_tok", minimum=1) if experts > 0 else r.integer("num_experts_per_tok", 1)
        if experts > 0 and not 1 <= top_k <= experts:
            raise ConfigError(f"{r.source}: num_experts_per_tok must be between 1 and num_experts ({experts}), found {top_k}")
        use_window = r.boolean("use_sliding_window", False)
        window = r.integer("sliding_window", 0, minimum=0)
        max_window_layers = r.integer("max_window_layers", layers, minimum=0)
        if use_window and window < 1:
            raise ConfigError(f"{r.source}: use_sliding_window is true but sliding_window is {window}")
        sparse_step = r.integer("decoder_sparse_step", 1, minimum=1)
        mlp_only = r.integer_list("mlp_only_layers", ())
        for l in mlp_only:
            if not 0 <= l < layers:
                raise ConfigError(f"{r.source}: mlp_only_layers names layer {l}; the model has {layers}")
        eos = r.integer_list("eos_token_id", ())
        cfg = cls(
            architecture=arch,
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=r.integer("vocab_size", minimum=1),
            max_position_embeddings=r.integer("max_position_embeddings", 32768, minimum=1),
            rms_norm_eps=r.number("rms_norm_eps"),
            rope_theta=r.number("rope_theta", 10000.0),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            hidden_act=act,
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=max_window_layers,
            num_experts=experts,
            num_experts_per_tok=top_k,
            moe_intermediate_size=(r.integer("moe_intermediate_size", minimum=1) if experts > 0
                                   else r.integer("moe_intermediate_size", 0, minimum=0)),
            shared_expert_intermediate_size=r.integer("shared_expert_intermediate_size", 0, minimum=0),
            norm_topk_prob=r.boolean("norm_topk_prob", False),
            decoder_sparse_step=sparse_step,
            mlp_only_layers=tuple(sorted(set(mlp_only))),
            eos_token_ids=tuple(eos),
        )
        if cfg.rms_norm_eps <= 0.0:
            raise ConfigError(f"{r.source}: rms_norm_eps must be positive, found {cfg.rms_norm_eps}")
        if cfg.rope_theta <= 0.0:
            raise ConfigError(f"{r.source}: rope_theta must be positive, found {cfg.rope_theta}")
        return cfg

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2_moe",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "num_experts": self.num_experts,
            "num_experts_per_tok": self.num_experts_per_tok,
            "moe_intermediate_size": self.moe_intermediate_size,
            "shared_expert_intermediate_size": self.shared_expert_intermediate_size,
            "norm_topk_prob": self.norm_topk_prob,
            "decoder_sparse_step": self.decoder_sparse_step,
            "mlp_only_layers": list(self.mlp_only_layers),
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    # derived, per layer -------------------------------------------------------------
    def layer_is_sparse(self, layer: int) -> bool:
        return (layer not in self.mlp_only_layers and self.num_experts > 0
                and (layer + 1) % self.decoder_sparse_step == 0)

    def layer_window(self, layer: int) -> int:
        """Keys a query of this layer sees, counting itself; 0 means all of them."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return 0


def build_plan(cfg: Qwen2MoeConfig) -> ModelPlan:
    """Layer specs, run order and tensor names of one Qwen2-MoE model."""
    h = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"dim": h, "eps": cfg.rms_norm_eps})
    layers = []
    for l in range(cfg.num_hidden_layers):
        position = PartSpec("rope", {"head_dim": cfg.head_dim, "rotary_dim": cfg.head_dim, "theta": cfg.rope_theta})
        mixer = PartSpec("attention", {
            "hidden_size": h,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "window": cfg.layer_window(l),
            "qkv_bias": True,
            "out_bias": False,
            "scale": None,                 # 1/sqrt(head_dim), model/Attention.cajeta:67-71
            "position": position,
        })
        if cfg.layer_is_sparse(l):
            ffn = PartSpec("sparse_moe", {
                "hidden_size": h,
                "num_experts": cfg.num_experts,
                "top_k": cfg.num_experts_per_tok,
                "expert_intermediate_size": cfg.moe_intermediate_size,
                "shared_intermediate_size": cfg.shared_expert_intermediate_size,
                "shared_gate": cfg.shared_expert_intermediate_size > 0,
                "norm_topk_prob": cfg.norm_topk_prob,
            })
        else:
            ffn = PartSpec("dense_swiglu", {"hidden_size": h, "intermediate_size": cfg.intermediate_size})
        layers.append(LayerSpec(
            prefix=f"model.layers.{l}",
            block=PartSpec("prenorm", {"mixer_norm_name": "input_layernorm",
                                       "feed_forward_norm_name": "post_attention_layernorm",
                                       "mixer_name": "self_attn", "feed_forward_name": "mlp"}),
            mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm))
    plan = ModelPlan(
        architecture=cfg.architecture,
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        embedding_name="model.embed_tokens.weight",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=l) for l in range(cfg.num_hidden_layers)),
        final_norm=norm,
        final_norm_prefix="model.norm",
        lm_head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        eog_token_ids=cfg.eos_token_ids,
        max_position=cfg.max_position_embeddings,
    )
    plan.validate()
    return plan


register_architecture(ARCHITECTURE, Qwen2MoeConfig, build_plan, replace=True)
