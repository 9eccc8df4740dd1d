"""Typed configuration of the Qwen1.5-MoE architecture (``Qwen2MoeForCausalLM``).

Every size and constant of the model comes from ``config.json``; nothing is
fixed in code.  The reference reads the same quantities from GGUF metadata
(shared keys src/locus/model/llama.cpp:188-209, ``qwen2moe_hparams``
src/locus/model/arch.cpp:550-575) and derives ``head_dim = n_embd / n_heads``
(arch.cpp:553-559).  Here ``head_dim`` may also be given explicitly; the
projections are sized ``heads * head_dim``.

Options the reference fixes in code and this configuration carries as data:

* ``norm_topk_prob``: the reference hard-codes "no renormalisation" for this
  architecture (arch.cpp:571) but implements the renormalising branch in
  ``moe_select`` (llama.cpp:966-978); both are supported here.
* ``decoder_sparse_step`` / ``mlp_only_layers``: layer ``l`` is a sparse-MoE
  layer iff ``num_experts > 0``, ``l`` is not in ``mlp_only_layers`` and
  ``(l + 1) % decoder_sparse_step == 0``; other layers use the dense SwiGLU
  feed-forward of width ``intermediate_size`` (llama.cpp:493-503).
* ``use_sliding_window``: layers with index ``>= max_window_layers`` attend to
  the last ``sliding_window`` keys only (a query at position p sees keys t with
  ``p - sliding_window < t <= p``); the other layers see all keys.  The reference
  has no window for this architecture; the cache manager keeps such layers in a
  group of their own so that pages behind the window are given back.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Tuple

from .base import ConfigError, take


@dataclass(frozen=True)
class Qwen2MoeConfig:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    num_experts: int
    num_experts_per_tok: int
    norm_topk_prob: bool
    moe_intermediate_size: int
    shared_expert_intermediate_size: int
    decoder_sparse_step: int
    mlp_only_layers: Tuple[int, ...]
    qkv_bias: bool
    tie_word_embeddings: bool
    use_sliding_window: bool
    sliding_window: int
    max_window_layers: int
    eos_token_id: int
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    architecture = "Qwen2MoeForCausalLM"

    # ---- derived ---------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def is_moe_layer(self, layer: int) -> bool:
        return (
            self.num_experts > 0
            and layer not in self.mlp_only_layers
            and (layer + 1) % self.decoder_sparse_step == 0
        )

    def layer_window(self, layer: int) -> int:
        """Number of keys layer ``layer`` may look back on; 0 means all of them."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return 0

    # ---- parsing ---------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen2MoeConfig":
        hidden = take(raw, "hidden_size", int)
        layers = take(raw, "num_hidden_layers", int)
        heads = take(raw, "num_attention_heads", int)
        kv_heads = take(raw, "num_key_value_heads", int, heads)
        if hidden <= 0 or layers <= 0:
            raise ConfigError("config.json: hidden_size and num_hidden_layers must be positive")
        if heads <= 0:
            raise ConfigError("invalid head configuration: num_attention_heads must be positive")
        if "head_dim" in raw and raw["head_dim"] is not None:
            head_dim = take(raw, "head_dim", int)
        else:
            # the reference's rule (arch.cpp:553-556)
            if hidden % heads != 0:
                raise ConfigError(
                    f"invalid head configuration: hidden_size {hidden} is not a multiple "
                    f"of num_attention_heads {heads} and no head_dim is given"
                )
            head_dim = hidden // heads
        if head_dim <= 0 or head_dim % 2 != 0:
            raise ConfigError(f"invalid head configuration: head_dim {head_dim} must be even")
        if kv_heads <= 0 or heads % kv_heads != 0:
            # arch.cpp:557-559
            raise ConfigError(
                f"invalid kv head configuration: num_attention_heads {heads} is not a "
                f"multiple of num_key_value_heads {kv_heads}"
            )
        experts = take(raw, "num_experts", int, 0)
        top_k = take(raw, "num_experts_per_tok", int, 0)
        if experts < 0:
            raise ConfigError("config.json: num_experts must not be negative")
        if experts > 0 and not (1 <= top_k <= experts):
            # llama.cpp:198-204
            raise ConfigError(
                f"invalid num_experts_per_tok: {top_k} (must be 1..num_experts={experts})"
            )
        sparse_step = take(raw, "decoder_sparse_step", int, 1)
        if sparse_step <= 0:
            raise ConfigError("config.json: decoder_sparse_step must be positive")
        mlp_only = tuple(int(v) for v in take(raw, "mlp_only_layers", list, []))
        for v in mlp_only:
            if not (0 <= v < layers):
                raise ConfigError(f"config.json: mlp_only_layers names layer {v} of {layers}")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (silu only)")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: rope_scaling is not supported for this architecture")
        use_window = take(raw, "use_sliding_window", bool, False)
        window = take(raw, "sliding_window", int, 0)
        max_window_layers = take(raw, "max_window_layers", int, layers)
        if use_window and window <= 0:
            raise ConfigError("config.json: use_sliding_window needs a positive sliding_window")
        if not use_window:
            window = 0
        eps = take(raw, "rms_norm_eps", float, 1e-6)
        if not (eps > 0.0):
            raise ConfigError("config.json: rms_norm_eps must be positive")
        theta = take(raw, "rope_theta", float, 10000.0)
        if not (theta > 0.0):
            raise ConfigError("config.json: rope_theta must be positive")
        cfg = cls(
            vocab_size=take(raw, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=take(raw, "intermediate_size", int, 0),
            max_position_embeddings=take(raw, "max_position_embeddings", int),
            rms_norm_eps=eps,
            rope_theta=theta,
            num_experts=experts,
            num_experts_per_tok=top_k,
            norm_topk_prob=take(raw, "norm_topk_prob", bool, False),
            moe_intermediate_size=take(raw, "moe_intermediate_size", int, 0),
            shared_expert_intermediate_size=take(raw, "shared_expert_intermediate_size", int, 0),
            decoder_sparse_step=sparse_step,
            mlp_only_layers=mlp_only,
            qkv_bias=take(raw, "qkv_bias", bool, True),
            tie_word_embeddings=take(raw, "tie_word_embeddings", bool, False),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=max_window_layers,
            eos_token_id=_first_int(raw.get("eos_token_id"), -1),
            extra={k: v for k, v in raw.items()},
        )
        if cfg.vocab_size <= 0 or cfg.max_position_embeddings <= 0:
            raise ConfigError("config.json: vocab_size and max_position_embeddings must be positive")
        any_moe = any(cfg.is_moe_layer(l) for l in range(layers))
        any_dense = any(not cfg.is_moe_layer(l) for l in range(layers))
        if any_moe and cfg.moe_intermediate_size <= 0:
            raise ConfigError("config.json: missing key: moe_intermediate_size (the model has expert layers)")
        if any_dense and cfg.intermediate_size <= 0:
            raise ConfigError("config.json: missing key: intermediate_size (the model has dense layers)")
        if cfg.shared_expert_intermediate_size < 0:
            raise ConfigError("config.json: shared_expert_intermediate_size must not be negative")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` dictionary of this configuration."""
        return {
            "architectures": [self.architecture],
            "model_type": "qwen2_moe",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "hidden_act": "silu",
            "num_experts": self.num_experts,
            "num_experts_per_tok": self.num_experts_per_tok,
            "norm_topk_prob": self.norm_topk_prob,
            "moe_intermediate_size": self.moe_intermediate_size,
            "shared_expert_intermediate_size": self.shared_expert_intermediate_size,
            "decoder_sparse_step": self.decoder_sparse_step,
            "mlp_only_layers": list(self.mlp_only_layers),
            "qkv_bias": self.qkv_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "eos_token_id": self.eos_token_id,
        }


def _first_int(v, default: int) -> int:
    if isinstance(v, list) and v:
        v = v[0]
    if isinstance(v, bool) or not isinstance(v, int):
        return default
    return v
