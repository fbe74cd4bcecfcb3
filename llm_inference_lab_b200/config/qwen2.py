"""Qwen2 dense GQA decoder: typed configuration and blueprint.

Keys, defaults and checks follow the reference's `Qwen2Config`
(rust/engine/src/runner/model/qwen2/engine.rs:197-216) and the validation in
`Qwen2Engine::load` (engine.rs:260-288).  Two things are wider here than in
the reference: the head size is read (``head_dim``, default
``hidden_size / num_attention_heads``) instead of being fixed at 64
(engine.rs:272), and ``use_sliding_window`` is honoured instead of refused
(engine.rs:262): layers with index >= ``max_window_layers`` then see only the
last ``sliding_window`` keys (a key at position j is visible to a query at
position p iff 0 <= p - j < sliding_window).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional

from .base import ConfigError, ModelConfig, finite_positive, optional, positive, required
from ..parts.spec import LayerCall, LayerSpec, ModelBlueprint, PartSpec


@dataclasses.dataclass
class Qwen2Config(ModelConfig):
    architecture = "Qwen2ForCausalLM"

    vocab_size: int = required(int, positive)
    hidden_size: int = required(int, positive)
    intermediate_size: int = required(int, positive)
    num_hidden_layers: int = required(int, positive)
    num_attention_heads: int = required(int, positive)
    num_key_value_heads: int = required(int, positive)
    rms_norm_eps: float = required(float, finite_positive)
    rope_theta: float = required(float, finite_positive)
    max_position_embeddings: int = required(int, positive)
    hidden_act: str = required(str)
    model_type: str = optional(str, "qwen2")
    head_dim: Optional[int] = optional(int, None, positive)
    tie_word_embeddings: bool = optional(bool, False)
    eos_token_id: Any = optional("any", None)
    bos_token_id: Any = optional("any", None)
    use_sliding_window: bool = optional(bool, False)
    sliding_window: Optional[int] = optional(int, None)
    max_window_layers: Optional[int] = optional(int, None)
    rope_scaling: Any = optional("any", None)

    def validate(self) -> None:
        if self.model_type != "qwen2":
            raise ConfigError(f"config key 'model_type' must be 'qwen2', got {self.model_type!r}")
        if self.hidden_act != "silu":
            raise ConfigError(f"config key 'hidden_act' must be 'silu', got {self.hidden_act!r}")
        if self.rope_scaling is not None:
            raise ConfigError("config key 'rope_scaling' must be null: scaled rotary angles are not built")
        if self.head_dim is None:
            if self.hidden_size % self.num_attention_heads:
                raise ConfigError("'hidden_size' is not a multiple of 'num_attention_heads' and no 'head_dim' is given")
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.head_dim % 16 or self.head_dim > 256:
            raise ConfigError(f"'head_dim' must be a multiple of 16 up to 256, got {self.head_dim}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("'num_attention_heads' must be a multiple of 'num_key_value_heads'")
        if self.use_sliding_window:
            if not self.sliding_window or self.sliding_window <= 0:
                raise ConfigError("'use_sliding_window' is true but 'sliding_window' is not a positive integer")
            if self.max_window_layers is None:
                raise ConfigError("'use_sliding_window' is true but 'max_window_layers' is absent")
        eos = self.eos_token_id
        if eos is not None and not isinstance(eos, int) and not (
                isinstance(eos, list) and all(isinstance(e, int) for e in eos)):
            raise ConfigError("'eos_token_id' must be an integer or a list of integers")

    # ------------------------------------------------------------------------------------
    def eos_ids(self) -> tuple[int, ...]:
        if self.eos_token_id is None:
            return ()
        if isinstance(self.eos_token_id, int):
            return (self.eos_token_id,)
        return tuple(self.eos_token_id)

    def layer_window(self, index: int) -> int:
        """0 for a layer that sees every key, else the number of keys it sees."""
        if self.use_sliding_window and index >= self.max_window_layers:
            return int(self.sliding_window)
        return 0


def qwen2_blueprint(cfg: Qwen2Config) -> ModelBlueprint:
    """Layers of Qwen2 as data: every constant comes from `cfg`."""
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        rope = PartSpec("rope", {"theta": cfg.rope_theta, "rotary_dim": cfg.head_dim})
        mixer = PartSpec("gqa_attention", {
            "hidden": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
            "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "qkv_bias": True, "out_bias": False, "window": cfg.layer_window(i),
            "position": rope,
        }, prefix=p + "self_attn.")
        ffn = PartSpec("gated_mlp", {
            "hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size, "act": cfg.hidden_act,
        }, prefix=p + "mlp.")
        norms = (
            PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix=p + "input_layernorm."),
            PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                     prefix=p + "post_attention_layernorm."),
        )
        layers.append(LayerSpec("prenorm", mixer, ffn, norms, hidden=cfg.hidden_size))
    order = tuple(LayerCall(layer=i, cache=i) for i in range(cfg.num_hidden_layers))
    return ModelBlueprint(
        hidden=cfg.hidden_size,
        vocab=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size},
                           prefix="model.embed_tokens."),
        layers=tuple(layers),
        order=order,
        final_norm=PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix="model.norm."),
        head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size,
                                      "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None},
                      prefix="lm_head."),
        max_positions=cfg.max_position_embeddings,
        eos_token_ids=cfg.eos_ids(),
    )
