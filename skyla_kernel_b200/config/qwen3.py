"""Typed configuration of the Qwen3 dense decoder, read from config.json.

The reference reads the same quantities from GGUF metadata
(skyla-ref/src/lib.rs:77-118): layer count, width, head counts, head size
(default ``width / heads``, lib.rs:88-90), feed-forward width, rope base,
optional YaRN scaling (skyla-ref/src/rope.rs:14-31) and the norms' epsilon.
Every size the model code uses comes from here; none stands in code.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import (ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                   optional, require)

ARCHITECTURE = "Qwen3ForCausalLM"


@dataclass(frozen=True)
class RopeScaling:
    """YaRN parameters (skyla-ref/src/rope.rs:7-12)."""

    factor: float
    original_max_position_embeddings: float
    attn_factor: float = 1.0


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rms_norm_eps: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    rope_scaling: Optional[RopeScaling] = None
    eos_token_ids: List[int] = field(default_factory=list)
    torch_dtype: str = "bfloat16"

    architecture = ARCHITECTURE

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        hidden = require(d, "hidden_size", int)
        n_head = require(d, "num_attention_heads", int)
        if n_head <= 0:
            raise ConfigError("config.json: 'num_attention_heads' must be positive")
        n_kv = optional(d, "num_key_value_heads", int, n_head)
        head_dim = optional(d, "head_dim", int, None)
        if head_dim is None:
            if hidden % n_head:
                raise ConfigError(
                    "config.json: 'head_dim' is absent and 'hidden_size' "
                    f"({hidden}) is not a multiple of 'num_attention_heads' ({n_head})")
            head_dim = hidden // n_head
        act = optional(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' must be 'silu' (got {act!r})")
        if optional(d, "attention_bias", bool, False):
            raise ConfigError("config.json: 'attention_bias' must be false: "
                              "the architecture has no bias tensors")
        if optional(d, "use_sliding_window", bool, False):
            raise ConfigError("config.json: 'use_sliding_window' must be false: "
                              "the architecture attends to every earlier position")
        scaling = cls._rope_scaling(d.get("rope_scaling"))
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: List[int] = []
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = [eos]
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = list(eos)
        else:
            raise ConfigError(f"config.json: 'eos_token_id' is not an integer or a list of them (got {eos!r})")
        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=require(d, "num_hidden_layers", int),
            num_attention_heads=n_head,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            intermediate_size=require(d, "intermediate_size", int),
            vocab_size=require(d, "vocab_size", int),
            rope_theta=require(d, "rope_theta", float),
            rms_norm_eps=require(d, "rms_norm_eps", float),
            max_position_embeddings=require(d, "max_position_embeddings", int),
            tie_word_embeddings=optional(d, "tie_word_embeddings", bool, False),
            rope_scaling=scaling,
            eos_token_ids=eos_ids,
            torch_dtype=optional(d, "torch_dtype", str, optional(d, "dtype", str, "bfloat16")),
        )
        cfg.validate()
        return cfg

    @staticmethod
    def _rope_scaling(rs) -> Optional[RopeScaling]:
        if rs is None:
            return None
        if not isinstance(rs, dict):
            raise ConfigError("config.json: 'rope_scaling' is not an object")
        kind = rs.get("rope_type", rs.get("type"))
        if kind in (None, "none", "default"):
            return None
        if kind != "yarn":
            # skyla-ref/src/rope.rs:29: other scaling types are an error
            raise ConfigError(f"config.json: unsupported rope scaling {kind!r} (none or 'yarn')")
        return RopeScaling(
            factor=require(rs, "factor", float, "config.json rope_scaling"),
            original_max_position_embeddings=require(
                rs, "original_max_position_embeddings", float, "config.json rope_scaling"),
            attn_factor=optional(rs, "attn_factor", float, 1.0, "config.json rope_scaling"),
        )

    @classmethod
    def from_folder(cls, folder: str) -> "Qwen3Config":
        with open(os.path.join(folder, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def validate(self) -> None:
        pos = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
               "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings")
        for k in pos:
            if getattr(self, k) <= 0:
                raise ConfigError(f"config.json: '{k}' must be positive (got {getattr(self, k)})")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: 'num_attention_heads' ({self.num_attention_heads}) is not a multiple "
                f"of 'num_key_value_heads' ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: 'head_dim' ({self.head_dim}) must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError("config.json: 'rms_norm_eps' must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("config.json: 'rope_theta' must be positive")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "use_sliding_window": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.rope_scaling is not None:
            d["rope_scaling"] = {
                "rope_type": "yarn",
                "factor": self.rope_scaling.factor,
                "original_max_position_embeddings": self.rope_scaling.original_max_position_embeddings,
                "attn_factor": self.rope_scaling.attn_factor,
            }
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d

    # ------------------------------------------------------------- description
    def to_spec(self) -> ModelSpec:
        """The architecture as data: which parts, with which constants, in which order.

        Block arrangement and tensor roles follow skyla-ref/src/model.rs:29-50,97-122.
        """
        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"width": self.hidden_size, "eps": self.rms_norm_eps},
                            {"weight": name})

        rope = PartSpec("rotary_neox", {
            "n_rot": self.head_dim,  # skyla-ref/src/lib.rs:92-95: whole head when no count is given
            "theta": self.rope_theta,
            "max_positions": self.max_position_embeddings,
            "scaling": None if self.rope_scaling is None else {
                "factor": self.rope_scaling.factor,
                "original_max_position_embeddings": self.rope_scaling.original_max_position_embeddings,
                "attn_factor": self.rope_scaling.attn_factor,
            },
        })
        attn_params = {
            "hidden_size": self.hidden_size,
            "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "qk_norm": True,
            "qk_norm_eps": self.rms_norm_eps,
            "scale": None,  # 1/sqrt(head_dim), skyla-ref/src/model.rs:150
            "window": None,
            "position": rope,
        }
        ffn_params = {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size}
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}"
            mixer = PartSpec("gqa_attention", attn_params, {
                "q_proj": f"{p}.self_attn.q_proj.weight",
                "k_proj": f"{p}.self_attn.k_proj.weight",
                "v_proj": f"{p}.self_attn.v_proj.weight",
                "o_proj": f"{p}.self_attn.o_proj.weight",
                "q_norm": f"{p}.self_attn.q_norm.weight",
                "k_norm": f"{p}.self_attn.k_norm.weight",
            })
            ffn = PartSpec("swiglu", ffn_params, {
                "gate_proj": f"{p}.mlp.gate_proj.weight",
                "up_proj": f"{p}.mlp.up_proj.weight",
                "down_proj": f"{p}.mlp.down_proj.weight",
            })
            layers.append(LayerSpec(prefix=p, block="prenorm_residual", parts={
                "mixer_norm": norm(f"{p}.input_layernorm.weight"), "mixer": mixer,
                "ffn_norm": norm(f"{p}.post_attention_layernorm.weight"), "feed_forward": ffn}))
        schedule = [ScheduleEntry(layer=i) for i in range(self.num_hidden_layers)]
        return ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size,
                                                   "hidden_size": self.hidden_size},
                               {"weight": "model.embed_tokens.weight"}),
            layers=layers,
            schedule=schedule,
            final_norm=norm("model.norm.weight"),
            # skyla-ref/src/model.rs:70-73: without an output matrix the embedding is the head
            head=PartSpec("linear_head", {"vocab_size": self.vocab_size,
                                          "hidden_size": self.hidden_size},
                          {"weight": "model.embed_tokens.weight" if self.tie_word_embeddings
                           else "lm_head.weight"}),
            stop_token_ids=list(self.eos_token_ids),
            # a tied checkpoint may still store a copy of the output matrix
            optional_tensors=["lm_head.weight"] if self.tie_word_embeddings else [],
        )
