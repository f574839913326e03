"""Typed configuration of the ``LlamaForCausalLM`` architecture.

Every number comes from the model folder's ``config.json``; no size lives in
code.  Keys and defaults follow the reference's ``Llama31Config``
(crates/runner/src/llama31_engine.rs:44-76) with three deliberate differences:

* ``rope_scaling`` is optional (the reference requires it, line 69, so a
  config without scaling cannot even be parsed there); absent or ``null``
  means unscaled rotary frequencies.  ``rope_type`` must be ``"llama3"`` or
  ``"default"``.
* ``num_key_value_heads`` defaults to ``num_attention_heads`` and
  ``rope_theta`` to 10000.
* ``tie_word_embeddings`` is honoured as written; the reference decides tying
  by whether ``lm_head.weight`` exists (llama31_engine.rs:184-192).

Keys the reference never reads (``hidden_act``, ``attention_bias``,
``mlp_bias``) are checked so that a model this engine would compute wrongly is
refused instead of run.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import (BlockSpec, ConfigError, ModelSpec, PartSpec,
                   default_schedule)

ARCHITECTURE = "LlamaForCausalLM"


@dataclass(frozen=True)
class RopeScaling:
    """The ``rope_scaling`` block (llama31_engine.rs:44-50)."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> Optional["RopeScaling"]:
        rope_type = d.get("rope_type", d.get("type", "llama3"))
        if rope_type == "default":
            return None
        if rope_type != "llama3":
            raise ConfigError(f"rope_scaling.rope_type {rope_type!r} is not supported "
                              "(known: 'llama3', 'default')")
        missing = [k for k in ("factor", "low_freq_factor", "high_freq_factor",
                               "original_max_position_embeddings") if k not in d]
        if missing:
            raise ConfigError(f"rope_scaling is missing {missing}")
        rs = RopeScaling(
            rope_type="llama3",
            factor=float(d["factor"]),
            low_freq_factor=float(d["low_freq_factor"]),
            high_freq_factor=float(d["high_freq_factor"]),
            original_max_position_embeddings=int(d["original_max_position_embeddings"]),
        )
        if rs.factor <= 0 or rs.high_freq_factor == rs.low_freq_factor:
            raise ConfigError("rope_scaling needs factor > 0 and "
                              "high_freq_factor != low_freq_factor")
        return rs

    def to_dict(self) -> Dict[str, Any]:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "max_position_embeddings", "rms_norm_eps")


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    eos_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    torch_dtype: str = "bfloat16"
    architectures: List[str] = field(default_factory=lambda: [ARCHITECTURE])
    model_type: str = "llama"

    # ---- reading -----------------------------------------------------
    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "LlamaConfig":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json is missing required keys: {missing}")
        nq = int(d["num_attention_heads"])
        hidden = int(d["hidden_size"])
        if nq <= 0:
            raise ConfigError("num_attention_heads must be positive")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % nq:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {nq} and head_dim is not given")
            head_dim = hidden // nq
        nkv = d.get("num_key_value_heads")
        nkv = nq if nkv is None else int(nkv)
        scaling = d.get("rope_scaling")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: List[int] = []
        elif isinstance(eos, int):
            eos_ids = [eos]
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = list(eos)          # int or list, as qwen35/src/config.rs:135-146
        else:
            raise ConfigError(f"eos_token_id must be an int or a list of ints, got {eos!r}")
        cfg = LlamaConfig(
            vocab_size=int(d["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(d["intermediate_size"]),
            num_hidden_layers=int(d["num_hidden_layers"]),
            num_attention_heads=nq,
            num_key_value_heads=nkv,
            head_dim=int(head_dim),
            max_position_embeddings=int(d["max_position_embeddings"]),
            rms_norm_eps=float(d["rms_norm_eps"]),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(scaling) if scaling else None,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids,
            bos_token_id=d.get("bos_token_id"),
            hidden_act=str(d.get("hidden_act", "silu")),
            attention_bias=bool(d.get("attention_bias", False)),
            mlp_bias=bool(d.get("mlp_bias", False)),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            architectures=list(d.get("architectures", [ARCHITECTURE])),
            model_type=str(d.get("model_type", "llama")),
        )
        cfg.validate()
        return cfg

    @staticmethod
    def from_json_file(path: str) -> "LlamaConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return LlamaConfig.from_dict(json.load(f))

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim",
                     "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if self.attention_bias or self.mlp_bias:
            raise ConfigError("attention_bias / mlp_bias = true is not supported")
        for e in self.eos_token_ids:
            if not 0 <= e < self.vocab_size:
                raise ConfigError(f"eos_token_id {e} is outside the vocabulary")

    # ---- writing -----------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "torch_dtype": self.torch_dtype,
        }
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    # ---- derived -----------------------------------------------------
    def kv_bytes_per_token(self, dtype_bytes: int) -> int:
        """K and V of every layer for one token (qwen35/src/config.rs:169-172)."""
        return (self.num_hidden_layers * 2 * self.num_key_value_heads
                * self.head_dim * dtype_bytes)

    def parameter_count(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        q = self.num_attention_heads * self.head_dim
        kv = self.num_key_value_heads * self.head_dim
        per_layer = h * q + 2 * h * kv + q * h + 3 * h * i + 2 * h
        head = 0 if self.tie_word_embeddings else self.vocab_size * h
        return self.vocab_size * h + self.num_hidden_layers * per_layer + h + head

    # ---- the architecture as parts ----------------------------------
    def build_spec(self) -> ModelSpec:
        """The model as blocks of parts with HF tensor names
        (llama31_engine.rs:170-287: names are used as stored, prefix ``model``)."""
        rope_params: Dict[str, Any] = {
            "head_dim": self.head_dim,
            "rotary_dim": self.head_dim,       # partial factor 1.0 (llama31_engine.rs:99-103)
            "theta": self.rope_theta,
            "max_positions": self.max_position_embeddings,
            "scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
        }
        blocks = []
        for n in range(self.num_hidden_layers):
            p = f"model.layers.{n}"
            blocks.append(BlockSpec(
                kind="pre_norm",
                mixer=PartSpec(
                    kind="attention",
                    params={
                        "hidden_size": self.hidden_size,
                        "num_heads": self.num_attention_heads,
                        "num_kv_heads": self.num_key_value_heads,
                        "head_dim": self.head_dim,
                        # scale 1/sqrt(hd): prefill_engine.rs:2200, decode_engine.rs:8653
                        "scale": self.head_dim ** -0.5,
                        "window": None,
                    },
                    weights={"q": f"{p}.self_attn.q_proj.weight",
                             "k": f"{p}.self_attn.k_proj.weight",
                             "v": f"{p}.self_attn.v_proj.weight",
                             "o": f"{p}.self_attn.o_proj.weight"}),
                feed_forward=PartSpec(
                    kind="swiglu",
                    params={"hidden_size": self.hidden_size,
                            "intermediate_size": self.intermediate_size},
                    weights={"gate": f"{p}.mlp.gate_proj.weight",
                             "up": f"{p}.mlp.up_proj.weight",
                             "down": f"{p}.mlp.down_proj.weight"}),
                mixer_norm=PartSpec(
                    kind="rmsnorm",
                    params={"size": self.hidden_size, "eps": self.rms_norm_eps},
                    weights={"weight": f"{p}.input_layernorm.weight"}),
                feed_forward_norm=PartSpec(
                    kind="rmsnorm",
                    params={"size": self.hidden_size, "eps": self.rms_norm_eps},
                    weights={"weight": f"{p}.post_attention_layernorm.weight"}),
                position=PartSpec(kind="rotary", params=dict(rope_params)),
            ))
        head_weight = ("model.embed_tokens.weight" if self.tie_word_embeddings
                       else "lm_head.weight")
        spec = ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec(kind="embedding",
                               params={"vocab_size": self.vocab_size,
                                       "hidden_size": self.hidden_size},
                               weights={"weight": "model.embed_tokens.weight"}),
            blocks=blocks,
            schedule=default_schedule(self.num_hidden_layers),
            final_norm=PartSpec(kind="rmsnorm",
                                params={"size": self.hidden_size, "eps": self.rms_norm_eps},
                                weights={"weight": "model.norm.weight"}),
            head=PartSpec(kind="linear_head",
                          params={"vocab_size": self.vocab_size,
                                  "hidden_size": self.hidden_size},
                          weights={"weight": head_weight}),
            stop_token_ids=list(self.eos_token_ids),
        )
        spec.validate()
        return spec

    def tensor_shapes(self) -> Dict[str, List[int]]:
        """Every tensor the model folder must hold, with its shape ([out, in])."""
        h, i = self.hidden_size, self.intermediate_size
        q = self.num_attention_heads * self.head_dim
        kv = self.num_key_value_heads * self.head_dim
        shapes: Dict[str, List[int]] = {"model.embed_tokens.weight": [self.vocab_size, h],
                                        "model.norm.weight": [h]}
        if not self.tie_word_embeddings:
            shapes["lm_head.weight"] = [self.vocab_size, h]
        for n in range(self.num_hidden_layers):
            p = f"model.layers.{n}"
            shapes[f"{p}.input_layernorm.weight"] = [h]
            shapes[f"{p}.post_attention_layernorm.weight"] = [h]
            shapes[f"{p}.self_attn.q_proj.weight"] = [q, h]
            shapes[f"{p}.self_attn.k_proj.weight"] = [kv, h]
            shapes[f"{p}.self_attn.v_proj.weight"] = [kv, h]
            shapes[f"{p}.self_attn.o_proj.weight"] = [h, q]
            shapes[f"{p}.mlp.gate_proj.weight"] = [i, h]
            shapes[f"{p}.mlp.up_proj.weight"] = [i, h]
            shapes[f"{p}.mlp.down_proj.weight"] = [h, i]
        return shapes

    def ignorable_tensor(self, name: str) -> bool:
        """Stored tensors that are no parameters: the rotary frequency buffer some exporters write
        per layer (this engine computes the frequencies from the configuration)."""
        return name.endswith("rotary_emb.inv_freq")

    def is_norm_tensor(self, name: str) -> bool:
        return name.endswith("norm.weight") or name.endswith("layernorm.weight")
