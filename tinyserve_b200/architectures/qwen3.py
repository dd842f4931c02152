"""The dense Qwen3 decoder (``Qwen3ForCausalLM``): its typed configuration and how its
``config.json`` keys become a ``ModelSpec`` of generic parts.

Which keys are read, their defaults and what is rejected follow the upstream engine
(src/tinyserve/config.py:41-79): required ``vocab_size, hidden_size, intermediate_size,
num_hidden_layers, num_attention_heads, num_key_value_heads, rms_norm_eps,
max_position_embeddings`` and a rope theta (top level or ``rope_parameters.rope_theta``);
``head_dim`` defaults to ``hidden_size // num_attention_heads``; ``tie_word_embeddings``
defaults to False; ``hidden_act`` must be "silu", ``attention_bias`` false, ``rope_scaling``
null and the rope type "default". Upstream ignores the sliding-window keys; here
``use_sliding_window=true`` is refused, because honouring it silently would change results.

What the architecture fixes in code rather than in ``config.json`` (upstream
src/tinyserve/model.py:137-214) is passed to the parts as arguments by ``to_spec``: the
attention scale ``head_dim ** -0.5``, per-head q/k RMSNorm with the model's eps, rotate-half
RoPE over the whole head, causal masking, no biases, plain-weight RMSNorm.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.base import (
    LayerCall,
    LayerSpec,
    ModelConfig,
    ModelSpec,
    PartSpec,
    UnsupportedConfigError,
)
from ..config.registry import register_architecture

ARCHITECTURE = "Qwen3ForCausalLM"


def _required(d: Mapping[str, Any], key: str) -> Any:
    if key not in d or d[key] is None:
        raise UnsupportedConfigError(f"config.json has no {key!r}")
    return d[key]


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False

    architecture = ARCHITECTURE

    def __post_init__(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_layers",
                     "num_heads", "num_kv_heads", "head_dim", "max_position_embeddings"):
            if int(getattr(self, name)) <= 0:
                raise UnsupportedConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_heads % self.num_kv_heads != 0:
            raise UnsupportedConfigError(
                f"num_attention_heads={self.num_heads} is not a multiple of "
                f"num_key_value_heads={self.num_kv_heads}"
            )
        if self.head_dim % 2 != 0:
            raise UnsupportedConfigError(f"head_dim={self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise UnsupportedConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise UnsupportedConfigError(f"rope_theta must be positive, got {self.rope_theta}")

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        if ARCHITECTURE not in (d.get("architectures") or []):
            raise UnsupportedConfigError(f"expected {ARCHITECTURE}, got {d.get('architectures')}")
        if d.get("hidden_act", "silu") != "silu":
            raise UnsupportedConfigError(f"hidden_act={d['hidden_act']!r}: only 'silu' is implemented")
        if d.get("attention_bias", False):
            raise UnsupportedConfigError("attention_bias=true is not implemented")
        if d.get("rope_scaling") is not None:
            raise UnsupportedConfigError(f"rope_scaling={d['rope_scaling']!r} is not implemented")
        rope = d.get("rope_parameters") or {}
        if rope.get("rope_type", "default") != "default":
            raise UnsupportedConfigError(f"rope_parameters={dict(rope)!r} is not implemented")
        if d.get("use_sliding_window", False):
            raise UnsupportedConfigError("use_sliding_window=true is not implemented for Qwen3")
        theta = d.get("rope_theta") or rope.get("rope_theta")
        if theta is None:
            raise UnsupportedConfigError("config.json has no rope_theta")
        hidden = int(_required(d, "hidden_size"))
        heads = int(_required(d, "num_attention_heads"))
        head_dim = d.get("head_dim")
        return cls(
            vocab_size=int(_required(d, "vocab_size")),
            hidden_size=hidden,
            intermediate_size=int(_required(d, "intermediate_size")),
            num_layers=int(_required(d, "num_hidden_layers")),
            num_heads=heads,
            num_kv_heads=int(_required(d, "num_key_value_heads")),
            head_dim=int(head_dim) if head_dim is not None else hidden // heads,
            rms_norm_eps=float(_required(d, "rms_norm_eps")),
            rope_theta=float(theta),
            max_position_embeddings=int(_required(d, "max_position_embeddings")),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
        )

    def to_dict(self) -> dict[str, Any]:
        return {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "attention_bias": False,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": False,
        }

    def to_spec(self) -> ModelSpec:
        h, d = self.hidden_size, self.head_dim
        rope = PartSpec("rope", {"head_dim": d, "rotary_dim": d, "theta": self.rope_theta,
                                 "pairing": "half"})
        layers = []
        for i in range(self.num_layers):
            layers.append(LayerSpec(
                prefix=f"model.layers.{i}.",
                block="prenorm",
                parts={"mixer": PartSpec("gqa_attention", {
                    "prefix": "self_attn.", "hidden_size": h, "num_heads": self.num_heads,
                    "num_kv_heads": self.num_kv_heads, "head_dim": d, "scale": d ** -0.5,
                    "qk_norm": True, "qk_norm_eps": self.rms_norm_eps, "window": None,
                }),
                "feed_forward": PartSpec("swiglu", {
                    "prefix": "mlp.", "hidden_size": h,
                    "intermediate_size": self.intermediate_size,
                }),
                "mixer_norm": PartSpec("rms_norm", {
                    "name": "input_layernorm.weight", "size": h, "eps": self.rms_norm_eps}),
                "feed_forward_norm": PartSpec("rms_norm", {
                    "name": "post_attention_layernorm.weight", "size": h,
                    "eps": self.rms_norm_eps})},
                position=rope,
            ))
        return ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab_size,
            hidden_size=h,
            layers=tuple(layers),
            order=tuple(LayerCall(i) for i in range(self.num_layers)),
            embedding=PartSpec("token_embedding", {
                "name": "model.embed_tokens.weight", "vocab_size": self.vocab_size,
                "hidden_size": h}),
            final_norm=PartSpec("rms_norm", {
                "name": "model.norm.weight", "size": h, "eps": self.rms_norm_eps}),
            head=PartSpec("lm_head", {
                "name": "model.embed_tokens.weight" if self.tie_word_embeddings else "lm_head.weight",
                "tied": self.tie_word_embeddings, "ignored_when_tied": "lm_head.weight",
                "vocab_size": self.vocab_size, "hidden_size": h}),
            max_position_embeddings=self.max_position_embeddings,
        )


register_architecture(ARCHITECTURE, Qwen3Config)
