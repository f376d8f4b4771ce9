"""Typed configuration of the Llama-style dense GQA decoder, read from ``config.json``.

The architecture is the ``TransformerLM`` of the reference (src/scratch_llm/model.py:439-505):
pre-norm blocks of RMSNorm, grouped-query attention with rotary positions, and a SwiGLU
feed-forward, without biases.  The reference keeps these sizes in a ``ModelConfig`` dataclass
(src/scratch_llm/model.py:56-114) and has no ``config.json``; the keys here are the public
checkpoint-format ones, mapped onto the reference's fields as follows:

=========================  ==========================  =======================
config.json key            reference field             default
=========================  ==========================  =======================
hidden_size                d_model                     required
num_hidden_layers          n_layers                    required
num_attention_heads        n_heads                     required
num_key_value_heads        n_kv_heads                  num_attention_heads
head_dim                   d_model // n_heads          hidden_size // heads
intermediate_size          d_ff                        required
vocab_size                 vocab_size                  required
rope_theta                 rope_theta                  10000.0
rms_norm_eps               RMSNorm eps (model.py:153)  1e-5
tie_word_embeddings        tie_embeddings              false
max_position_embeddings    context_length              2048
rope_interleaved           (adjacent pairs, :204-220)  true
torch_dtype                parameter dtype             "bfloat16"
=========================  ==========================  =======================
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Any, Mapping

from .spec import ModelSpec, PartSpec, sequential_order, standard_layer

_UNSUPPORTED_TRUE = ("attention_bias", "mlp_bias")


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int
    vocab_size: int
    num_key_value_heads: int | None = None
    head_dim: int | None = None
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 2048
    rope_interleaved: bool = True
    torch_dtype: str = "bfloat16"

    architecture = "LlamaForCausalLM"

    def __post_init__(self) -> None:
        # the three checks of the reference (src/scratch_llm/model.py:90-99) and the ones that
        # an explicit head_dim and a config file add
        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                     "intermediate_size", "vocab_size", "max_position_embeddings"):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value < 1:
                raise ValueError(f"{name} must be a positive integer, got {value!r}")
        if self.head_dim is None and self.hidden_size % self.num_attention_heads != 0:
            raise ValueError(f"hidden_size={self.hidden_size} not divisible by "
                             f"num_attention_heads={self.num_attention_heads}")
        if self.kv_heads < 1 or self.num_attention_heads % self.kv_heads != 0:
            raise ValueError(f"num_attention_heads={self.num_attention_heads} not divisible by "
                             f"num_key_value_heads={self.kv_heads} (query heads must group "
                             "evenly over kv heads)")
        if self.head_size < 2 or self.head_size % 2 != 0:
            raise ValueError(f"head_dim={self.head_size} must be even for rotary positions")
        if not (self.rms_norm_eps > 0 and math.isfinite(self.rms_norm_eps)):
            raise ValueError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ValueError(f"rope_theta must be positive, got {self.rope_theta!r}")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ValueError(f"torch_dtype must be 'bfloat16' or 'float32', got "
                             f"{self.torch_dtype!r}")

    @property
    def kv_heads(self) -> int:
        return (self.num_attention_heads if self.num_key_value_heads is None
                else self.num_key_value_heads)

    @property
    def head_size(self) -> int:
        return (self.hidden_size // self.num_attention_heads if self.head_dim is None
                else self.head_dim)

    # -- config.json ---------------------------------------------------------------------

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LlamaConfig":
        for key in _UNSUPPORTED_TRUE:
            if raw.get(key):
                raise ValueError(f"config.json sets {key}=true: biases are not part of this "
                                 "architecture and are unsupported")
        if raw.get("rope_scaling") is not None:
            raise ValueError("config.json sets rope_scaling: rescaled rotary frequencies are "
                             "unsupported (the architecture has none, "
                             "src/scratch_llm/model.py:197)")
        if raw.get("sliding_window") is not None:
            raise ValueError("config.json sets sliding_window: this architecture attends to "
                             "all keys")
        required = ("hidden_size", "num_hidden_layers", "num_attention_heads",
                    "intermediate_size", "vocab_size")
        missing = [k for k in required if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in raw.items() if k in known})

    def to_dict(self) -> dict[str, Any]:
        out = asdict(self)
        out["architectures"] = [self.architecture]
        out["num_key_value_heads"] = self.kv_heads
        out["head_dim"] = self.head_size
        return out

    # -- layers as data ------------------------------------------------------------------

    def model_spec(self) -> ModelSpec:
        attention = PartSpec("gqa_attention", {
            "hidden_size": self.hidden_size,
            "n_heads": self.num_attention_heads,
            "n_kv_heads": self.kv_heads,
            "head_dim": self.head_size,
            # divide-after-matmul by sqrt(head_dim), src/scratch_llm/model.py:177
            "scale": 1.0 / math.sqrt(self.head_size),
            "window": None,
        })
        swiglu = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                     "intermediate_size": self.intermediate_size})
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        rotary = PartSpec("rotary", {"head_dim": self.head_size, "theta": self.rope_theta,
                                     "max_position": self.max_position_embeddings,
                                     "interleaved": self.rope_interleaved})
        names = {"mixer": "self_attn", "feed_forward": "mlp",
                 "mixer_norm": "input_layernorm",
                 "feed_forward_norm": "post_attention_layernorm"}
        layers = tuple(
            standard_layer(f"model.layers.{i}", "pre_norm", mixer=attention,
                           feed_forward=swiglu, mixer_norm=norm, feed_forward_norm=norm,
                           position=rotary, names=names)
            for i in range(self.num_hidden_layers))
        return ModelSpec(
            hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            max_position=self.max_position_embeddings, layers=layers,
            order=sequential_order(self.num_hidden_layers), final_norm=norm,
            embed_name="model.embed_tokens.weight", final_norm_name="model.norm",
            lm_head_name="lm_head.weight", tie_embeddings=self.tie_word_embeddings)

    # tensor names of a scratch_llm state_dict (src/scratch_llm/model.py:449-459), accepted as
    # aliases of the checkpoint-format names
    def reference_aliases(self) -> dict[str, str]:
        alias = {"token_emb.weight": "model.embed_tokens.weight",
                 "final_norm.weight": "model.norm.weight",
                 "lm_head.weight": "lm_head.weight"}
        per_layer = {"attn_norm.weight": "input_layernorm.weight",
                     "attn.q_proj.weight": "self_attn.q_proj.weight",
                     "attn.k_proj.weight": "self_attn.k_proj.weight",
                     "attn.v_proj.weight": "self_attn.v_proj.weight",
                     "attn.o_proj.weight": "self_attn.o_proj.weight",
                     "ffn_norm.weight": "post_attention_layernorm.weight",
                     "ffn.w1.weight": "mlp.gate_proj.weight",
                     "ffn.w3.weight": "mlp.up_proj.weight",
                     "ffn.w2.weight": "mlp.down_proj.weight"}
        for i in range(self.num_hidden_layers):
            for ref, ours in per_layer.items():
                alias[f"blocks.{i}.{ref}"] = f"model.layers.{i}.{ours}"
        return alias
