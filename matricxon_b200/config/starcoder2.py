"""StarCoder2 configuration: ``config.json`` keys to a typed record and a model description.

The reference reads the same quantities from GGUF metadata
(app/architectures/starcoder2.py:63-79): embedding length, head counts (KV heads
default to the head count, :67), key length (default ``hidden // heads``, :68),
block count, feed-forward length, LayerNorm epsilon, vocabulary size and the
rope base. It hard-codes a bias on every projection (:22-25) and detects tied
embeddings by a missing output tensor (:37-39, :123); it reads no window. Here
``use_bias``, ``tie_word_embeddings`` and ``sliding_window`` are config.json keys.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any

from matricxon_b200.config.base import ConfigError, ConfigReader
from matricxon_b200.parts.spec import (
    AttentionSpec,
    LayerNormSpec,
    LayerSpec,
    MlpSpec,
    ModelSpec,
    RotarySpec,
    sequential_schedule,
)

_ACTIVATIONS = {"gelu_pytorch_tanh": "gelu_tanh"}


@dataclass(frozen=True)
class Starcoder2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    sliding_window: int | None
    max_position_embeddings: int
    norm_epsilon: float
    use_bias: bool = True
    tie_word_embeddings: bool = True
    hidden_act: str = "gelu_pytorch_tanh"
    torch_dtype: str = "bfloat16"

    model_type = "starcoder2"
    architecture = "Starcoder2ForCausalLM"

    def __post_init__(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 16 != 0 or not 16 <= self.head_dim <= 256:
            raise ConfigError(f"head_dim ({self.head_dim}) must be a multiple of 16 between 16 and 256: "
                              "the attention kernels take no other size")
        if self.hidden_act not in _ACTIVATIONS:
            raise ConfigError(
                f"hidden_act {self.hidden_act!r} is not supported; StarCoder2 uses "
                f"{sorted(_ACTIVATIONS)}")
        if self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError("sliding_window must be positive, or null for plain causal attention")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"torch_dtype {self.torch_dtype!r} is not bfloat16 or float32")

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config.json") -> "Starcoder2Config":
        r = ConfigReader(raw, where)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        window = r.optional_integer("sliding_window", minimum=0)
        return cls(
            hidden_size=hidden,
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            num_attention_heads=heads,
            num_key_value_heads=r.integer("num_key_value_heads", heads, minimum=1),
            head_dim=r.integer("head_dim", hidden // heads, minimum=2),
            intermediate_size=r.integer("intermediate_size", minimum=1),
            vocab_size=r.integer("vocab_size", minimum=1),
            rope_theta=r.number("rope_theta", positive=True),
            sliding_window=window if window else None,
            max_position_embeddings=r.integer("max_position_embeddings", minimum=1),
            norm_epsilon=r.number("norm_epsilon", positive=True),
            use_bias=r.boolean("use_bias", True),
            tie_word_embeddings=r.boolean("tie_word_embeddings", True),
            hidden_act=r.string("hidden_act", "gelu_pytorch_tanh"),
            torch_dtype=_dtype_name(r.string("torch_dtype", "bfloat16")),
        )

    def to_dict(self) -> dict[str, Any]:
        out = asdict(self)
        out["model_type"] = self.model_type
        out["architectures"] = [self.architecture]
        return out

    def model_spec(self) -> ModelSpec:
        """The generic description the parts are built from: L identical pre-norm layers."""
        norm = LayerNormSpec(size=self.hidden_size, eps=self.norm_epsilon, bias=True)
        attention = AttentionSpec(
            hidden_size=self.hidden_size,
            num_heads=self.num_attention_heads,
            num_kv_heads=self.num_key_value_heads,
            head_dim=self.head_dim,
            bias=self.use_bias,
            window=self.sliding_window,
            scale=float(self.head_dim) ** -0.5,
            projection_names=("q_proj", "k_proj", "v_proj"),
            output_name="o_proj",
            position=RotarySpec(rotary_dim=self.head_dim, theta=self.rope_theta),
        )
        mlp = MlpSpec(
            hidden_size=self.hidden_size,
            intermediate_size=self.intermediate_size,
            bias=self.use_bias,
            activation=_ACTIVATIONS[self.hidden_act],
            up_name="c_fc",
            down_name="c_proj",
        )
        layer = LayerSpec(mixer=attention, feed_forward=mlp, mixer_norm=norm, ffn_norm=norm,
                          mixer_name="self_attn", feed_forward_name="mlp",
                          mixer_norm_name="input_layernorm",
                          ffn_norm_name="post_attention_layernorm")
        return ModelSpec(
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            layers=tuple(layer for _ in range(self.num_hidden_layers)),
            schedule=sequential_schedule(self.num_hidden_layers),
            final_norm=norm,
            tie_word_embeddings=self.tie_word_embeddings,
            max_position_embeddings=self.max_position_embeddings,
            embedding_name="model.embed_tokens",
            layer_prefix="model.layers",
            final_norm_name="model.norm",
            head_name="lm_head",
        )


def _dtype_name(name: str) -> str:
    aliases = {"bf16": "bfloat16", "fp32": "float32", "float": "float32",
               "torch.bfloat16": "bfloat16", "torch.float32": "float32"}
    return aliases.get(name, name)
