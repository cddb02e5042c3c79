"""Typed configuration of the Qwen3 dense decoder, read from its own config.json keys.

Keys and defaults follow the reference's reading of a Hugging Face folder
(src/convert/hf.zig:229-313) and its engine-side checks (src/engine/config.zig:227-315):
`num_key_value_heads` defaults to the head count, `head_dim` to hidden/heads,
`rms_norm_eps` to 1e-6, `rope_theta` to 10000, `max_position_embeddings` to 4096,
`partial_rotary_factor` to 1, `tie_word_embeddings` to false; `hidden_act` must be
silu, `mlp_bias`/`attention_bias` must be off.  `rope_scaling` may be absent or of type
default, linear, llama3 or yarn with the parameters the reference's engine reads
(src/engine/config.zig:42-62,163-223: factor at least 1, the original context length
defaulting to `max_position_embeddings`, llama3's low/high frequency factors, yarn's beta_fast,
beta_slow and attention factor); any other type is refused, since wrong positions give
plausible but worse output.

One step beyond the reference: it refuses a sliding window in use
(src/convert/hf.zig:256-262, src/engine/config.zig:271-279); here `use_sliding_window`
with `sliding_window` and `layer_types` (or `max_window_layers`) selects, layer by
layer, the windowed or the full attention mixer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .base import (ConfigError, ModelConfig, need_int, opt_bool, opt_float, opt_int)

FULL = "full_attention"
SLIDING = "sliding_attention"


@dataclass
class Qwen3Config(ModelConfig):
    hidden_size: int = 0
    num_hidden_layers: int = 0
    intermediate_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    vocab_size: int = 0
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 1.0
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    layer_types: List[str] = field(default_factory=list)
    eos_token_ids: List[int] = field(default_factory=list)
    initializer_range: float = 0.02
    rope_scaling: Optional[dict] = None      # kind, factor, orig_ctx, ... as `parts.RopeScaling` takes them

    # -- derived sizes -----------------------------------------------------------------
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    def layer_window(self, layer: int) -> Optional[int]:
        if self.layer_types and self.layer_types[layer] == SLIDING:
            return self.sliding_window
        return None

    # -- reading -----------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        arch = "Qwen3ForCausalLM"
        act = raw.get("hidden_act")
        if act is not None and act != "silu":
            raise ConfigError(f"config.json 'hidden_act' = {act!r} is not supported (only 'silu')")
        if opt_bool(raw, "mlp_bias", False):
            raise ConfigError("config.json 'mlp_bias' = true is not supported")
        if opt_bool(raw, "attention_bias", False):
            raise ConfigError("config.json 'attention_bias' = true is not supported for Qwen3")
        rs = raw.get("rope_scaling")
        scaling = None
        if isinstance(rs, dict):
            kind = rs.get("rope_type", rs.get("type"))
            if kind is None and rs.get("factor") is not None:
                kind = "linear"           # a factor without a type has always meant linear (src/engine/config.zig:183-186)
            if kind not in (None, "default", "none", "linear", "llama3", "yarn"):
                raise ConfigError(f"config.json 'rope_scaling' of type {kind!r} is not supported "
                                  "(supported: default, linear, llama3, yarn)")
            if kind in ("linear", "llama3", "yarn"):
                if rs.get("factor") is None:
                    raise ConfigError(f"config.json 'rope_scaling' of type '{kind}' needs a 'factor'")
                scaling = {"kind": kind, "factor": float(rs["factor"])}
                for src, dst, conv in (("original_max_position_embeddings", "orig_ctx", int), ("low_freq_factor", "low_freq_factor", float),
                                       ("high_freq_factor", "high_freq_factor", float), ("beta_fast", "beta_fast", float),
                                       ("beta_slow", "beta_slow", float), ("attention_factor", "attn_factor", float)):
                    if rs.get(src) is not None:
                        scaling[dst] = conv(rs[src])
        elif rs is not None:
            raise ConfigError(f"config.json 'rope_scaling' = {rs!r} is not an object")

        hidden = need_int(raw, "hidden_size")
        layers = need_int(raw, "num_hidden_layers")
        ffn = need_int(raw, "intermediate_size")
        heads = need_int(raw, "num_attention_heads")
        kv_heads = opt_int(raw, "num_key_value_heads", heads)
        if heads % kv_heads != 0:
            raise ConfigError(
                f"config.json 'num_attention_heads' = {heads} is not a multiple of 'num_key_value_heads' = {kv_heads}")
        if raw.get("head_dim") is None and hidden % heads != 0:
            raise ConfigError(
                f"config.json 'hidden_size' = {hidden} is not divisible by 'num_attention_heads' = {heads} and no 'head_dim' is given")
        head_dim = opt_int(raw, "head_dim", hidden // heads)
        if head_dim > 256 or head_dim % 2 != 0:
            raise ConfigError(f"config.json 'head_dim' = {head_dim} is not supported (an even number up to 256)")
        prf = opt_float(raw, "partial_rotary_factor", 1.0)
        rot = int(head_dim * prf)
        if not 0 < prf <= 1.0 or rot % 2 != 0 or rot < 2:
            raise ConfigError(
                f"config.json 'partial_rotary_factor' = {prf} gives a rotary width of {rot} for 'head_dim' = {head_dim}; it must be even and in (0, head_dim]")
        vocab = need_int(raw, "vocab_size")
        eps = opt_float(raw, "rms_norm_eps", 1e-6)
        if not eps > 0:
            raise ConfigError(f"config.json 'rms_norm_eps' = {eps} must be positive")
        theta = opt_float(raw, "rope_theta", 10000.0)
        if not theta > 0:
            raise ConfigError(f"config.json 'rope_theta' = {theta} must be positive")

        use_window = opt_bool(raw, "use_sliding_window", False)
        window = opt_int(raw, "sliding_window", None)
        layer_types: List[str] = []
        if use_window and window:
            lt = raw.get("layer_types")
            if lt is None:
                first = opt_int(raw, "max_window_layers", layers, minimum=0)
                lt = [SLIDING if i >= first else FULL for i in range(layers)]
            if not isinstance(lt, list) or len(lt) != layers:
                raise ConfigError(f"config.json 'layer_types' must list {layers} entries, one per layer")
            for t in lt:
                if t not in (FULL, SLIDING):
                    raise ConfigError(f"config.json 'layer_types' entry {t!r} is neither '{FULL}' nor '{SLIDING}'")
            layer_types = list(lt)
        else:
            window = None
            use_window = False

        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: List[int] = []
        elif isinstance(eos, list):
            eos_ids = [int(e) for e in eos]
        else:
            eos_ids = [int(eos)]

        max_pos = opt_int(raw, "max_position_embeddings", 4096)
        if scaling is not None:
            scaling.setdefault("orig_ctx", max_pos)
            from ..parts.position import RopeScaling
            try:
                RopeScaling(**scaling)
            except ValueError as e:
                raise ConfigError(f"config.json 'rope_scaling' = {rs!r}: {e}") from None

        return cls(
            rope_scaling=scaling,
            architecture=arch, hidden_size=hidden, num_hidden_layers=layers, intermediate_size=ffn,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, vocab_size=vocab,
            max_position_embeddings=max_pos,
            rms_norm_eps=eps, rope_theta=theta, partial_rotary_factor=prf,
            tie_word_embeddings=opt_bool(raw, "tie_word_embeddings", False),
            use_sliding_window=use_window, sliding_window=window, layer_types=layer_types,
            eos_token_ids=eos_ids, initializer_range=opt_float(raw, "initializer_range", 0.02),
        )

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "partial_rotary_factor": self.partial_rotary_factor,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "initializer_range": self.initializer_range,
        }
        if self.rope_scaling:
            r = self.rope_scaling
            names = {"orig_ctx": "original_max_position_embeddings", "attn_factor": "attention_factor"}
            d["rope_scaling"] = {"rope_type": r["kind"], **{names.get(k, k): v for k, v in r.items() if k != "kind"}}
        if self.layer_types:
            d["layer_types"] = list(self.layer_types)
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d
