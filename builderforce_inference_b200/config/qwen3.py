"""``Qwen3Config``: the hyper-parameters of a Qwen3 dense decoder, read from config.json.

The reference reads the same quantities from GGUF metadata
(crates/bfi-models/src/qwen3.rs:26-38, 328-370); here each comes from the key a Qwen3 model
folder uses for it.  Options the reference's model does not have (bias, rope scaling, experts,
another activation, partial rotary) are refused by name, as the reference refuses experts
(qwen3.rs:87-96).  A sliding window, which the config.json keys can describe, selects the
windowed form of the attention part layer by layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ConfigReader


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    # One entry per layer: the number of most recent keys a layer attends to, or None for all.
    layer_windows: Tuple[Optional[int], ...]
    eos_token_ids: Tuple[int, ...]
    torch_dtype: str

    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_dict(cls, data: Dict[str, Any], what: str = "config.json") -> "Qwen3Config":
        r = ConfigReader(data, what)
        n_layer = r.integer("num_hidden_layers", minimum=1)
        hidden = r.integer("hidden_size", minimum=1)
        inter = r.integer("intermediate_size", minimum=1)
        vocab = r.integer("vocab_size", minimum=1)
        n_ctx = r.integer("max_position_embeddings", minimum=1)
        n_head = r.integer("num_attention_heads", minimum=1)
        # kv heads default to the q heads and must divide them (qwen3.rs:334-342)
        n_kv = r.integer("num_key_value_heads", default=n_head, minimum=1)
        if n_head % n_kv != 0:
            raise ConfigError(
                f"{what}: GQA: num_attention_heads {n_head} % num_key_value_heads {n_kv} != 0")
        # head_dim is its own key, not hidden/heads (qwen3.rs:343-348)
        if r.has("head_dim"):
            head_dim = r.integer("head_dim", minimum=1)
        else:
            if hidden % n_head != 0:
                raise ConfigError(
                    f"{what}: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {n_head}")
            head_dim = hidden // n_head
        if head_dim % 2 != 0:
            raise ConfigError(f"{what}: key 'head_dim' must be even for rotary pairs, got {head_dim}")
        eps = r.number("rms_norm_eps", default=1e-6, positive=True)
        theta = r.number("rope_theta", default=1_000_000.0, positive=True)
        tied = r.boolean("tie_word_embeddings", default=False)

        # ---- options the reference's qwen3 does not have: refused by name
        n_exp = r.integer("num_experts", default=0)
        n_exp = n_exp or r.integer("num_local_experts", default=0)
        if n_exp:
            raise ConfigError(
                f"{what}: qwen3moe (num_experts={n_exp}) is not implemented; dense qwen3 only")
        if r.boolean("attention_bias", default=False):
            raise ConfigError(f"{what}: 'attention_bias': true is not supported (qwen3 has no bias)")
        if r.boolean("mlp_bias", default=False):
            raise ConfigError(f"{what}: 'mlp_bias': true is not supported (qwen3 has no bias)")
        if r.raw("rope_scaling") is not None:
            raise ConfigError(f"{what}: 'rope_scaling' is not supported (must be null)")
        act = r.string("hidden_act", default="silu")
        if act != "silu":
            raise ConfigError(f"{what}: 'hidden_act' must be \"silu\", got {act!r}")
        prf = r.number("partial_rotary_factor", default=1.0)
        if prf != 1.0:
            raise ConfigError(f"{what}: 'partial_rotary_factor' must be 1, got {prf}")
        if r.number("attention_dropout", default=0.0) != 0.0:
            pass  # inference: dropout is never applied

        # ---- sliding window: per layer, None = all keys
        windows: Tuple[Optional[int], ...] = (None,) * n_layer
        use_window = r.boolean("use_sliding_window", default=False)
        window = r.integer("sliding_window", default=None, minimum=1)
        kinds = r.string_list("layer_types", default=None)
        first_windowed = r.integer("max_window_layers", default=n_layer, minimum=0)
        if kinds is not None:
            if len(kinds) != n_layer:
                raise ConfigError(
                    f"{what}: 'layer_types' has {len(kinds)} entries for {n_layer} layers")
            for k in kinds:
                if k not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"{what}: 'layer_types' entry {k!r} is not a known layer kind")
        if use_window:
            if window is None:
                raise ConfigError(f"{what}: 'use_sliding_window' is true but 'sliding_window' is null")
            if kinds is not None:
                windows = tuple(window if k == "sliding_attention" else None for k in kinds)
            elif not r.has("max_window_layers"):
                # the usual tooling fills this key with a fixed default of its own; guessing one
                # here would silently window other layers than the writer of the file meant
                raise ConfigError(
                    f"{what}: 'use_sliding_window' is true but neither 'layer_types' nor "
                    f"'max_window_layers' says which layers are windowed")
            else:
                windows = tuple(window if i >= first_windowed else None for i in range(n_layer))
        elif kinds is not None and any(k == "sliding_attention" for k in kinds):
            raise ConfigError(
                f"{what}: 'layer_types' names sliding_attention layers but 'use_sliding_window' is false")

        eos = tuple(r.int_or_list("eos_token_id"))
        dtype = r.string("torch_dtype", default=r.string("dtype", default="bfloat16"))
        return cls(
            vocab_size=vocab, hidden_size=hidden, intermediate_size=inter,
            num_hidden_layers=n_layer, num_attention_heads=n_head, num_key_value_heads=n_kv,
            head_dim=head_dim, rms_norm_eps=eps, rope_theta=theta,
            max_position_embeddings=n_ctx, tie_word_embeddings=tied,
            layer_windows=windows, eos_token_ids=eos, torch_dtype=dtype,
        )

    def to_dict(self) -> Dict[str, Any]:
        """A config.json dictionary that reads back to this configuration."""
        d: Dict[str, Any] = {
            "architectures": ["Qwen3ForCausalLM"],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "rope_scaling": None,
            "torch_dtype": self.torch_dtype,
        }
        wins = [w for w in self.layer_windows if w is not None]
        if wins:
            d["use_sliding_window"] = True
            d["sliding_window"] = wins[0]
            d["layer_types"] = ["sliding_attention" if w is not None else "full_attention"
                                for w in self.layer_windows]
        else:
            d["use_sliding_window"] = False
            d["sliding_window"] = None
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 \
                else self.eos_token_ids[0]
        return d
