"""Qwen3 dense as data: its configuration turned into a ``ModelSpec``.

Layer structure and formulas: crates/bfi-models/src/qwen3.rs:190-266.  Tensor names: the
reference reads llama.cpp GGUF names (qwen3.rs:109-144); a model folder stores the same tensors
under the names below (``blk.{i}.attn_q.weight`` <-> ``model.layers.{i}.self_attn.q_proj.weight``
and so on), all ``[out, in]`` row-major, which is the reference's layout after its dim reversal
(crates/bfi-models/src/tutil.rs:73-75).  Rotate-half pairing needs no row permutation.
"""
from __future__ import annotations

from typing import Any, Dict

from ..config.qwen3 import Qwen3Config
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec


def qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    norm = PartSpec("rms", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    position = PartSpec("rotary", {"theta": cfg.rope_theta, "rot_dim": cfg.head_dim})
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = PartSpec("attention", {
            "width": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
            "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "position": position, "qk_norm": True, "eps": cfg.rms_norm_eps,
            "window": cfg.layer_windows[i],
        })
        ffn = PartSpec("gated_mlp", {"width": cfg.hidden_size, "inner": cfg.intermediate_size,
                                     "activation": "silu"})
        block = PartSpec("prenorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "ffn": ffn})
        p = f"model.layers.{i}."
        names = {
            "norm1.weight": p + "input_layernorm.weight",
            "mixer.q_proj": p + "self_attn.q_proj.weight",
            "mixer.k_proj": p + "self_attn.k_proj.weight",
            "mixer.v_proj": p + "self_attn.v_proj.weight",
            "mixer.o_proj": p + "self_attn.o_proj.weight",
            "mixer.q_norm": p + "self_attn.q_norm.weight",
            "mixer.k_norm": p + "self_attn.k_norm.weight",
            "norm2.weight": p + "post_attention_layernorm.weight",
            "ffn.gate_proj": p + "mlp.gate_proj.weight",
            "ffn.up_proj": p + "mlp.up_proj.weight",
            "ffn.down_proj": p + "mlp.down_proj.weight",
        }
        layers.append(LayerSpec(block=block, names=names))
    tied = cfg.tie_word_embeddings
    return ModelSpec(
        vocab_size=cfg.vocab_size,
        width=cfg.hidden_size,
        embedding_name="model.embed_tokens.weight",
        layers=tuple(layers),
        schedule=tuple(RunSpec(layer=i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm,
        final_norm_names={"weight": "model.norm.weight"},
        head_name=None if tied else "lm_head.weight",
        # a tied checkpoint may still carry a copy of the head; it is not used
        ignored_names=("lm_head.weight",) if tied else (),
        max_positions=cfg.max_position_embeddings,
        stop_ids=tuple(cfg.eos_token_ids),
    )


def describe(config: Dict[str, Any]) -> ModelSpec:
    return qwen3_spec(Qwen3Config.from_dict(config))
