"""The LFM2 dense architecture as an arrangement of parts.

Layer structure, tensor names and shapes are the ones celeg binds for an LFM2
checkpoint: short-convolution mixer for layers that own ``conv.in_proj``
(src/model/inference/rules.cpp:12-90), standard attention with per-head q/k
norms for layers that own ``self_attn.q_proj``
(src/model/inference/rules_attention.cpp:72-92, 138-326), dense SwiGLU
feed-forward ``feed_forward.w1/w3/w2`` (src/model/inference/support.cpp:80-112),
``operator_norm`` / ``ffn_norm`` pre-norms (src/model/inference/layer_bindings.cpp:267-303),
``model.embedding_norm`` as the final norm (layer_bindings.cpp:97-106) and a
head tied to the embedding when ``lm_head.weight`` is absent (layer_bindings.cpp:31-95).
"""
from __future__ import annotations

from typing import Any, Mapping

from .lfm2 import CONV, FULL_ATTENTION, Lfm2Config
from .registry import Architecture, register_architecture
from .spec import ExecutionEntry, LayerSpec, ModelSpec, PartSpec, TensorRef


def _rmsnorm(name: str, width: int, eps: float) -> PartSpec:
    return PartSpec(kind="rmsnorm", params={"width": width, "eps": eps},
                    tensors={"weight": TensorRef(name, (width,))})


def build_lfm2_spec(config: Lfm2Config) -> ModelSpec:
    config.require_resolved()
    hidden = config.hidden_size
    q_width = config.num_attention_heads * config.head_dim
    kv_width = config.num_key_value_heads * config.head_dim
    inner = config.intermediate_size
    layers = []
    for index, kind in enumerate(config.layer_types):
        base = f"model.layers.{index}"
        if kind == CONV:
            taps = config.conv_L_cache
            mixer = PartSpec(
                kind="short_conv",
                params={"hidden_size": hidden, "taps": taps},
                tensors={
                    "in_proj": TensorRef(f"{base}.conv.in_proj.weight", (3 * hidden, hidden)),
                    "conv": TensorRef(f"{base}.conv.conv.weight", (hidden, taps),
                                      alt_shapes=((hidden, 1, taps),)),
                    "out_proj": TensorRef(f"{base}.conv.out_proj.weight", (hidden, hidden)),
                })
        elif kind == FULL_ATTENTION:
            position = PartSpec(kind="rope_split_half",
                                params={"theta": config.rope_theta, "rotary_dim": config.head_dim,
                                        "head_dim": config.head_dim})
            mixer = PartSpec(
                kind="attention",
                params={"hidden_size": hidden, "num_heads": config.num_attention_heads,
                        "num_kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                        "qk_norm_eps": config.norm_eps, "window": None,
                        "softmax_scale": config.head_dim ** -0.5},
                tensors={
                    "q_proj": TensorRef(f"{base}.self_attn.q_proj.weight", (q_width, hidden)),
                    "k_proj": TensorRef(f"{base}.self_attn.k_proj.weight", (kv_width, hidden)),
                    "v_proj": TensorRef(f"{base}.self_attn.v_proj.weight", (kv_width, hidden)),
                    "out_proj": TensorRef(f"{base}.self_attn.out_proj.weight", (hidden, q_width)),
                    "q_norm": TensorRef(f"{base}.self_attn.q_layernorm.weight", (config.head_dim,)),
                    "k_norm": TensorRef(f"{base}.self_attn.k_layernorm.weight", (config.head_dim,)),
                },
                parts={"position": position})
        else:  # validate() has refused every other kind
            raise AssertionError(kind)
        feed_forward = PartSpec(
            kind="swiglu",
            params={"hidden_size": hidden, "intermediate_size": inner},
            tensors={
                "gate": TensorRef(f"{base}.feed_forward.w1.weight", (inner, hidden)),
                "up": TensorRef(f"{base}.feed_forward.w3.weight", (inner, hidden)),
                "down": TensorRef(f"{base}.feed_forward.w2.weight", (hidden, inner)),
            })
        layers.append(LayerSpec(
            name=base, arrangement="prenorm_residual",
            mixer_norm=_rmsnorm(f"{base}.operator_norm.weight", hidden, config.norm_eps),
            mixer=mixer,
            feed_forward_norm=_rmsnorm(f"{base}.ffn_norm.weight", hidden, config.norm_eps),
            feed_forward=feed_forward))
    spec = ModelSpec(
        architecture=config.model_type,
        vocab_size=config.vocab_size,
        hidden_size=hidden,
        max_context=config.max_position_embeddings,
        embedding=TensorRef("model.embed_tokens.weight", (config.vocab_size, hidden)),
        layers=tuple(layers),
        order=tuple(ExecutionEntry(layer=i) for i in range(len(layers))),
        final_norm=_rmsnorm("model.embedding_norm.weight", hidden, config.norm_eps),
        lm_head=None if config.tie_word_embeddings else TensorRef("lm_head.weight", (config.vocab_size, hidden)),
        eos_token_ids=tuple(config.eos_token_ids),
        bos_token_id=config.bos_token_id,
    )
    spec.validate()
    return spec


def lfm2_random_init(config: Lfm2Config, name: str, shape: tuple) -> str:
    """Distribution of a tensor in random-weights mode: norm weights 1+N(0,0.05),
    conv kernels N(0,0.1), every matrix N(0,0.02)."""
    if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
        return "norm"
    if name.endswith(".conv.conv.weight"):
        return "conv"
    return "linear"


def _parse(raw: Mapping[str, Any]) -> Lfm2Config:
    return Lfm2Config.from_dict(raw)


def _resolve(config: Lfm2Config, tensor_shapes: Mapping[str, Any]) -> Lfm2Config:
    return config.resolved_with(tensor_shapes)


LFM2 = Architecture(name="lfm2", parse_config=_parse, resolve_config=_resolve,
                    build_spec=build_lfm2_spec, random_init=lfm2_random_init)
register_architecture(LFM2, replace=True)
