"""Typed configuration of the LFM2 dense decoder, read from its own config.json keys.

Key names, aliases and defaults follow celeg's metadata normaliser
(src/model/inference/metadata.cpp:350-432, 630-666): every size comes from
config.json (or, where celeg takes it from a tensor shape, from the checkpoint's
tensor index); nothing is hard-wired here.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Mapping, Optional, Sequence

from .errors import ConfigError

CONV = "conv"
FULL_ATTENTION = "full_attention"
_LAYER_KINDS = (CONV, FULL_ATTENTION)

_MISSING = object()


def _lookup(raw: Mapping[str, Any], names: Sequence[str], default: Any = _MISSING) -> Any:
    """First present key among ``names``; dotted names descend into nested objects;
    ``text_config.`` is tried as a fallback scope, as celeg's flattened metadata does
    (src/checkpoint/formats/metadata.cpp, dotted keys)."""
    for scope in ((), ("text_config",)):
        for name in names:
            node: Any = raw
            for part in (*scope, *name.split(".")):
                if isinstance(node, Mapping) and part in node:
                    node = node[part]
                else:
                    node = _MISSING
                    break
            if node is not _MISSING and node is not None:
                return node
    return default


def _as_int(raw: Mapping[str, Any], names: Sequence[str], default: Any = _MISSING) -> Any:
    value = _lookup(raw, names, default)
    if value is _MISSING:
        raise ConfigError(f"config.json lacks required key '{names[0]}' (aliases: {', '.join(names[1:]) or 'none'})")
    if value is None:
        return None
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
        raise ConfigError(f"config key '{names[0]}' must be an integer, got {value!r}")
    return int(value)


def _as_float(raw: Mapping[str, Any], names: Sequence[str], default: Any = _MISSING) -> Any:
    value = _lookup(raw, names, default)
    if value is _MISSING:
        raise ConfigError(f"config.json lacks required key '{names[0]}' (aliases: {', '.join(names[1:]) or 'none'})")
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config key '{names[0]}' must be a number, got {value!r}")
    return float(value)


def _token_ids(value: Any, key: str) -> tuple:
    if value is None:
        return ()
    if isinstance(value, (list, tuple)):
        items = list(value)
    else:
        items = [value]
    for item in items:
        if isinstance(item, bool) or not isinstance(item, int):
            raise ConfigError(f"config key '{key}' must be an integer or a list of integers, got {value!r}")
    return tuple(int(item) for item in items)


@dataclass(frozen=True)
class Lfm2Config:
    """All sizes and constants of one LFM2 dense model.

    ``layer_types``, ``intermediate_size`` and ``tie_word_embeddings`` may be ``None``
    after :meth:`from_dict` when config.json does not state them; :meth:`resolved_with`
    fills them from the checkpoint's tensor names and shapes, which is where celeg
    itself finds them (src/model/inference/global_facts.cpp:101-158,
    src/model/inference/rules.cpp:150-212, src/model/inference/layer_bindings.cpp:31-95).
    """

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    conv_L_cache: Optional[int]
    rope_theta: Optional[float]
    norm_eps: float
    max_position_embeddings: int
    layer_types: Optional[tuple] = None
    intermediate_size: Optional[int] = None
    tie_word_embeddings: Optional[bool] = None
    bos_token_id: int = 0
    eos_token_ids: tuple = (0,)
    pad_token_id: int = 1
    model_type: str = "lfm2"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Lfm2Config":
        if not isinstance(raw, Mapping):
            raise ConfigError("config.json must hold a JSON object")
        hidden = _as_int(raw, ("hidden_size", "n_embd", "d_model"))
        layers = _as_int(raw, ("num_hidden_layers", "n_layer", "num_layers"))
        vocab = _as_int(raw, ("vocab_size", "n_vocab"))
        heads = _as_int(raw, ("num_attention_heads", "n_head"))
        kv_heads = _as_int(raw, ("num_key_value_heads", "n_kv_heads"), heads)
        head_dim = _as_int(raw, ("head_dim",), None)
        if head_dim is None:
            # src/model/inference/rules_attention.cpp:194-204: hidden_size / num_attention_heads
            if heads <= 0 or hidden % heads != 0:
                raise ConfigError(
                    f"head_dim is absent and hidden_size {hidden} is not divisible by num_attention_heads {heads}")
            head_dim = hidden // heads
        context = _as_int(raw, ("max_position_embeddings", "max_seq_len", "context_length"))
        # src/model/inference/metadata.cpp:643: 1e-6 when no epsilon key is present
        eps = _as_float(raw, ("norm_eps", "rms_norm_eps", "rms_norm_epsilon", "layer_norm_epsilon"), 1e-6)
        conv_cache = _as_int(raw, ("conv_L_cache",), None)
        theta = _lookup(raw, ("rope_theta", "rope_parameters.rope_theta",
                              "rope_parameters.full_attention.rope_theta"), None)
        if theta is not None:
            if isinstance(theta, bool) or not isinstance(theta, (int, float)):
                raise ConfigError(f"config key 'rope_theta' must be a number, got {theta!r}")
            theta = float(theta)

        layer_types = _lookup(raw, ("layer_types",), None)
        if layer_types is not None:
            if not isinstance(layer_types, (list, tuple)) or not all(isinstance(t, str) for t in layer_types):
                raise ConfigError("config key 'layer_types' must be a list of strings")
            layer_types = tuple(layer_types)
        else:
            attn_idxs = _lookup(raw, ("full_attn_idxs",), None)
            if attn_idxs is not None:
                if not isinstance(attn_idxs, (list, tuple)) or not all(
                        isinstance(i, int) and not isinstance(i, bool) for i in attn_idxs):
                    raise ConfigError("config key 'full_attn_idxs' must be a list of integers")
                bad = [i for i in attn_idxs if not 0 <= i < layers]
                if bad:
                    raise ConfigError(f"full_attn_idxs {bad} lie outside 0..{layers - 1}")
                marked = set(attn_idxs)
                layer_types = tuple(FULL_ATTENTION if i in marked else CONV for i in range(layers))

        intermediate = _as_int(raw, ("intermediate_size", "n_inner", "ffn_dim"), None)
        if intermediate is None:
            block_ff = _as_int(raw, ("block_ff_dim",), None)
            auto_adjust = _lookup(raw, ("block_auto_adjust_ff_dim",), False)
            # With auto-adjust on, celeg reads the width from feed_forward.w1.weight's
            # shape (global_facts.cpp:144-150); resolved_with() does the same.
            if block_ff is not None and not auto_adjust:
                intermediate = block_ff

        tie = _lookup(raw, ("tie_word_embeddings", "tied_embeddings", "tie_embedding"), None)
        if tie is not None and not isinstance(tie, bool):
            raise ConfigError(f"config key 'tie_word_embeddings' must be true or false, got {tie!r}")

        if _lookup(raw, ("conv_bias",), False):
            raise ConfigError("conv_bias=true is not supported: the short convolution has no bias "
                              "(celeg src/model/inference/rules.cpp:41-42)")
        for key in ("rope_scaling", "sliding_window"):
            if _lookup(raw, (key,), None) not in (None, {}, 0):
                raise ConfigError(f"config key '{key}' is not part of the LFM2 dense architecture and is not supported")
        rotary = _lookup(raw, ("rotary_fraction", "partial_rotary_factor"), 1.0)
        if float(rotary) != 1.0:
            raise ConfigError("LFM2 dense applies rotary embedding to the whole head; partial_rotary_factor != 1 "
                              "is not supported")

        bos = _as_int(raw, ("bos_token_id",), 0)       # metadata.cpp:640-642 defaults
        pad = _as_int(raw, ("pad_token_id",), 1)
        eos = _token_ids(_lookup(raw, ("eos_token_id",), 0), "eos_token_id")
        known = {"hidden_size", "num_hidden_layers", "vocab_size", "num_attention_heads",
                 "num_key_value_heads", "head_dim", "max_position_embeddings", "norm_eps", "conv_L_cache",
                 "rope_theta", "layer_types", "full_attn_idxs", "intermediate_size", "block_ff_dim",
                 "block_auto_adjust_ff_dim", "tie_word_embeddings", "bos_token_id", "eos_token_id",
                 "pad_token_id", "model_type", "conv_bias"}
        config = cls(
            vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            conv_L_cache=conv_cache, rope_theta=theta, norm_eps=eps,
            max_position_embeddings=context, layer_types=layer_types,
            intermediate_size=intermediate, tie_word_embeddings=tie,
            bos_token_id=bos, eos_token_ids=eos, pad_token_id=pad,
            model_type=str(raw.get("model_type", "lfm2")),
            extra={k: v for k, v in raw.items() if k not in known},
        )
        config.validate()
        return config

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        """Checks of celeg's global facts (src/model/inference/global_facts.cpp:10-21, 213-219)
        and attention rule (src/model/inference/rules_attention.cpp:181-204)."""
        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config key '{name}' must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary embedding")
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm_eps must be positive, got {self.norm_eps}")
        if self.intermediate_size is not None and self.intermediate_size <= 0:
            raise ConfigError(f"intermediate_size must be positive, got {self.intermediate_size}")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(f"layer_types names {len(self.layer_types)} layers, "
                                  f"num_hidden_layers is {self.num_hidden_layers}")
            for index, kind in enumerate(self.layer_types):
                if kind not in _LAYER_KINDS:
                    raise ConfigError(f"layer_types[{index}] is '{kind}'; known kinds: {', '.join(_LAYER_KINDS)}")
            if CONV in self.layer_types:
                # src/model/inference/rules.cpp:36-40
                if self.conv_L_cache is None:
                    raise ConfigError("a conv layer exists but config.json lacks 'conv_L_cache'")
                if self.conv_L_cache < 1:
                    raise ConfigError(f"conv_L_cache must be at least 1, got {self.conv_L_cache}")
            if FULL_ATTENTION in self.layer_types and self.rope_theta is None:
                # src/model/inference/metadata.cpp:663-666
                raise ConfigError("an attention layer applies RoPE but config.json does not specify 'rope_theta'")
        if self.rope_theta is not None and not self.rope_theta > 0.0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        for token in (self.bos_token_id, self.pad_token_id, *self.eos_token_ids):
            if token < 0:
                raise ConfigError(f"token id {token} is negative")

    # ---------------------------------------------- completion from the tensors
    def resolved_with(self, tensor_shapes: Mapping[str, Sequence[int]]) -> "Lfm2Config":
        """Fill what config.json left open from the checkpoint's tensor names and shapes."""
        updates: dict = {}
        prefix = "model.layers."
        if self.layer_types is None:
            kinds = []
            for index in range(self.num_hidden_layers):
                has_conv = f"{prefix}{index}.conv.in_proj.weight" in tensor_shapes
                has_attn = f"{prefix}{index}.self_attn.q_proj.weight" in tensor_shapes
                if has_conv == has_attn:
                    raise ConfigError(
                        f"config.json gives no layer_types and layer {index} has "
                        f"{'both a conv and an attention' if has_conv else 'neither a conv nor an attention'} "
                        f"mixer among the tensors")
                kinds.append(CONV if has_conv else FULL_ATTENTION)
            updates["layer_types"] = tuple(kinds)
        if self.intermediate_size is None:
            name = f"{prefix}0.feed_forward.w1.weight"
            shape = tensor_shapes.get(name)
            if shape is None or len(shape) != 2:
                raise ConfigError(f"config.json gives no intermediate_size and tensor '{name}' is absent")
            updates["intermediate_size"] = int(shape[0])
        if self.tie_word_embeddings is None:
            updates["tie_word_embeddings"] = "lm_head.weight" not in tensor_shapes
        config = replace(self, **updates) if updates else self
        config.validate()
        return config

    def require_resolved(self) -> None:
        missing = [name for name in ("layer_types", "intermediate_size", "tie_word_embeddings")
                   if getattr(self, name) is None]
        if missing:
            raise ConfigError("config.json does not state " + ", ".join(missing) +
                              "; without a checkpoint to read them from they must be given")

    # ------------------------------------------------------------------- output
    def to_dict(self) -> dict:
        """config.json content that :meth:`from_dict` reads back to an equal configuration."""
        self.require_resolved()
        out = {
            "model_type": self.model_type,
            "architectures": ["Lfm2ForCausalLM"],
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "max_position_embeddings": self.max_position_embeddings,
            "norm_eps": self.norm_eps,
            "layer_types": list(self.layer_types),
            "tie_word_embeddings": self.tie_word_embeddings,
            "conv_bias": False,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": list(self.eos_token_ids) if len(self.eos_token_ids) != 1 else self.eos_token_ids[0],
            "pad_token_id": self.pad_token_id,
        }
        if self.conv_L_cache is not None:
            out["conv_L_cache"] = self.conv_L_cache
        if self.rope_theta is not None:
            out["rope_theta"] = self.rope_theta
        return out
