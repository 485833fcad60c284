"""A plain, slow LFM2 dense model: whole sequences, no cache, float64, one function a part.

It rests on the formulas of celsowm/celeg's source (cited per function, paths inside
that project). It shares no code with the ``celeg_b200`` package: it reads
config.json with ``json`` and model.safetensors with the ``safetensors`` library.
One deliberate difference from celeg's CPU backend: attention scores are scaled by
1/sqrt(head_dim) ONCE, which is what celeg's CUDA kernel does
(src/backend/cuda/kernels/attention_paged.cuh:21) and what its CPU attention kernel
states (src/backend/cpu/attention/paged_attention.cpp:254); the CPU backend's QK-norm
branch multiplies the query by the same factor a second time
(src/backend/cpu/operators/attention.cpp:77-79). ``tests/golden/`` holds a comparison
with celeg's compiled CPU kernels where they could be built.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np


# --------------------------------------------------------------------------- loading
def load_model_folder(model_dir: str):
    """(config dict, {tensor name: float64 array})."""
    import torch
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as handle:
        config = json.load(handle)
    tensors = {name: value.to(torch.float64).numpy()
               for name, value in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return config, tensors


def layer_kinds(config: dict, tensors: Dict[str, np.ndarray]) -> List[str]:
    """``layer_types`` if stated; else by which mixer tensors a layer owns, as celeg
    decides (src/model/inference/rules.cpp:150-212)."""
    count = config["num_hidden_layers"]
    if config.get("layer_types") is not None:
        return list(config["layer_types"])
    if config.get("full_attn_idxs") is not None:
        marked = set(config["full_attn_idxs"])
        return ["full_attention" if i in marked else "conv" for i in range(count)]
    return ["conv" if f"model.layers.{i}.conv.in_proj.weight" in tensors else "full_attention"
            for i in range(count)]


# ----------------------------------------------------------------------------- parts
def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """y_i = x_i / sqrt(mean_j x_j^2 + eps) * w_i over the last axis; the weight is a
    direct scale. src/backend/cpu/kernels/elementwise.cpp:72-75."""
    mean_square = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(mean_square + eps) * weight


def rope_split_half(x: np.ndarray, positions: np.ndarray, theta: float) -> np.ndarray:
    """Rotate pairs (i, i + d/2) of each head by angle position * theta^(-2i/d).
    x is [T, heads, d]. Pairing: src/backend/cpu/kernels/rope.cpp:30-36 (split half);
    frequency: include/celeg/model/position.hpp:77-78; rotation: rope.cpp:104-109."""
    d = x.shape[-1]
    half = d // 2
    frequency = theta ** (-2.0 * np.arange(half, dtype=np.float64) / d)
    angle = positions.astype(np.float64)[:, None] * frequency[None, :]          # [T, half]
    cos = np.cos(angle)[:, None, :]
    sin = np.sin(angle)[:, None, :]
    a = x[..., :half]
    b = x[..., half:]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1)


def short_conv_mixer(n: np.ndarray, w_in: np.ndarray, kernel: np.ndarray, w_out: np.ndarray) -> np.ndarray:
    """[B|C|X] = n W_in^T in that order; bx = B*X; conv_t = sum_tap K[c,tap] * bx_{t-(L-1)+tap}
    (tap L-1 multiplies the current token, earlier-than-start terms are zero); y = C*conv;
    out = y W_out^T. No bias, no activation.
    src/backend/cpu/kernels/convolution.cpp:7-28 (order of B, C, X at :16-18; taps at :21-25,
    with the kernel stored channel-major [H,1,L]: src/backend/cpu/weights_loader.cpp:453-463)."""
    tokens, hidden = n.shape
    projected = n @ w_in.T
    b, c, x = projected[:, :hidden], projected[:, hidden:2 * hidden], projected[:, 2 * hidden:]
    bx = b * x
    kernel = kernel.reshape(hidden, -1)
    taps = kernel.shape[1]
    conv = np.zeros_like(bx)
    for t in range(tokens):
        for tap in range(taps):
            source = t - (taps - 1) + tap
            if source >= 0:
                conv[t] += kernel[:, tap] * bx[source]
    return (c * conv) @ w_out.T


def attention_mixer(n: np.ndarray, wq: np.ndarray, wk: np.ndarray, wv: np.ndarray, wo: np.ndarray,
                    q_norm: np.ndarray, k_norm: np.ndarray, heads: int, kv_heads: int, head_dim: int,
                    theta: float, eps: float, positions: Optional[np.ndarray] = None,
                    window: Optional[int] = None, score_scale: Optional[float] = None) -> np.ndarray:
    """q,k,v projections; per-head RMSNorm of q and k (weights [d]); split-half RoPE on q and k;
    causal grouped-query softmax(q k^T / sqrt(d)) v (:func:`causal_attention`); out projection.
    src/backend/cpu/operators/attention_token.cpp:151-204; norm+RoPE
    src/backend/cpu/kernels/rope.cpp:61-110."""
    tokens = n.shape[0]
    if positions is None:
        positions = np.arange(tokens)
    q = (n @ wq.T).reshape(tokens, heads, head_dim)
    k = (n @ wk.T).reshape(tokens, kv_heads, head_dim)
    v = (n @ wv.T).reshape(tokens, kv_heads, head_dim)
    q = rope_split_half(rmsnorm(q, q_norm, eps), positions, theta)
    k = rope_split_half(rmsnorm(k, k_norm, eps), positions, theta)
    # (``score_scale`` exists for one test only: celeg's CPU build scales the scores of this branch twice)
    out = causal_attention(q, k, v, 1.0 / math.sqrt(head_dim) if score_scale is None else score_scale, window)
    return out.reshape(tokens, heads * head_dim) @ wo.T


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float,
                     window: Optional[int] = None) -> np.ndarray:
    """softmax(q k^T * scale) v over one sequence: q [T, heads, d], k and v [T, kv_heads, d], all after norm
    and rotation. Query head h reads kv head h // (heads / kv_heads) (paged_attention.cpp:259); the query at
    position p reads keys 0..p (with a window only the last ``window`` of them); the scale is applied once, to
    the dot product (paged_attention.cpp:254, :204); softmax subtracts the row maximum (:206-210).
    src/backend/cpu/attention/paged_attention.cpp:185-283."""
    tokens, heads, head_dim = q.shape
    group = heads // k.shape[1]
    out = np.zeros((tokens, heads, head_dim))
    for h in range(heads):
        kh = h // group
        scores = (q[:, h, :] @ k[:, kh, :].T) * scale                       # [T, T]
        row = np.arange(tokens)[:, None]
        col = np.arange(tokens)[None, :]
        mask = col > row
        if window is not None:
            mask |= col <= row - window
        scores = np.where(mask, -np.inf, scores)
        scores = scores - scores.max(axis=-1, keepdims=True)
        weights = np.exp(scores)
        weights /= weights.sum(axis=-1, keepdims=True)
        out[:, h, :] = weights @ v[:, kh, :]
    return out


def swiglu(n: np.ndarray, w1: np.ndarray, w3: np.ndarray, w2: np.ndarray) -> np.ndarray:
    """(silu(n W1^T) * (n W3^T)) W2^T with silu(g) = g / (1 + exp(-g)).
    src/backend/cpu/operators/feed_forward.cpp:54-71; src/backend/cpu/kernels/elementwise.cpp:114-118."""
    gate = n @ w1.T
    up = n @ w3.T
    return (gate / (1.0 + np.exp(-gate)) * up) @ w2.T


def block(x: np.ndarray, index: int, kind: str, config: dict, w: Dict[str, np.ndarray],
          score_scale: Optional[float] = None) -> np.ndarray:
    """h = x + Mixer(RMSNorm(x; operator_norm)); y = h + FFN(RMSNorm(h; ffn_norm)).
    src/backend/cpu/model_forward_token.cpp:89-176."""
    p = f"model.layers.{index}."
    eps = norm_eps(config)
    n = rmsnorm(x, w[p + "operator_norm.weight"], eps)
    if kind == "conv":
        mixed = short_conv_mixer(n, w[p + "conv.in_proj.weight"], w[p + "conv.conv.weight"],
                                 w[p + "conv.out_proj.weight"])
    else:
        heads = config["num_attention_heads"]
        mixed = attention_mixer(
            n, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
            w[p + "self_attn.v_proj.weight"], w[p + "self_attn.out_proj.weight"],
            w[p + "self_attn.q_layernorm.weight"], w[p + "self_attn.k_layernorm.weight"],
            heads, config.get("num_key_value_heads", heads), head_dim(config), rope_theta(config), eps,
            score_scale=score_scale)
    h = x + mixed
    n2 = rmsnorm(h, w[p + "ffn_norm.weight"], eps)
    return h + swiglu(n2, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"],
                      w[p + "feed_forward.w2.weight"])


def norm_eps(config: dict) -> float:
    """src/model/inference/metadata.cpp:404-406 (aliases), :643 (1e-6 when absent)."""
    for key in ("norm_eps", "rms_norm_eps", "rms_norm_epsilon", "layer_norm_epsilon"):
        if key in config:
            return float(config[key])
    return 1e-6


def head_dim(config: dict) -> int:
    """src/model/inference/rules_attention.cpp:194-204."""
    return int(config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"])


def rope_theta(config: dict) -> float:
    if "rope_theta" in config:
        return float(config["rope_theta"])
    return float(config["rope_parameters"]["rope_theta"])


def forward(config: dict, w: Dict[str, np.ndarray], tokens: Sequence[int],
            score_scale: Optional[float] = None) -> np.ndarray:
    """Logits [T, V] of a whole sequence: embedding rows, the blocks, RMSNorm with
    ``model.embedding_norm``, then the head (``lm_head.weight`` if present, else the
    embedding table). src/backend/cpu/model_forward_token.cpp:50-54, 213-230."""
    x = w["model.embed_tokens.weight"][np.asarray(tokens, dtype=np.int64)]
    for index, kind in enumerate(layer_kinds(config, w)):
        x = block(x, index, kind, config, w, score_scale)
    z = rmsnorm(x, w["model.embedding_norm.weight"], norm_eps(config))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return z @ head.T


# -------------------------------------------------------------------------- sampling
_MASK64 = (1 << 64) - 1


def xorshift64star(state: int):
    """src/backend/cpu/sampler.cpp:10-15. Returns (new state, output bits)."""
    state ^= state >> 12
    state = (state ^ (state << 25)) & _MASK64
    state ^= state >> 27
    return state, (state * 2685821657736338717) & _MASK64


def random_unit(state: int):
    """src/backend/cpu/sampler.cpp:17-22: ((bits >> 11) + 0.5) / 2^53 as a float32."""
    state, bits = xorshift64star(state)
    return state, float(np.float32(((bits >> 11) + 0.5) * (1.0 / 9007199254740992.0)))


def sample_token(logits: np.ndarray, seen: np.ndarray, rng_state: int, temperature: float, top_k: int,
                 top_p: float, repetition_penalty: float):
    """celeg's sampler, src/backend/cpu/sampler.cpp:26-101, in float32 like the original.
    Returns (token, new rng state)."""
    f32 = np.float32
    values = logits.astype(f32).copy()
    if repetition_penalty > 1.0:
        penalty = f32(repetition_penalty)
        marked = seen.astype(bool)
        values[marked] = np.where(values[marked] >= 0, values[marked] / penalty, values[marked] * penalty)
    if temperature <= 0.0 or top_k == 1:
        return int(np.argmax(values)), rng_state          # first maximum wins (:44-55)
    scores = values / f32(temperature)
    k = min(top_k, scores.shape[0])
    order = np.lexsort((np.arange(scores.shape[0]), -scores))[:k]      # score desc, then token asc (:62-64)
    chosen = scores[order]
    probabilities = np.exp(chosen - chosen[0]).astype(f32)
    total = f32(0.0)
    for p in probabilities:
        total = f32(total + p)
    probabilities = (probabilities / total).astype(f32)
    active = len(probabilities)
    if top_p < 1.0:
        cumulative = f32(0.0)
        active = 0
        while True:
            cumulative = f32(cumulative + probabilities[active])
            active += 1
            if not (active < len(probabilities) and cumulative < f32(top_p)):
                break
        total = f32(0.0)
        for p in probabilities[:active]:
            total = f32(total + p)
    else:
        total = f32(1.0)
    rng_state, unit = random_unit(rng_state)
    target = f32(f32(unit) * total)
    for i in range(active):
        target = f32(target - probabilities[i])
        if target <= 0.0:
            return int(order[i]), rng_state
    return int(order[active - 1]), rng_state


def generate(config: dict, w: Dict[str, np.ndarray], prompt: Sequence[int], max_new_tokens: int,
             temperature: float = 0.0, top_k: int = 1, top_p: float = 1.0, repetition_penalty: float = 1.0,
             seed: int = 1, eos_tokens: Sequence[int] = ()) -> List[int]:
    """Whole-sequence forward pass for every new token (no cache); the token is drawn from the
    logits of the last position; tokens of the prompt and generated ones count as seen
    (src/backend/cpu/model.cpp:144-160); generation stops after an eos token, which is emitted
    (src/backend/cuda/runtime/decode_scheduler.cpp:95-98)."""
    sequence = list(prompt)
    seen = np.zeros(w["model.embed_tokens.weight"].shape[0], dtype=np.uint8)
    seen[np.asarray(sequence, dtype=np.int64)] = 1
    produced: List[int] = []
    state = seed
    for _ in range(max_new_tokens):
        logits = forward(config, w, sequence)[-1]
        token, state = sample_token(logits, seen, state, temperature, top_k, top_p, repetition_penalty)
        produced.append(token)
        sequence.append(token)
        seen[token] = 1
        if token in eos_tokens:
            break
    return produced
