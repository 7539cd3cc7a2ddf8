"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache.

Written from the formulas of beyondHJM/tinyinfer.cpp (file:line cited at each
function); it rests on those formulas only.  The reference's own model code cannot
be run on a CPU: every weight path calls cudaMalloc (src/model.cpp:63-117) and all
model arithmetic lives in CUDA kernels (src/cuda/*.cu), so there is no output of
the reference to compare with here.

This file shares no code with the engine.  It reads ``config.json`` as a plain
dictionary and tensors through the ``safetensors`` library.  Arithmetic is float64,
except where the architecture fixes a precision:

* the rotation angle is float32: ``float32(pos) * float32(theta ** (-2k/hd))``;
* with ``emulate_bf16=True`` values are rounded to bfloat16 exactly where the
  reference rounds them: the normed input of every product (src/inference.cu:40,59),
  keys and values entering the cache (src/cuda/attention.cu:82-84), the attention
  output (src/inference.cu:53), the SwiGLU output (src/inference.cu:63) and the
  final-norm rows (src/cuda/lm_head.cu:8).
"""
from __future__ import annotations

import json
import math
import os

import torch

F64 = torch.float64


def _round(x: torch.Tensor, emulate_bf16: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(F64) if emulate_bf16 else x


def plain_embedding(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """x[t] = E[token[t]], no scaling (src/inference.cu:14-24)."""
    return table.to(F64)[tokens.long()]


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w over the last axis (src/cuda/rms_norm.cu:15-25)."""
    x = x.to(F64)
    mean_sq = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(mean_sq + eps) * weight.to(F64)


def plain_rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """angle[t, k] = pos[t] * theta^(-2k/head_dim), k < head_dim/2 (src/cuda/attention.cu:38,64-66).
    The angle is a float32 product of float32 factors."""
    k = torch.arange(head_dim // 2, dtype=F64)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=F64), -2.0 * k / head_dim).to(torch.float32)
    return positions.to(torch.float32)[:, None] * inv_freq[None, :]


def plain_rope_neox(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of x[t, head, :]: pairs (x[k], x[k + hd/2]) (src/cuda/attention.cu:67-73)."""
    half = x.shape[-1] // 2
    c = torch.cos(angles.to(F64))[:, None, :]
    s = torch.sin(angles.to(F64))[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                    window: int | None = None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence (src/cuda/attention.cu:127-130,147-197).

    q [S, heads, hd], k and v [S, kv_heads, hd].  Query head i uses kv head
    i // (heads / kv_heads); position t sees p <= t, and p > t - window if a window is given.
    """
    s_len, heads, hd = q.shape
    group = heads // k.shape[1]
    out = torch.zeros_like(q)
    pos = torch.arange(s_len)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - window
    for h in range(heads):
        kh, vh = k[:, h // group, :], v[:, h // group, :]
        scores = (q[:, h, :] @ kh.T) * scale
        scores = scores.masked_fill(~allowed, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ vh
    return out


def plain_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """gate / (1 + exp(-gate)) * up (src/cuda/ffn.cu:13-15)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def plain_attention_block(x, w, prefix, cfg, positions, window, emulate_bf16):
    """norm -> q,k,v -> per-head q/k norm -> rotation -> attention -> o (src/inference.cu:39-55,
    src/cuda/attention.cu:51-74)."""
    heads, kv_heads = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // heads
    eps = cfg.get("rms_norm_eps", 1e-6)
    s_len = x.shape[0]
    h = _round(plain_rmsnorm(x, w[prefix + "input_layernorm.weight"], eps), emulate_bf16)
    a = prefix + "self_attn."
    q = (h @ w[a + "q_proj.weight"].to(F64).T).view(s_len, heads, hd)
    k = (h @ w[a + "k_proj.weight"].to(F64).T).view(s_len, kv_heads, hd)
    v = (h @ w[a + "v_proj.weight"].to(F64).T).view(s_len, kv_heads, hd)
    q = plain_rmsnorm(q, w[a + "q_norm.weight"], eps)
    k = plain_rmsnorm(k, w[a + "k_norm.weight"], eps)
    angles = plain_rope_angles(positions, hd, cfg.get("rope_theta", 1e6))
    q = plain_rope_neox(q, angles)
    k = _round(plain_rope_neox(k, angles), emulate_bf16)
    v = _round(v, emulate_bf16)
    o = plain_attention(q, k, v, 1.0 / math.sqrt(hd), window)
    o = _round(o.reshape(s_len, heads * hd), emulate_bf16)
    return o @ w[a + "o_proj.weight"].to(F64).T


def plain_mlp_block(x, w, prefix, cfg, emulate_bf16):
    """norm -> gate, up -> SwiGLU -> down (src/inference.cu:58-64)."""
    eps = cfg.get("rms_norm_eps", 1e-6)
    h = _round(plain_rmsnorm(x, w[prefix + "post_attention_layernorm.weight"], eps), emulate_bf16)
    m = prefix + "mlp."
    gate = h @ w[m + "gate_proj.weight"].to(F64).T
    up = h @ w[m + "up_proj.weight"].to(F64).T
    y = _round(plain_swiglu(gate, up), emulate_bf16)
    return y @ w[m + "down_proj.weight"].to(F64).T


def plain_forward(cfg: dict, w: dict, tokens, emulate_bf16: bool = False) -> torch.Tensor:
    """Logits [S, vocab] (float64) of one whole sequence (src/inference.cu:28-72)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    layer_types = cfg.get("layer_types") or ["full_attention"] * cfg["num_hidden_layers"]
    x = plain_embedding(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        window = cfg.get("sliding_window") if layer_types[i] == "sliding_attention" else None
        x = x + plain_attention_block(x, w, p, cfg, positions, window, emulate_bf16)
        x = x + plain_mlp_block(x, w, p, cfg, emulate_bf16)
    h = _round(plain_rmsnorm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6)), emulate_bf16)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return h @ head.to(F64).T


def plain_greedy(cfg: dict, w: dict, prompt, steps: int, emulate_bf16: bool = False) -> list[int]:
    """Greedy continuation, the first maximum winning ties (src/main.cpp:31-38); every step
    recomputes the whole sequence."""
    seq = list(prompt)
    out = []
    for _ in range(steps):
        logits = plain_forward(cfg, w, seq, emulate_bf16)[-1]
        nxt = int(torch.argmax(logits))
        out.append(nxt)
        seq.append(nxt)
    return out


def load_folder(model_dir: str):
    """(config dictionary, tensors by name as stored) of a model folder."""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    return cfg, load_file(os.path.join(model_dir, "model.safetensors"))
