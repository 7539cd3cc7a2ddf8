"""Typed configuration of the Qwen3 dense decoder and its plan.

Field meanings follow the reference's ``Qwen3Config`` (src/model.h:11-21, read
at src/model.cpp:32-41 and checked at src/model.cpp:43-47); the key names are
those of the architecture's ``config.json``.  Sizes have no defaults: a missing
size is an error.  ``rope_theta`` and ``rms_norm_eps`` default as the reference
defaults them (1e6 and 1e-6, src/model.cpp:39-40).

The layer formulas the plan stands for (reference order, src/inference.cu:35-66):
x -> RMSNorm -> QKV -> per-head q/k RMSNorm -> NeoX RoPE -> cache -> causal GQA
attention -> O -> +x -> RMSNorm -> gate/up -> SwiGLU -> down -> +x.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Any, Mapping, Optional

from .plan import LayerPlan, ModelPlan, PartSpec, default_schedule
from .registry import Architecture, ConfigError, register_architecture

FULL = "full_attention"
SLIDING = "sliding_attention"


def _need_int(cfg: Mapping[str, Any], key: str, *, minimum: int = 1) -> int:
    if key not in cfg or cfg[key] is None:
        raise ConfigError(f"config.json lacks '{key}'")
    v = cfg[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"'{key}' must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"'{key}' must be >= {minimum}, got {v}")
    return v


def _float(cfg: Mapping[str, Any], key: str, default: float) -> float:
    v = cfg.get(key, default)
    if v is None:
        v = default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"'{key}' must be a number, got {v!r}")
    v = float(v)
    if not math.isfinite(v) or v <= 0.0:
        raise ConfigError(f"'{key}' must be positive and finite, got {v}")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float = 1.0e6
    rms_norm_eps: float = 1.0e-6
    tie_word_embeddings: bool = False
    sliding_window: Optional[int] = None
    layer_types: tuple[str, ...] = ()
    eos_token_ids: tuple[int, ...] = ()

    ARCHITECTURE = "Qwen3ForCausalLM"

    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "Qwen3Config":
        layers = _need_int(cfg, "num_hidden_layers")
        hidden = _need_int(cfg, "hidden_size")
        heads = _need_int(cfg, "num_attention_heads")
        kv_heads = _need_int(cfg, "num_key_value_heads")
        if cfg.get("head_dim") is None:
            if hidden % heads:
                raise ConfigError(
                    f"'head_dim' is absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}")
            head_dim = hidden // heads
        else:
            head_dim = _need_int(cfg, "head_dim")
        inter = _need_int(cfg, "intermediate_size")
        vocab = _need_int(cfg, "vocab_size")
        max_pos = _need_int(cfg, "max_position_embeddings")
        if heads % kv_heads:
            raise ConfigError(
                f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} must be even (rotation works on pairs)")

        # Options the reference does not have are refused, not ignored.
        if cfg.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"rope_scaling {cfg['rope_scaling']!r} is not supported")
        if cfg.get("attention_bias"):
            raise ConfigError("attention_bias is not supported (the projections have no bias)")
        if cfg.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {cfg['hidden_act']!r} is not supported (only 'silu')")
        tie = cfg.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise ConfigError(f"'tie_word_embeddings' must be true or false, got {tie!r}")

        window = cfg.get("sliding_window")
        layer_types = cfg.get("layer_types")
        if layer_types is None:
            if cfg.get("use_sliding_window"):
                raise ConfigError(
                    "use_sliding_window is set without 'layer_types'; list each layer as "
                    f"'{FULL}' or '{SLIDING}'")
            layer_types = [FULL] * layers
        if not isinstance(layer_types, (list, tuple)) or len(layer_types) != layers:
            raise ConfigError(f"'layer_types' must list {layers} entries")
        for i, t in enumerate(layer_types):
            if t not in (FULL, SLIDING):
                raise ConfigError(f"layer_types[{i}] = {t!r}; known: '{FULL}', '{SLIDING}'")
        if SLIDING in layer_types:
            if isinstance(window, bool) or not isinstance(window, int) or window < 1:
                raise ConfigError(
                    f"'{SLIDING}' layers need a positive integer 'sliding_window', got {window!r}")
        else:
            window = None
        eos = cfg.get("eos_token_id")
        if eos is None:
            eos = []
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos = [eos]
        if not isinstance(eos, (list, tuple)) or any(
                isinstance(e, bool) or not isinstance(e, int) or not 0 <= e < vocab for e in eos):
            raise ConfigError(f"'eos_token_id' must be token ids below vocab_size, got {eos!r}")
        return Qwen3Config(
            eos_token_ids=tuple(eos),
            num_hidden_layers=layers, hidden_size=hidden, num_attention_heads=heads,
            num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
            vocab_size=vocab, max_position_embeddings=max_pos,
            rope_theta=_float(cfg, "rope_theta", 1.0e6),
            rms_norm_eps=_float(cfg, "rms_norm_eps", 1.0e-6),
            tie_word_embeddings=tie, sliding_window=window, layer_types=tuple(layer_types))

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        d = asdict(self)
        d["layer_types"] = list(self.layer_types)
        d["eos_token_id"] = list(d.pop("eos_token_ids")) or None
        d["architectures"] = [self.ARCHITECTURE]
        d["model_type"] = "qwen3"
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        return d


def build_plan(cfg: Qwen3Config) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    position = PartSpec("rope_neox", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    layers = []
    for i in range(cfg.num_hidden_layers):
        window = cfg.sliding_window if cfg.layer_types[i] == SLIDING else None
        mixer = PartSpec("attention", {
            "hidden_size": cfg.hidden_size,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "qk_norm_eps": cfg.rms_norm_eps,
            "window": window,
            "position": position,
        })
        ffn = PartSpec("swiglu", {
            "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
        p = f"model.layers.{i}."
        layers.append(LayerPlan(
            block=PartSpec("prenorm"), mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm,
            names={"mixer": p + "self_attn.", "ffn": p + "mlp.",
                   "mixer_norm": p + "input_layernorm.",
                   "ffn_norm": p + "post_attention_layernorm."}))
    return ModelPlan(
        architecture=cfg.ARCHITECTURE,
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        layers=layers, schedule=default_schedule(cfg.num_hidden_layers),
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab_size,
                                         "hidden_size": cfg.hidden_size}),
        final_norm=norm,
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                  "tied": cfg.tie_word_embeddings}),
        names={"embedding": "model.embed_tokens.", "final_norm": "model.norm.",
               "head": "lm_head."})


def config_from_gguf(meta: Mapping[str, Any], shapes: Mapping[str, tuple]) -> dict[str, Any]:
    """The config.json dictionary that a GGUF file's metadata stands for.  Keys as the reference
    reads them (src/model.cpp:32-41); the vocabulary falls back to the embedding's row count
    (src/model.cpp:48-52); the head is tied iff the file has no ``output.weight``."""
    def need(key):
        if key not in meta:
            raise ConfigError(f"GGUF metadata lacks '{key}'")
        return meta[key]

    vocab = meta.get("qwen3.vocab_size") or (shapes.get("token_embd.weight") or (0,))[0]
    cfg = {
        "architectures": [Qwen3Config.ARCHITECTURE],
        "num_hidden_layers": need("qwen3.block_count"),
        "hidden_size": need("qwen3.embedding_length"),
        "intermediate_size": need("qwen3.feed_forward_length"),
        "num_attention_heads": need("qwen3.attention.head_count"),
        "num_key_value_heads": need("qwen3.attention.head_count_kv"),
        "head_dim": need("qwen3.attention.key_length"),
        "vocab_size": vocab,
        "rope_theta": meta.get("qwen3.rope.freq_base", 1.0e6),
        "rms_norm_eps": meta.get("qwen3.attention.layer_norm_rms_epsilon", 1.0e-6),
        "max_position_embeddings": need("qwen3.context_length"),
        "tie_word_embeddings": "output.weight" not in shapes,
    }
    eos = meta.get("tokenizer.ggml.eos_token_id")
    if eos is not None and 0 <= eos < vocab:
        cfg["eos_token_id"] = eos
    return cfg


_GGUF_LAYER = {
    "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
    "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
    "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight",
    "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight",
    "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
    "mlp.down_proj.weight": "ffn_down.weight",
}
_GGUF_GLOBAL = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
                "lm_head.weight": "output.weight"}


def gguf_tensor_name(name: str) -> str:
    """GGUF name of a checkpoint tensor (names as the reference loads them, src/model.cpp:120-149)."""
    if name in _GGUF_GLOBAL:
        return _GGUF_GLOBAL[name]
    parts = name.split(".", 3)                       # model.layers.<i>.<rest>
    if len(parts) == 4 and parts[:2] == ["model", "layers"] and parts[3] in _GGUF_LAYER:
        return f"blk.{parts[2]}.{_GGUF_LAYER[parts[3]]}"
    raise KeyError(name)


def gguf_metadata(cfg: Qwen3Config) -> dict[str, Any]:
    """The GGUF metadata that reads back as ``cfg`` (windowed layers have no GGUF keys here)."""
    if cfg.sliding_window is not None:
        raise ConfigError("windowed layers cannot be written to GGUF metadata")
    meta = {
        "general.architecture": "qwen3", "qwen3.block_count": cfg.num_hidden_layers,
        "qwen3.embedding_length": cfg.hidden_size, "qwen3.feed_forward_length": cfg.intermediate_size,
        "qwen3.attention.head_count": cfg.num_attention_heads,
        "qwen3.attention.head_count_kv": cfg.num_key_value_heads,
        "qwen3.attention.key_length": cfg.head_dim, "qwen3.vocab_size": cfg.vocab_size,
        "qwen3.rope.freq_base": float(cfg.rope_theta),
        "qwen3.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps),
        "qwen3.context_length": cfg.max_position_embeddings,
    }
    if cfg.eos_token_ids:
        meta["tokenizer.ggml.eos_token_id"] = cfg.eos_token_ids[0]
    return meta


register_architecture(Architecture(
    name=Qwen3Config.ARCHITECTURE, from_dict=Qwen3Config.from_dict, build_plan=build_plan,
    aliases=("qwen3",), config_from_gguf=config_from_gguf, gguf_tensor_name=gguf_tensor_name))
