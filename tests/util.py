"""Tiny configurations, model folders and comparisons shared by the tests."""
from __future__ import annotations

import os

import torch

from tinyinfer_b200 import write_random_model

ARCH = ["Qwen3ForCausalLM"]

# Two tiny configurations that differ in every size and option, and a third with
# windowed layers, a head size that is no power of two and one kv head.
TINY_A = dict(architectures=ARCH, num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=128)
TINY_B = dict(architectures=ARCH, num_hidden_layers=3, hidden_size=96, num_attention_heads=8,
              num_key_value_heads=2, head_dim=32, intermediate_size=224, vocab_size=512,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=256)
TINY_C = dict(architectures=ARCH, num_hidden_layers=4, hidden_size=80, num_attention_heads=3,
              num_key_value_heads=1, head_dim=48, intermediate_size=176, vocab_size=331,
              rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
              max_position_embeddings=512, sliding_window=24,
              layer_types=["full_attention", "sliding_attention", "sliding_attention",
                           "full_attention"])
# sizes that the tensor-core kernels of the bfloat16 path take (head size 64, widths that are
# multiples of 32), with one windowed layer
TINY_D = dict(architectures=ARCH, num_hidden_layers=3, hidden_size=128, num_attention_heads=8,
              num_key_value_heads=2, head_dim=64, intermediate_size=320, vocab_size=1008,
              rope_theta=200000.0, rms_norm_eps=2e-6, tie_word_embeddings=True,
              max_position_embeddings=1024, sliding_window=40,
              layer_types=["full_attention", "sliding_attention", "full_attention"])
# head size 128: prompts of more than 64 tokens take the tcgen05 products (with the QKV epilogue)
# and the tcgen05 attention
TINY_E = dict(architectures=ARCH, num_hidden_layers=2, hidden_size=192, num_attention_heads=3,
              num_key_value_heads=1, head_dim=128, intermediate_size=272, vocab_size=777,
              rope_theta=300000.0, rms_norm_eps=4e-6, tie_word_embeddings=False,
              max_position_embeddings=640)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}

FP32_RTOL = 2e-5      # of the largest reference logit: float32 engine against float64 plain
BF16_RTOL = 2e-2      # bfloat16 engine against plain with the reference's rounding points


def make_model(tmp_path, name: str, seed: int = 7, dtype=None) -> str:
    d = os.path.join(str(tmp_path), f"tiny_{name}_{seed}")
    if not os.path.isdir(d):
        write_random_model(d, TINY[name], seed=seed, dtype=dtype)
    return d


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def assert_close_logits(got: torch.Tensor, ref: torch.Tensor, rtol: float, what: str = "") -> float:
    """max |got - ref| <= rtol * max |ref|; returns the error as a fraction of max |ref|."""
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = ref.abs().max().item()
    err = (got - ref).abs().max().item()
    if err > rtol * scale:
        bad = (got - ref).abs().max(dim=-1).values
        first = int((bad > rtol * scale).nonzero()[0])
        raise AssertionError(
            f"{what}: max error {err:.3e} exceeds {rtol:g} x {scale:.3e}; first wrong row "
            f"{first} of {got.shape[0]} (error {bad[first]:.3e})")
    return err / scale
