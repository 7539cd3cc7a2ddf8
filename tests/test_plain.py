"""The plain implementation itself: each part against properties that follow from its formula."""
import math

import torch

from plain_qwen3 import (load_folder, plain_attention, plain_forward, plain_greedy, plain_rmsnorm,
                         plain_rope_angles, plain_rope_neox, plain_swiglu)
from util import make_model, random_tokens


def test_rmsnorm_formula():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    # mean square 12.5; eps inside the root; weight multiplies directly
    want = x.double() / math.sqrt(12.5 + 0.5) * w.double()
    assert torch.allclose(plain_rmsnorm(x, w, 0.5), want, atol=1e-12)


def test_rope_is_a_rotation_by_pos_times_inv_freq():
    hd, theta = 8, 100.0
    pos = torch.tensor([0, 1, 7])
    ang = plain_rope_angles(pos, hd, theta)
    assert ang.dtype == torch.float32 and ang.shape == (3, 4)
    assert torch.allclose(ang[1].double(), torch.tensor([100.0 ** (-2 * k / hd) for k in range(4)],
                                                        dtype=torch.float64), atol=1e-7)
    x = torch.randn(3, 2, hd, dtype=torch.float64)
    y = plain_rope_neox(x, ang)
    assert torch.equal(y[0], x[0])                                   # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))            # lengths are kept
    # pair (k, k + hd/2) turns by the angle
    k = 1
    a = ang[2, k].double()
    assert torch.allclose(y[2, 0, k], x[2, 0, k] * torch.cos(a) - x[2, 0, k + 4] * torch.sin(a))
    assert torch.allclose(y[2, 0, k + 4], x[2, 0, k] * torch.sin(a) + x[2, 0, k + 4] * torch.cos(a))
    # scores depend on the distance only
    q, kk = torch.randn(1, 1, hd, dtype=torch.float64), torch.randn(1, 1, hd, dtype=torch.float64)
    def score(pq, pk):
        return (plain_rope_neox(q, plain_rope_angles(torch.tensor([pq]), hd, theta)) *
                plain_rope_neox(kk, plain_rope_angles(torch.tensor([pk]), hd, theta))).sum()
    assert torch.allclose(score(5, 2), score(13, 10), atol=1e-5)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    s, heads, kv, hd = 12, 4, 2, 8
    q = torch.randn(s, heads, hd, dtype=torch.float64)
    k = torch.randn(s, kv, hd, dtype=torch.float64)
    v = torch.randn(s, kv, hd, dtype=torch.float64)
    out = plain_attention(q, k, v, 0.3)
    assert torch.allclose(out[0], v[0].repeat_interleave(2, dim=0))  # first token sees itself only
    k2, v2 = k.clone(), v.clone()
    k2[7:], v2[7:] = 9.0, -9.0                                        # the future does not matter
    assert torch.equal(plain_attention(q, k2, v2, 0.3)[:7], out[:7])
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    v3 = v.clone()
    v3[:, 1] += 1.0
    d = plain_attention(q, k, v3, 0.3) - out
    assert d[:, :2].abs().max() == 0 and torch.allclose(d[:, 2:], torch.ones_like(d[:, 2:]))
    # a window of w: position t sees exactly t-w+1 .. t
    w = 3
    outw = plain_attention(q, k, v, 0.3, window=w)
    t = 9
    sc = (q[t, 0] @ k[t - w + 1:t + 1, 0].T) * 0.3
    assert torch.allclose(outw[t, 0], torch.softmax(sc, -1) @ v[t - w + 1:t + 1, 0])
    assert torch.allclose(plain_attention(q, k, v, 0.3, window=s), out)


def test_swiglu():
    g, u = torch.tensor([0.0, 2.0, -3.0], dtype=torch.float64), torch.tensor([5.0, 1.0, 2.0], dtype=torch.float64)
    want = torch.tensor([0.0, 2.0 / (1 + math.exp(-2.0)), -3.0 / (1 + math.exp(3.0)) * 2.0])
    assert torch.allclose(plain_swiglu(g, u), want.double())


def test_forward_is_causal_and_rounding_is_small(tmp_path):
    for name in ("A", "C"):
        cfg, w = load_folder(make_model(tmp_path, name))
        toks = random_tokens(cfg["vocab_size"], 40, seed=1)
        full = plain_forward(cfg, w, toks)
        assert full.shape == (40, cfg["vocab_size"]) and full.dtype == torch.float64
        assert torch.allclose(plain_forward(cfg, w, toks[:25]), full[:25], atol=1e-12)
        rounded = plain_forward(cfg, w, toks, emulate_bf16=True)
        rel = (rounded - full).abs().max() / full.abs().max()
        assert 1e-5 < rel < 3e-2                                      # bfloat16 rounding, no more


def test_greedy_takes_the_first_maximum(tmp_path):
    cfg, w = load_folder(make_model(tmp_path, "B"))
    prompt = random_tokens(cfg["vocab_size"], 6, seed=2)
    out = plain_greedy(cfg, w, prompt, 3)
    seq = list(prompt)
    for tok in out:
        assert tok == int(plain_forward(cfg, w, seq)[-1].argmax())
        seq.append(tok)
