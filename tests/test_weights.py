"""Weights by tensor name: storage dtypes, one clear error, the random-weights mode."""
import json
import os

import pytest
import torch

from plain_qwen3 import load_folder
from tinyinfer_b200.config import get_architecture
from tinyinfer_b200.parts import CausalLM
from tinyinfer_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError,
                                    load_model_weights, storage_dtype, write_random_model,
                                    write_safetensors)
from ref_ops import RefOps
from util import TINY_A, TINY_B, make_model


def _model(cfg):
    arch = get_architecture("qwen3")
    return CausalLM(arch.build_plan(arch.from_dict(cfg)))


def test_writer_and_reader_agree_with_the_safetensors_library(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32),
               "c.d": torch.randn(2, 2, 2), "e": torch.zeros(0, 4)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, metadata={"k": "v"})
    from safetensors.torch import load_file
    lib = load_file(path)
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(tensors) and f.metadata == {"k": "v"}
    for n, t in tensors.items():
        assert torch.equal(lib[n], t) and torch.equal(f.get(n), t)
        assert f.dtype(n) == t.dtype and f.shape(n) == tuple(t.shape)


def test_reader_errors(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x05")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile(str(tmp_path / "none.safetensors"))


def test_random_model_folder(tmp_path):
    d = make_model(tmp_path, "B", seed=3)
    cfg, w = load_folder(d)
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["head_dim"] == 32
    expected = _model(TINY_B).expected_tensors()
    assert set(w) == set(expected) and "lm_head.weight" in w
    assert w["model.layers.1.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert w["model.layers.1.self_attn.q_norm.weight"].dtype == torch.float32
    # matrices N(0, 0.02), norm weights 1 + N(0, 0.02)
    m = w["model.embed_tokens.weight"].float()
    assert abs(m.std().item() - 0.02) < 0.002 and abs(m.mean().item()) < 0.002
    n = torch.cat([v.float().flatten() for k, v in w.items() if "norm" in k])
    assert abs(n.mean().item() - 1.0) < 0.01 and abs(n.std().item() - 0.02) < 0.005
    # the same seed gives the same bits, another seed does not; tied models store no head
    d2 = str(tmp_path / "again")
    write_random_model(d2, TINY_B, seed=3)
    assert all(torch.equal(w[k], load_folder(d2)[1][k]) for k in w)
    d3 = str(tmp_path / "other")
    write_random_model(d3, TINY_B, seed=4)
    assert not torch.equal(w["model.norm.weight"], load_folder(d3)[1]["model.norm.weight"])
    assert "lm_head.weight" not in load_folder(make_model(tmp_path, "A"))[1]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model(tmp_path, "A", seed=5)
    _, w = load_folder(d)
    w = dict(w)
    del w["model.layers.0.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    w["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(8)
    w["lm_head.weight"] = torch.zeros(255, 64, dtype=torch.bfloat16)      # tied: allowed, but of the table's shape
    w["model.layers.9.extra"] = torch.zeros(1)
    write_safetensors(os.path.join(d, "model.safetensors"), w)
    with pytest.raises(WeightsError) as info:
        load_model_weights(_model(TINY_A), d, "cpu", RefOps())
    e = info.value
    assert e.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.9.extra"]
    assert [(n, tuple(a), tuple(b)) for n, a, b in e.wrong_shape] == [
        ("lm_head.weight", (256, 64), (255, 64)),
        ("model.layers.0.self_attn.q_norm.weight", (16,), (8,)),
        ("model.layers.1.self_attn.k_proj.weight", (32, 64), (16, 64))]
    text = str(e)
    for piece in ("missing (2)", "unexpected (1)", "wrong shape (3)", "expected [32, 64] found [16, 64]"):
        assert piece in text


def test_tied_checkpoint_may_store_the_head_again(tmp_path):
    """A folder with tied embeddings that also holds ``lm_head.weight`` loads; the embedding's
    table is the one used, and a copy with other values is reported, not followed.  An untied
    model still refuses a tensor it does not know."""
    import warnings
    d = make_model(tmp_path, "A", seed=6)
    _, w = load_folder(d)
    w = dict(w)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), w)
    model = _model(TINY_A)
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        load_model_weights(model, d, "cpu", RefOps())
    assert model.head.table is model.embedding.table
    assert torch.equal(model.embedding.table, w["model.embed_tokens.weight"])
    w["lm_head.weight"] = torch.zeros_like(w["model.embed_tokens.weight"])
    write_safetensors(os.path.join(d, "model.safetensors"), w)
    model = _model(TINY_A)
    with pytest.warns(UserWarning, match="lm_head.weight is stored beside model.embed_tokens.weight"):
        load_model_weights(model, d, "cpu", RefOps())
    assert torch.equal(model.head.table, w["model.embed_tokens.weight"])
    db = make_model(tmp_path, "B", seed=6)
    _, wb = load_folder(db)
    wb = dict(wb)
    wb["model.embed_tokens.copy"] = wb["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(db, "model.safetensors"), wb)
    with pytest.raises(WeightsError) as info:
        load_model_weights(_model(TINY_B), db, "cpu", RefOps())
    assert info.value.unexpected == ["model.embed_tokens.copy"]


def test_storage_precision_is_never_narrowed(tmp_path):
    assert storage_dtype(torch.bfloat16) == torch.bfloat16
    assert storage_dtype(torch.float32) == torch.float32
    assert storage_dtype(torch.float16) == torch.float32
    assert storage_dtype(torch.float64) == torch.float32
    assert storage_dtype(torch.int64) == torch.int32
    d = str(tmp_path / "f32")
    write_random_model(d, TINY_A, seed=1, dtype=torch.float32)
    model = _model(TINY_A)
    load_model_weights(model, d, "cpu", RefOps())
    assert model.blocks[0].mixer.w_qkv.dtype == torch.float32       # stored in 32-bit: stays so
    assert model.blocks[0].mixer.w_qkv.shape == (64 + 2 * 32, 64)
    model_b = _model(TINY_A)
    load_model_weights(model_b, make_model(tmp_path, "A", seed=1), "cpu", RefOps())
    assert model_b.blocks[0].mixer.w_qkv.dtype == torch.bfloat16    # kept in bfloat16
    assert model_b.final_norm.weight.dtype == torch.float32
    assert model_b.head.table is model_b.embedding.table            # tied head aliases the table


def test_no_safetensors_file(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        load_model_weights(_model(TINY_A), str(tmp_path), "cpu", RefOps())


def test_random_weights_are_a_function_of_seed_name_and_index():
    """The generator is counter-based: pieces of a stream equal the stream, a tensor does not
    depend on the others, and the values are close to a normal distribution."""
    from tinyinfer_b200.parts.base import MATRIX, NORM_WEIGHT, WeightSpec
    from tinyinfer_b200.weights.random_init import random_tensor, standard_normal
    whole = standard_normal(99, 0, 5000)
    assert torch.equal(standard_normal(99, 1234, 700), whole[1234:1934])
    assert not torch.equal(standard_normal(98, 0, 5000), whole)
    big = standard_normal(7, 0, 1 << 20)
    assert abs(big.mean().item()) < 5e-3 and abs(big.std().item() - 1.0) < 5e-3
    assert 2.8 < (big ** 4).mean().item() < 3.1 and big.abs().max().item() <= 6.0
    spec = WeightSpec((33, 17), MATRIX)
    a = random_tensor(5, "x.weight", spec)
    assert a.dtype == torch.bfloat16 and tuple(a.shape) == (33, 17)
    assert torch.equal(a, random_tensor(5, "x.weight", spec))
    assert not torch.equal(a, random_tensor(5, "y.weight", spec))
    assert not torch.equal(a, random_tensor(6, "x.weight", spec))
    # the bfloat16 tensor is the rounded float32 draw
    assert torch.equal(a, random_tensor(5, "x.weight", spec, dtype=torch.float32).to(torch.bfloat16))
    n = random_tensor(5, "n.weight", WeightSpec((64,), NORM_WEIGHT))
    assert n.dtype == torch.float32 and abs(n.mean().item() - 1.0) < 0.02
