"""The GGUF reader (the second loader): round trips, the reference's names and keys, errors."""
import os
import struct

import pytest
import torch

from plain_qwen3 import load_folder, plain_forward
from ref_ops import RefOps
from tinyinfer_b200 import Engine, StepEntry
from tinyinfer_b200.config import ConfigError, Qwen3Config
from tinyinfer_b200.config.qwen3 import gguf_metadata, gguf_tensor_name
from tinyinfer_b200.weights import GgufError, GgufFile, WeightsError, write_gguf
from util import assert_close_logits, make_model, random_tokens


def _to_gguf(tmp_path, name, drop=(), extra=None, version=3):
    d = make_model(tmp_path, name)
    cfg, w = load_folder(d)
    tensors = {gguf_tensor_name(n): t for n, t in w.items() if gguf_tensor_name(n) not in drop}
    if extra:
        tensors.update(extra)
    path = os.path.join(str(tmp_path), f"{name}.gguf")
    meta = gguf_metadata(Qwen3Config.from_dict(cfg))
    meta["tokenizer.ggml.tokens"] = ["a", "b", "c"]          # an array the loader has to skip over
    write_gguf(path, meta, tensors, version=version)
    return path, cfg, w


def test_names_follow_the_reference():
    assert gguf_tensor_name("model.embed_tokens.weight") == "token_embd.weight"
    assert gguf_tensor_name("model.norm.weight") == "output_norm.weight"
    assert gguf_tensor_name("lm_head.weight") == "output.weight"
    assert gguf_tensor_name("model.layers.12.self_attn.q_norm.weight") == "blk.12.attn_q_norm.weight"
    assert gguf_tensor_name("model.layers.3.mlp.down_proj.weight") == "blk.3.ffn_down.weight"


@pytest.mark.parametrize("version", [2, 3])
def test_file_round_trip(tmp_path, version):
    path, cfg, w = _to_gguf(tmp_path, "B", version=version)
    f = GgufFile(path)
    assert f.version == version and f.metadata["general.architecture"] == "qwen3"
    assert f.metadata["qwen3.attention.key_length"] == 32 and f.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"]
    assert abs(f.metadata["qwen3.attention.layer_norm_rms_epsilon"] - 1e-5) < 1e-12
    for n, t in w.items():
        g = gguf_tensor_name(n)
        assert f.shape(g) == tuple(t.shape) and f.dtype(g) == t.dtype and torch.equal(f.get(g), t)


@pytest.mark.parametrize("name", ["A", "B"])
def test_engine_loads_a_gguf_file_like_the_folder(tmp_path, name):
    path, cfg, w = _to_gguf(tmp_path, name)
    eng = Engine(path, dtype="float32", device="cpu", ops=RefOps(), max_tokens=128)
    assert eng.config.tie_word_embeddings == cfg["tie_word_embeddings"]       # tied iff no output.weight
    assert eng.config.max_position_embeddings == cfg["max_position_embeddings"]
    toks = random_tokens(cfg["vocab_size"], 30, seed=4)
    got = eng.step([StepEntry("a", toks, list(range(30)))])
    assert_close_logits(got, plain_forward(cfg, w, toks), 2e-5, f"gguf {name}")


def test_errors(tmp_path):
    path, cfg, _ = _to_gguf(tmp_path, "A", drop=("blk.1.ffn_up.weight",),
                            extra={"blk.0.attn_k.weight": torch.zeros(8, 64, dtype=torch.bfloat16),
                                   "rope_freqs.weight": torch.zeros(4)})
    with pytest.raises(WeightsError) as info:
        Engine(path, dtype="float32", device="cpu", ops=RefOps())
    e = info.value
    assert e.missing == ["blk.1.ffn_up.weight"] and e.unexpected == ["rope_freqs.weight"]
    assert [n for n, _, _ in e.wrong_shape] == ["blk.0.attn_k.weight"]
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 40)
    with pytest.raises(GgufError, match="magic"):
        GgufFile(str(bad))
    bad.write_bytes(b"GGUF" + struct.pack("<IQQ", 1, 0, 0))
    with pytest.raises(GgufError, match="version 1"):
        GgufFile(str(bad))
    bad.write_bytes(b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 99))
    with pytest.raises(GgufError, match="value type 99"):
        GgufFile(str(bad))
    write_gguf(str(bad), {"general.architecture": "llama"}, {})
    with pytest.raises(ConfigError, match="unknown architecture 'llama'"):
        Engine(str(bad), dtype="float32", device="cpu", ops=RefOps())
    write_gguf(str(bad), {"general.architecture": "qwen3", "qwen3.block_count": 2}, {})
    with pytest.raises(ConfigError, match="qwen3.embedding_length"):
        Engine(str(bad), dtype="float32", device="cpu", ops=RefOps())
    with pytest.raises(GgufError, match="cannot open"):
        GgufFile(str(tmp_path / "none.gguf"))
