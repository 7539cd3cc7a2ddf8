"""The command line's byte-level BPE tokenizer: its own properties, and, where g++ and the
reference's sources are at hand, the same ids as the reference's tokenizer (src/tokenizer.cpp,
compiled as it stands) on a small vocabulary trained here."""
import collections
import json
import os
import shutil
import subprocess

import pytest

from tinyinfer_b200.tokenizer import (TOKEN_CONTROL, TOKEN_NORMAL, Tokenizer, byte_table, chat_wrap)
from tinyinfer_b200.weights import write_gguf

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("TINYINFER_REFERENCE", os.path.join(os.path.dirname(HERE), "baseline", "_ref", "src"))

CORPUS = ("the quick brown fox jumps over the lazy dog. The dog didn't mind; it's the fox's habit!\n"
          "numbers 12345 and 3.14159, tabs\tand  double  spaces, CamelCase and snake_case words\n"
          "naïve café résumé über straße — 日本語のテキスト と 中文文本 그리고 한국어\n"
          "def f(x):\n    return x ** 2  # comment\n\n\nthe the the quick quick fox fox dog dog jumps\n") * 3
LINES = ["hello world", "The fox didn't jump; it's lazy!", "  leading and trailing  ", "12345 + 67890 = 80235",
         "naïve café — 日本語 と 中文", "line one\nline two\n\n\nline five", "tab\tseparated\tvalues", "x",
         "", "snake_case CamelCase UPPER lower", "a'b're'LL'd 's", "emoji 🙂 and symbols ©®™ ±×÷",
         "trailing spaces   \n   next", "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"]


def _train(corpus: str, merges: int):
    """A small byte-level BPE vocabulary: the 256 byte characters, then `merges` merges of the
    most frequent neighbouring pairs over the corpus's words."""
    tab = byte_table()
    tok = Tokenizer([tab[b] for b in range(256)])
    words = collections.Counter(tuple(tab[b] for b in w.encode("utf-8")) for w in tok._split(corpus))
    rules = []
    for _ in range(merges):
        pairs = collections.Counter()
        for w, n in words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] += n
        if not pairs:
            break
        (a, b), _ = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        rules.append(f"{a} {b}")
        merged = collections.Counter()
        for w, n in words.items():
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            merged[tuple(out)] += n
        words = merged
    tokens = [tab[b] for b in range(256)] + [r.replace(" ", "") for r in rules]
    types = [TOKEN_NORMAL] * len(tokens)
    for sp in ("<|im_start|>", "<|im_end|>", "<|endoftext|>"):
        tokens.append(sp)
        types.append(TOKEN_CONTROL)
    return tokens, types, rules


@pytest.fixture(scope="module")
def trained():
    tokens, types, rules = _train(CORPUS, 300)
    return tokens, types, rules, Tokenizer(tokens, types, rules, eos_token_id=len(tokens) - 1)


def test_round_trip_and_merges(trained):
    tokens, types, rules, tok = trained
    for text in LINES + [CORPUS]:
        ids = tok.encode(text)
        assert tok.decode(ids) == text
        assert all(0 <= i < len(tokens) for i in ids)
    # merges shorten: a trained word is fewer tokens than its bytes, an unseen script is its bytes
    assert len(tok.encode("the quick brown fox")) < len("the quick brown fox".encode()) // 2
    assert len(tok.encode("ъ")) == 2
    # special tokens are spelt unless asked for
    spelt = tok.encode("<|im_start|>user")
    parsed = tok.encode("<|im_start|>user", parse_special=True)
    assert parsed[0] == tokens.index("<|im_start|>") and len(parsed) < len(spelt)
    assert tok.decode(parsed) == "<|im_start|>user" and tok.decode(parsed, special=False) == "user"
    assert tok.is_eog(len(tokens) - 1) and not tok.is_eog(0)
    assert chat_wrap("hi").startswith("<|im_start|>user\nhi<|im_end|>") and "<think>\n\n</think>" in chat_wrap("hi")


def test_tokenizer_json_and_gguf_sources(tmp_path, trained):
    tokens, types, rules, tok = trained
    folder = tmp_path / "model"
    folder.mkdir()
    vocab = {t: i for i, t in enumerate(tokens) if types[i] == TOKEN_NORMAL}
    added = [{"id": i, "content": t, "special": True} for i, t in enumerate(tokens) if types[i] == TOKEN_CONTROL]
    (folder / "tokenizer.json").write_text(json.dumps(
        {"model": {"type": "BPE", "vocab": vocab, "merges": [r.split(" ") for r in rules]}, "added_tokens": added}))
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [len(tokens) - 1, 7]}))
    from_json = Tokenizer.for_model(str(folder))
    gguf = str(tmp_path / "tok.gguf")
    write_gguf(gguf, {"general.architecture": "qwen3", "tokenizer.ggml.tokens": tokens,
                      "tokenizer.ggml.token_type": types, "tokenizer.ggml.merges": rules,
                      "tokenizer.ggml.eos_token_id": len(tokens) - 1}, {})
    from_gguf = Tokenizer.for_model(gguf)
    for text in LINES:
        want = tok.encode(text, parse_special=True)
        assert from_json.encode(text, parse_special=True) == want
        assert from_gguf.encode(text, parse_special=True) == want
    assert from_json.eos_token_id == from_gguf.eos_token_id == len(tokens) - 1
    assert Tokenizer.for_model(str(tmp_path)) is None


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isfile(os.path.join(REFERENCE, "src", "tokenizer.cpp")),
                    reason="needs g++ and the reference's sources")
@pytest.mark.parametrize("special", [False, True])
def test_same_ids_as_the_reference_tokenizer(tmp_path, trained, special):
    """src/tokenizer.cpp and src/gguf_reader.cpp compiled as they stand, fed the same vocabulary
    through a GGUF file."""
    tokens, types, rules, tok = trained
    exe = str(tmp_path / "tokenize_reference")
    src = os.path.join(REFERENCE, "src")
    subprocess.run(["g++", "-std=c++17", "-O1", "-w", "-I", src, os.path.join(HERE, "golden", "tokenize_reference.cpp"),
                    os.path.join(src, "tokenizer.cpp"), os.path.join(src, "gguf_reader.cpp"), "-o", exe],
                   check=True, timeout=600)
    gguf = str(tmp_path / "tok.gguf")
    write_gguf(gguf, {"general.architecture": "qwen3", "tokenizer.ggml.tokens": tokens,
                      "tokenizer.ggml.token_type": types, "tokenizer.ggml.merges": rules}, {})
    lines = [l for l in LINES + CORPUS.split("\n")[:4] if l]
    with open(tmp_path / "lines.txt", "w", encoding="utf-8") as fh:
        for l in lines:
            fh.write(l.replace("\\", "\\\\").replace("\n", "\\n") + "\n")
    out = subprocess.run([exe, gguf, str(tmp_path / "lines.txt")] + (["--special"] if special else []),
                         capture_output=True, text=True, check=True, timeout=120).stdout.splitlines()
    assert len(out) == len(lines)
    for text, row in zip(lines, out):
        ids_text, verdict = row.split("\t")
        theirs = [int(x) for x in ids_text.split()] if ids_text else []
        mine = tok.encode(text, parse_special=special)
        if special:
            # The reference emits the ids of all special tokens it cut the text at first and the
            # tokens of the text between them afterwards (src/tokenizer.cpp:396-427 pushes a
            # special's id while scanning, the fragments are tokenized after the scan).  Here
            # they come in the order of the text; the two lists hold the same ids.
            control = {i for i, t in enumerate(types) if t == TOKEN_CONTROL}
            assert [i for i in mine if i in control] + [i for i in mine if i not in control] == theirs, text
        else:
            assert mine == theirs, text
            assert verdict == "round-trip"
