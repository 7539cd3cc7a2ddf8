"""Byte-level BPE tokenizer of the Qwen family, for the command line.

The engine itself works on token ids.  The command line turns text into ids with this
tokenizer when the model brings one: a GGUF file's ``tokenizer.ggml.tokens`` / ``token_type`` /
``merges`` / ``eos_token_id`` (what the reference reads, src/main.cpp:167-171), or a model
folder's ``tokenizer.json`` (``model.vocab``, ``model.merges``, ``added_tokens``).

The method is the reference's (src/tokenizer.cpp:390-542): optionally cut the text at special
tokens; split each piece with the Qwen2 pattern; write every UTF-8 byte of a word as one
printable character (the GPT-2 byte table); merge neighbouring symbols in the order of the
merge ranks, lowest rank first and leftmost among equals; look the symbols up, falling back to
one token per byte.  Decoding maps a normal token's characters back to bytes, leaves control and
user-defined tokens as they are written, and reads ``<0xXX>`` byte tokens
(src/tokenizer.cpp:545-575).
"""
from __future__ import annotations

import heapq
import json
import os
from typing import Iterable, Mapping, Optional, Sequence

TOKEN_NORMAL, TOKEN_UNKNOWN, TOKEN_CONTROL, TOKEN_USER_DEFINED, TOKEN_UNUSED, TOKEN_BYTE = 1, 2, 3, 4, 5, 6

# the split pattern of the Qwen2 pre-tokenizer (src/tokenizer.cpp:247-253 states it)
QWEN2_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*"
                 r"|\s*[\r\n]+|\s+(?!\S)|\s+")


class TokenizerError(ValueError):
    pass


def byte_table() -> dict[int, str]:
    """Byte -> printable character: bytes that print stay themselves, the others are moved to
    code points from 256 on (the table GPT-2 introduced; src/tokenizer.cpp builds the same)."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


class Tokenizer:
    def __init__(self, tokens: Sequence[str], token_types: Optional[Sequence[int]] = None,
                 merges: Iterable[str] = (), eos_token_id: Optional[int] = None):
        self.tokens = list(tokens)
        self.types = list(token_types) if token_types else [TOKEN_NORMAL] * len(self.tokens)
        if len(self.types) != len(self.tokens):
            raise TokenizerError(f"{len(self.tokens)} tokens but {len(self.types)} token types")
        self.token_to_id = {t: i for i, t in enumerate(self.tokens)}
        self.ranks: dict[tuple[str, str], int] = {}
        for i, line in enumerate(merges):
            cut = line.find(" ", 1)
            if cut > 0:
                self.ranks[(line[:cut], line[cut + 1:])] = i
        self.eos_token_id = eos_token_id
        self._byte_to_char = byte_table()
        self._char_to_byte = {c: b for b, c in self._byte_to_char.items()}
        # what parse_special cuts the text at: control and unknown tokens as in the reference
        # (src/tokenizer.h:44-48), and user-defined ones (added tokens of a tokenizer.json)
        self._specials = [(t, i) for i, t in enumerate(self.tokens)
                          if t and self.types[i] in (TOKEN_UNKNOWN, TOKEN_CONTROL, TOKEN_USER_DEFINED)]
        self._pattern = None

    # ---- loading -------------------------------------------------------------------------
    @classmethod
    def from_gguf_metadata(cls, metadata: Mapping) -> Optional["Tokenizer"]:
        """From a GGUF file's metadata; None if the file carries no tokenizer."""
        tokens = metadata.get("tokenizer.ggml.tokens")
        if not tokens:
            return None
        eos = metadata.get("tokenizer.ggml.eos_token_id")
        return cls(tokens, metadata.get("tokenizer.ggml.token_type"), metadata.get("tokenizer.ggml.merges") or (),
                   None if eos is None else int(eos))

    @classmethod
    def from_tokenizer_json(cls, path: str) -> "Tokenizer":
        with open(path, "r", encoding="utf-8") as fh:
            data = json.load(fh)
        model = data.get("model") or {}
        vocab = model.get("vocab")
        if not isinstance(vocab, dict):
            raise TokenizerError(f"{path}: no 'model.vocab' table (only byte-level BPE files are read)")
        size = max(vocab.values(), default=-1) + 1
        added = data.get("added_tokens") or []
        size = max([size] + [int(a["id"]) + 1 for a in added])
        tokens = [""] * size
        types = [TOKEN_UNUSED] * size
        for text, idx in vocab.items():
            tokens[idx], types[idx] = text, TOKEN_NORMAL
        for a in added:
            tokens[int(a["id"])] = a["content"]
            types[int(a["id"])] = TOKEN_CONTROL if a.get("special") else TOKEN_USER_DEFINED
        merges = [m if isinstance(m, str) else " ".join(m) for m in model.get("merges") or []]
        eos = None
        cfg = os.path.join(os.path.dirname(path), "generation_config.json")
        if os.path.isfile(cfg):
            with open(cfg, "r", encoding="utf-8") as fh:
                e = json.load(fh).get("eos_token_id")
            eos = e[0] if isinstance(e, list) and e else e if isinstance(e, int) else None
        return cls(tokens, types, merges, eos)

    @classmethod
    def for_model(cls, model_path: str) -> Optional["Tokenizer"]:
        """The tokenizer a model brings (a ``.gguf`` file's metadata, a folder's
        ``tokenizer.json``), or None."""
        if os.path.isfile(model_path):
            from .weights.gguf import GgufFile
            f = GgufFile(model_path)
            try:
                return cls.from_gguf_metadata(f.metadata)
            finally:
                f.close()
        path = os.path.join(model_path, "tokenizer.json")
        return cls.from_tokenizer_json(path) if os.path.isfile(path) else None

    # ---- text -> ids ---------------------------------------------------------------------
    def _split(self, text: str) -> list[str]:
        if self._pattern is None:
            try:
                import regex
            except ImportError:
                raise TokenizerError("the 'regex' package is needed to split text (Unicode classes)") from None
            self._pattern = regex.compile(QWEN2_PATTERN)
        return self._pattern.findall(text)

    def _merge(self, word: str) -> list[str]:
        """A word (already in byte characters) cut into the symbols the merges leave."""
        n = len(word)
        if n < 2:
            return [word] if word else []
        text = list(word)                       # symbol i's text; "" once merged into its left neighbour
        prev = list(range(-1, n - 1))
        nxt = list(range(1, n)) + [-1]
        heap: list[tuple[int, int, int, str]] = []

        def push(left: int, right: int) -> None:
            if left < 0 or right < 0:
                return
            rank = self.ranks.get((text[left], text[right]))
            if rank is not None:
                heapq.heappush(heap, (rank, left, right, text[left] + text[right]))

        for i in range(1, n):
            push(i - 1, i)
        while heap:
            _, left, right, joined = heapq.heappop(heap)
            if not text[left] or not text[right] or text[left] + text[right] != joined:
                continue                                        # one of the two has changed since
            text[left] = joined
            text[right] = ""
            nxt[left] = nxt[right]
            if nxt[right] >= 0:
                prev[nxt[right]] = left
            push(prev[left], left)
            push(left, nxt[left])
        return [t for t in text if t]

    def encode(self, text: str, parse_special: bool = False) -> list[int]:
        """Token ids of ``text``.  With ``parse_special`` control and user-defined tokens written
        out in the text (``<|im_start|>``) become their ids instead of being spelt."""
        pieces: list[tuple[Optional[int], str]] = []
        if parse_special and self._specials:
            rest = text
            while rest:
                best = None
                for tok, idx in self._specials:
                    at = rest.find(tok)
                    if at >= 0 and (best is None or at < best[0] or (at == best[0] and len(tok) > len(best[1]))):
                        best = (at, tok, idx)
                if best is None:
                    pieces.append((None, rest))
                    break
                if best[0] > 0:
                    pieces.append((None, rest[:best[0]]))
                pieces.append((best[2], best[1]))
                rest = rest[best[0] + len(best[1]):]
        else:
            pieces.append((None, text))
        out: list[int] = []
        for special, piece in pieces:
            if special is not None:
                out.append(special)
                continue
            for word in self._split(piece):
                chars = "".join(self._byte_to_char[b] for b in word.encode("utf-8"))
                for sym in self._merge(chars):
                    idx = self.token_to_id.get(sym)
                    if idx is not None:
                        out.append(idx)
                    else:                                       # one token per byte character
                        out.extend(self.token_to_id[c] for c in sym if c in self.token_to_id)
        return out

    # ---- ids -> text ---------------------------------------------------------------------
    def piece(self, idx: int, special: bool = True) -> bytes:
        if not 0 <= idx < len(self.tokens):
            return b""
        text, kind = self.tokens[idx], self.types[idx]
        if kind in (TOKEN_UNKNOWN, TOKEN_CONTROL):
            return text.encode("utf-8") if special else b""
        if kind == TOKEN_USER_DEFINED:
            return text.encode("utf-8")
        if kind == TOKEN_NORMAL:
            out = bytearray()
            for c in text:
                b = self._char_to_byte.get(c)
                out += bytes([b]) if b is not None else c.encode("utf-8")
            return bytes(out)
        if kind == TOKEN_BYTE and len(text) == 6 and text.startswith("<0x") and text.endswith(">"):
            return bytes([int(text[3:5], 16)])
        return b""

    def decode(self, ids: Iterable[int], special: bool = True) -> str:
        return b"".join(self.piece(int(i), special) for i in ids).decode("utf-8", errors="replace")

    def is_eog(self, idx: int) -> bool:
        return self.eos_token_id is not None and idx == self.eos_token_id


def chat_wrap(text: str) -> str:
    """The Qwen3 chat form with an empty think block, as the reference writes it (src/main.cpp:188-193)."""
    return "<|im_start|>user\n" + text + "<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n"
