"""Tokenizers (zml/tokenizer/* of the reference): one front `Tokenizer` over three back-ends.

* `hf`            - HF `tokenizer.json` through the `tokenizers` library when it is installed
                    (the reference uses the IREE tokenizer, patched to match HF);
* `sentencepiece` - `.model` / `.pb` files through the `sentencepiece` package (the
                    reference wraps the C++ library with SWIG);
* `homemade`      - the in-house tokenizers (no dependency): BPE (`zml_b200.tokenizer.bpe`) and Unigram
                    (`zml_b200.tokenizer.unigram`), chosen by the `model.type` of the tokenizer.json.

`Tokenizer.encoder()` / `.decoder()` give the reference's stateful objects: the decoder is
a streaming one (`next(id)` returns the text that became printable with that id, holding
back incomplete UTF-8 sequences).
"""
from __future__ import annotations

import os
from typing import Iterable, Optional

from .bpe import BpeTokenizer


class Encoder:
    def __init__(self, tok: "Tokenizer"):
        self.tok = tok
        self._ids: list[int] = []

    def reset(self) -> None:
        self._ids = []

    def encode(self, text: str) -> list[int]:
        self._ids = self.tok.encode(text)
        return self._ids

    encode_alloc = encode

    def append_tokens(self, out: list, tokens: Iterable[int]) -> None:
        out.extend(int(t) for t in tokens)


class Decoder:
    """Streaming decoder: feed ids one at a time, get printable text chunks back."""

    def __init__(self, tok: "Tokenizer"):
        self.tok = tok
        self._pending = b""
        self._ids: list[int] = []
        self._printed = 0

    def reset(self) -> None:
        self._pending, self._ids, self._printed = b"", [], 0

    def decode(self, ids: Iterable[int]) -> str:
        return self.tok.decode(list(ids))

    decode_alloc = decode

    def next(self, token_id: int) -> str:
        if self.tok.backend == "homemade":
            self._pending += self.tok.impl.token_bytes(int(token_id))
            # emit the longest valid UTF-8 prefix
            for cut in range(len(self._pending), max(len(self._pending) - 4, -1), -1):
                try:
                    s = self._pending[:cut].decode("utf-8")
                except UnicodeDecodeError:
                    continue
                self._pending = self._pending[cut:]
                return s
            return ""
        # generic back-ends: re-decode the tail and print the new suffix once it is stable
        self._ids.append(int(token_id))
        text = self.tok.decode(self._ids)
        if text.endswith("�"):
            return ""
        out = text[self._printed:]
        self._printed = len(text)
        return out

    feed_one = next                     # zml/tokenizer/tokenizer.zig:89

    def finalize(self) -> str:
        """What is still held back when generation ends (an incomplete UTF-8 sequence shows as U+FFFD), and resets
        the decoder (zml/tokenizer/tokenizer.zig:97)."""
        if self.tok.backend == "homemade":
            out = self._pending.decode("utf-8", errors="replace")
        else:
            out = self.tok.decode(self._ids)[self._printed:] if self._ids else ""
        self.reset()
        return out


class Tokenizer:
    def __init__(self, backend: str, impl):
        self.backend = backend
        self.impl = impl

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_file(path: str, backend: Optional[str] = None) -> "Tokenizer":
        """`path` is a tokenizer.json, a SentencePiece model, or a repo directory."""
        if os.path.isdir(path):
            for name in ("tokenizer.json", "tokenizer.model"):
                if os.path.exists(os.path.join(path, name)):
                    path = os.path.join(path, name)
                    break
            else:
                raise FileNotFoundError(f"no tokenizer.json / tokenizer.model in {path}")
        if path.endswith((".model", ".pb")):
            import sentencepiece as spm
            return Tokenizer("sentencepiece", spm.SentencePieceProcessor(model_file=path))
        if path.endswith(".bin"):
            return Tokenizer.from_tinyllama_file(path)
        with open(path, "rb") as f:
            return Tokenizer.from_bytes(f.read(), backend)

    @staticmethod
    def from_tinyllama_file(path: str, vocab_size: int = 1 << 20) -> "Tokenizer":
        """A llama2.c `tokenizer.bin` (zml/tokenizer/homemade.zig:1206): scored pieces merged best-first."""
        from .scored import ScoredTokenizer
        return Tokenizer("scored", ScoredTokenizer.from_tinyllama_file(path, vocab_size))

    @staticmethod
    def from_bytes(data: bytes, backend: Optional[str] = None) -> "Tokenizer":
        if backend in (None, "hf"):
            try:
                import tokenizers
                return Tokenizer("hf", tokenizers.Tokenizer.from_str(data.decode("utf-8")))
            except ImportError:
                if backend == "hf":
                    raise
        import json
        kind = json.loads(data.decode("utf-8")).get("model", {}).get("type", "BPE")
        if kind == "Unigram":
            from .unigram import UnigramTokenizer
            return Tokenizer("homemade", UnigramTokenizer.from_bytes(data))
        return Tokenizer("homemade", BpeTokenizer.from_bytes(data))

    # ------------------------------------------------------------------ API
    def encoder(self) -> Encoder:
        return Encoder(self)

    def decoder(self) -> Decoder:
        return Decoder(self)

    def encode(self, text: str) -> list[int]:
        if self.backend == "hf":
            return list(self.impl.encode(text, add_special_tokens=False).ids)
        if self.backend == "sentencepiece":
            return list(self.impl.encode(text))
        return self.impl.encode(text)

    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        ids = [int(i) for i in ids]
        if self.backend == "hf":
            return self.impl.decode(ids, skip_special_tokens=skip_special)
        if self.backend == "sentencepiece":
            return self.impl.decode(ids)
        return self.impl.decode(ids, skip_special)

    def token_id(self, token: str) -> Optional[int]:
        if self.backend == "hf":
            return self.impl.token_to_id(token)
        if self.backend == "sentencepiece":
            i = self.impl.piece_to_id(token)
            return None if i == self.impl.unk_id() and token != self.impl.id_to_piece(i) else i
        return self.impl.token_id(token)

    def vocab_size(self) -> int:
        if self.backend == "hf":
            return self.impl.get_vocab_size(with_added_tokens=True)
        if self.backend == "sentencepiece":
            return self.impl.get_piece_size()
        return self.impl.vocab_size()
