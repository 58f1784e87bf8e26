"""In-house tokenizer for HF `tokenizer.json` files: byte-level BPE (GPT-2 / Llama-3 /
Qwen style) and SentencePiece-style BPE with byte fallback (Llama-2 / Mistral style).

Plays the role of the reference's "homemade" tokenizer (zml/tokenizer/homemade.zig) and
of its IREE back-end for `tokenizer.json`: normaliser, pre-tokeniser regex, merge loop by
rank, added / special tokens matched first, GPT-2 byte decoder, streaming decode.
"""
from __future__ import annotations

import json
import unicodedata
from functools import lru_cache
from typing import Iterable, Optional

import regex as re

GPT2_SPLIT = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""


@lru_cache(maxsize=1)
def bytes_to_unicode() -> dict[int, str]:
    """GPT-2's reversible byte -> printable unicode character table."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


class BpeTokenizer:
    def __init__(self, spec: dict):
        model = spec["model"]
        if model.get("type", "BPE") != "BPE":
            raise ValueError(f"unsupported tokenizer model {model.get('type')}")
        self.vocab: dict[str, int] = dict(model["vocab"])
        merges = model.get("merges", [])
        self.ranks: dict[tuple[str, str], int] = {}
        for i, m in enumerate(merges):
            a, b = m.split(" ", 1) if isinstance(m, str) else m
            self.ranks[(a, b)] = i
        self.byte_fallback = bool(model.get("byte_fallback", False))
        self.unk = model.get("unk_token")
        self.added: dict[str, int] = {}
        self.special_ids: set[int] = set()
        for t in spec.get("added_tokens", []):
            self.added[t["content"]] = t["id"]
            if t.get("special", False):
                self.special_ids.add(t["id"])
        self.id_to_token = {i: t for t, i in self.vocab.items()}
        self.id_to_token.update({i: t for t, i in self.added.items()})
        self._added_re = None
        if self.added:
            alts = sorted(self.added, key=len, reverse=True)
            self._added_re = re.compile("(" + "|".join(re.escape(a) for a in alts) + ")")
        self.normalizers = self._flatten(spec.get("normalizer"))
        pre = self._flatten(spec.get("pre_tokenizer"))
        self.byte_level = any(p.get("type") == "ByteLevel" for p in pre) or \
            (spec.get("decoder") or {}).get("type") == "ByteLevel"
        self.add_prefix_space = any(p.get("type") == "ByteLevel" and p.get("add_prefix_space") for p in pre)
        self.split_re = None
        for p in pre:
            if p.get("type") == "Split":
                pat = p["pattern"]
                self.split_re = re.compile(pat.get("Regex") or re.escape(pat.get("String", " ")))
            elif p.get("type") == "ByteLevel" and p.get("use_regex", True) and self.split_re is None:
                self.split_re = re.compile(GPT2_SPLIT)
        self.metaspace = any(p.get("type") == "Metaspace" for p in pre) or \
            any(n.get("type") == "Replace" and (n.get("content") == "▁") for n in self.normalizers)
        self._b2u = bytes_to_unicode()
        self._u2b = {c: b for b, c in self._b2u.items()}
        self._cache: dict[str, list[int]] = {}

    @staticmethod
    def _flatten(node: Optional[dict]) -> list[dict]:
        if not node:
            return []
        if node.get("type") == "Sequence":
            out = []
            for n in node.get("normalizers", node.get("pretokenizers", [])):
                out.extend(BpeTokenizer._flatten(n))
            return out
        return [node]

    @staticmethod
    def from_file(path: str) -> "BpeTokenizer":
        with open(path, "r", encoding="utf-8") as f:
            return BpeTokenizer(json.load(f))

    @staticmethod
    def from_bytes(data: bytes) -> "BpeTokenizer":
        return BpeTokenizer(json.loads(data))

    # ------------------------------------------------------------------ encode
    def _normalize(self, text: str) -> str:
        for n in self.normalizers:
            t = n.get("type")
            if t in ("NFC", "NFD", "NFKC", "NFKD"):
                text = unicodedata.normalize(t, text)
            elif t == "Prepend":
                text = n.get("prepend", "") + text
            elif t == "Replace":
                pat = n.get("pattern", {})
                if "String" in pat:
                    text = text.replace(pat["String"], n.get("content", ""))
                elif "Regex" in pat:
                    text = re.sub(pat["Regex"], n.get("content", ""), text)
            elif t == "Lowercase":
                text = text.lower()
        return text

    def _bpe(self, symbols: list[str]) -> list[str]:
        if len(symbols) < 2:
            return symbols
        while True:
            best, best_i = None, -1
            for i in range(len(symbols) - 1):
                r = self.ranks.get((symbols[i], symbols[i + 1]))
                if r is not None and (best is None or r < best):
                    best, best_i = r, i
            if best is None:
                return symbols
            a, b = symbols[best_i], symbols[best_i + 1]
            out, i = [], 0
            while i < len(symbols):
                if i < len(symbols) - 1 and symbols[i] == a and symbols[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(symbols[i])
                    i += 1
            symbols = out
            if len(symbols) < 2:
                return symbols

    def _encode_word(self, word: str) -> list[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        if word in self.vocab:
            ids = [self.vocab[word]]
        else:
            ids = []
            for piece in self._bpe(list(word)):
                i = self.vocab.get(piece)
                if i is not None:
                    ids.append(i)
                elif self.byte_fallback:
                    for b in piece.encode("utf-8"):
                        ids.append(self.vocab.get(f"<0x{b:02X}>", self.vocab.get(self.unk, 0) if self.unk else 0))
                elif self.unk is not None and self.unk in self.vocab:
                    ids.append(self.vocab[self.unk])
        if len(self._cache) < 100000:
            self._cache[word] = ids
        return ids

    def _encode_plain(self, text: str) -> list[int]:
        if not text:
            return []
        text = self._normalize(text)
        if self.byte_level:
            if self.add_prefix_space and not text.startswith(" "):
                text = " " + text
            words = self.split_re.findall(text) if self.split_re is not None else [text]
            if self.split_re is not None and words and isinstance(words[0], tuple):
                words = ["".join(w) for w in words]
            if self.split_re is not None:
                # keep the text between matches too (Split with "Isolated" behaviour)
                words, pos = [], 0
                for m in self.split_re.finditer(text):
                    if m.start() > pos:
                        words.append(text[pos:m.start()])
                    words.append(m.group(0))
                    pos = m.end()
                if pos < len(text):
                    words.append(text[pos:])
            out = []
            for w in words:
                out.extend(self._encode_word("".join(self._b2u[b] for b in w.encode("utf-8"))))
            return out
        if self.metaspace and "▁" not in text:
            text = "▁" + text.replace(" ", "▁")
        return self._encode_word(text)

    def encode(self, text: str) -> list[int]:
        """Text -> ids; added / special tokens present verbatim in `text` map to their ids."""
        if self._added_re is None:
            return self._encode_plain(text)
        out = []
        for part in self._added_re.split(text):
            if not part:
                continue
            if part in self.added:
                out.append(self.added[part])
            else:
                out.extend(self._encode_plain(part))
        return out

    # ------------------------------------------------------------------ decode
    def token_id(self, token: str) -> Optional[int]:
        i = self.added.get(token)
        return i if i is not None else self.vocab.get(token)

    def token_bytes(self, tid: int) -> bytes:
        tok = self.id_to_token.get(tid)
        if tok is None:
            return b""
        if tid in self.added.values() and tok in self.added:
            return tok.encode("utf-8")
        if self.byte_level:
            return bytes(self._u2b.get(c, ord("?")) for c in tok)
        if self.byte_fallback and len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
            return bytes([int(tok[3:5], 16)])
        return tok.replace("▁", " ").encode("utf-8")

    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        raw = b"".join(self.token_bytes(i) for i in ids if not (skip_special and i in self.special_ids))
        text = raw.decode("utf-8", errors="replace")
        if not self.byte_level and self.metaspace and text.startswith(" "):
            text = text[1:]
        return text

    def vocab_size(self) -> int:
        return max(self.id_to_token) + 1 if self.id_to_token else 0
