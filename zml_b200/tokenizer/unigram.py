"""In-house Unigram tokenizer for HF `tokenizer.json` files whose model is `Unigram` (SentencePiece unigram language
model: T5 / ALBERT / XLM-R / Gemma style vocabularies).

The reference reads these through its SentencePiece back-end (zml/tokenizer/sentencepiece/*).  A text is split on
added tokens first, normalised (NFKC / Precompiled are approximated by NFKC, `Replace`, `Strip`, `Lowercase`), the
Metaspace pre-tokenizer turns spaces into U+2581, and each chunk is segmented by Viterbi search for the piece
sequence with the highest total log-probability; characters no piece covers become `<0xNN>` byte pieces
(`byte_fallback`) or the unknown token (consecutive unknowns are fused, as SentencePiece does).
"""
from __future__ import annotations

import json
import unicodedata
from typing import Iterable, Optional

import regex as re

SPACE = "▁"


class UnigramTokenizer:
    def __init__(self, spec: dict):
        model = spec["model"]
        if model.get("type") != "Unigram":
            raise ValueError(f"unsupported tokenizer model {model.get('type')}")
        self.pieces: list[tuple[str, float]] = [(p, float(s)) for p, s in model["vocab"]]
        self.unk_id: Optional[int] = model.get("unk_id")
        self.byte_fallback = bool(model.get("byte_fallback", False))
        self.vocab = {p: i for i, (p, _) in enumerate(self.pieces)}
        self.scores = [s for _, s in self.pieces]
        self.max_len = max((len(p) for p in self.vocab), default=1)
        self.min_score = min(self.scores, default=0.0)
        self.added: dict[str, int] = {}
        self.special_ids: set[int] = set()
        for t in spec.get("added_tokens", []):
            self.added[t["content"]] = t["id"]
            if t.get("special", False):
                self.special_ids.add(t["id"])
        self.id_to_token = {i: p for p, i in self.vocab.items()}
        self.id_to_token.update({i: t for t, i in self.added.items()})
        self._added_re = None
        if self.added:
            alts = sorted(self.added, key=len, reverse=True)
            self._added_re = re.compile("(" + "|".join(re.escape(a) for a in alts) + ")")
        self.normalizers = self._flatten(spec.get("normalizer"))
        self.add_prefix_space = True
        self.replacement = SPACE
        self.prepend_scheme = "always"
        for p in self._flatten(spec.get("pre_tokenizer")):
            if p.get("type") == "Metaspace":
                self.replacement = p.get("replacement", SPACE)
                self.prepend_scheme = p.get("prepend_scheme", "always" if p.get("add_prefix_space", True) else "never")
        self.add_prefix_space = self.prepend_scheme != "never"

    @staticmethod
    def _flatten(node) -> list[dict]:
        if node is None:
            return []
        if node.get("type") == "Sequence":
            out = []
            for n in node.get("normalizers", node.get("pretokenizers", [])):
                out.extend(UnigramTokenizer._flatten(n))
            return out
        return [node]

    @staticmethod
    def from_bytes(data: bytes) -> "UnigramTokenizer":
        return UnigramTokenizer(json.loads(data.decode("utf-8")))

    # ------------------------------------------------------------------ encode
    def _normalize(self, text: str) -> str:
        for n in self.normalizers:
            t = n.get("type")
            if t in ("NFKC", "Precompiled", "Nmt"):
                text = unicodedata.normalize("NFKC", text)
            elif t == "NFC":
                text = unicodedata.normalize("NFC", text)
            elif t == "NFKD":
                text = unicodedata.normalize("NFKD", text)
            elif t == "Lowercase":
                text = text.lower()
            elif t == "Strip":
                text = text.strip()
            elif t == "Replace":
                pat = n.get("pattern", {})
                if "String" in pat:
                    text = text.replace(pat["String"], n.get("content", ""))
                elif "Regex" in pat:
                    text = re.sub(pat["Regex"], n.get("content", ""), text)
        return text

    def _viterbi(self, s: str) -> list[int]:
        n = len(s)
        best = [float("-inf")] * (n + 1)
        back: list[tuple[int, int]] = [(-1, -1)] * (n + 1)          # (start, piece id or -1 for unknown)
        best[0] = 0.0
        unk_pen = self.min_score - 10.0                              # SentencePiece: unknown is worse than any piece
        for i in range(n):
            if best[i] == float("-inf"):
                continue
            hit_single = False
            for j in range(i + 1, min(n, i + self.max_len) + 1):
                pid = self.vocab.get(s[i:j])
                if pid is None:
                    continue
                if j == i + 1:
                    hit_single = True
                sc = best[i] + self.scores[pid]
                if sc > best[j]:
                    best[j], back[j] = sc, (i, pid)
            if not hit_single:
                sc = best[i] + unk_pen
                if sc > best[i + 1]:
                    best[i + 1], back[i + 1] = sc, (i, -1)
        out: list[int] = []
        j = n
        while j > 0:
            i, pid = back[j]
            if pid >= 0:
                out.append(pid)
            else:
                ch = s[i:j]
                if self.byte_fallback and all(f"<0x{b:02X}>" in self.vocab for b in ch.encode("utf-8")):
                    out.extend(reversed([self.vocab[f"<0x{b:02X}>"] for b in ch.encode("utf-8")]))
                elif self.unk_id is not None:
                    out.append(-1)
            j = i
        out.reverse()
        fused: list[int] = []
        prev_unknown = False
        for t in out:                                               # consecutive unknown characters -> one unknown token
            if t == -1:
                if not prev_unknown:
                    fused.append(self.unk_id)
                prev_unknown = True
            else:
                fused.append(t)
                prev_unknown = False
        return fused

    def _encode_chunk(self, text: str, first: bool) -> list[int]:
        text = self._normalize(text)
        if not text:
            return []
        text = text.replace(" ", self.replacement)
        if self.prepend_scheme == "always" or (self.prepend_scheme == "first" and first):
            if not text.startswith(self.replacement):
                text = self.replacement + text
        return self._viterbi(text)

    def encode(self, text: str) -> list[int]:
        parts = [text] if self._added_re is None else self._added_re.split(text)
        out: list[int] = []
        first = True
        for part in parts:
            if not part:
                continue
            if part in self.added:
                out.append(self.added[part])
            else:
                out.extend(self._encode_chunk(part, first))
            first = False
        return out

    # ------------------------------------------------------------------ decode
    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        buf = bytearray()
        for i in ids:
            i = int(i)
            if skip_special and i in self.special_ids:
                continue
            tok = self.id_to_token.get(i, "")
            if len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
                try:
                    buf.append(int(tok[3:5], 16))
                    continue
                except ValueError:
                    pass
            buf.extend(tok.encode("utf-8"))
        s = buf.decode("utf-8", errors="replace").replace(self.replacement, " ")
        return s[1:] if self.add_prefix_space and s.startswith(" ") else s

    def token_id(self, token: str) -> Optional[int]:
        return self.added.get(token, self.vocab.get(token))

    def vocab_size(self) -> int:
        return max(len(self.pieces), max(self.added.values(), default=-1) + 1)
