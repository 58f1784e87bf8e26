"""Score-driven merge tokenizer and its text normalizer: the reference's in-house tokenizer
(zml/tokenizer/homemade.zig), used there for `tokenizer.bin` files of the llama2.c / TinyLlama kind and for simple
SentencePiece-style vocabularies.

* `Normalizer` - the simplified SentencePiece normalizer (zml/tokenizer/homemade.zig:585-745): strips and collapses
  runs of spaces, optionally adds a leading / trailing space, writes spaces as U+2581, lower-cases ASCII, splits ASCII
  punctuation from the word in front of it; `normalize_with_mapping` also returns, per normalized byte, the offset of
  the input byte it came from.
* `ScoredTokenizer` - pieces with scores; text is first cut into single characters (bytes when a character is not
  in the vocabulary and the vocabulary has byte pieces, else the unknown token), then the adjacent pair whose
  concatenation is the best-scoring piece is merged until no pair is a piece (zml/tokenizer/homemade.zig:118-290).
  Pieces spelled `<0xNN>` are re-keyed as their byte at load (`rewriteByteFallbackTokens`).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Iterable, Optional, Sequence

SENTENCEPIECE_SPACE = "▁"


def _is_punct(ch: bytes) -> bool:
    if len(ch) > 1:
        return False
    b = ch[0]
    if b in (0x20, 0x09):
        return False
    return (b <= 8 or 10 <= b <= 31 or 0x21 <= b <= 0x2F or 0x3A <= b <= 0x40 or 0x5B <= b <= 0x60 or 0x7B <= b <= 0x7E)


@dataclass
class Normalizer:
    remove_extra_whitespaces: bool = True
    add_dummy_prefix: bool = True
    add_dummy_suffix: bool = False
    lower_case_ascii: bool = False
    split_on_punct_ascii: bool = False
    escaped_whitespace: Optional[str] = None        # e.g. U+2581; None: spaces stay spaces

    @staticmethod
    def well_known(impl: str) -> "Normalizer":
        """`sentencepiece` | `llama3` | `gpt2` (zml/tokenizer/homemade.zig:746-770)."""
        if impl == "sentencepiece":
            return Normalizer(True, True, False, False, False, SENTENCEPIECE_SPACE)
        if impl == "llama3":
            return Normalizer(True, False, False, False, False, None)
        if impl == "gpt2":
            return Normalizer(True, True, False, False, False, None)
        raise ValueError(f"unknown normalizer {impl!r}")

    def escaped_space(self) -> Optional[bytes]:
        e = self.escaped_whitespace.encode("utf-8") if self.escaped_whitespace else b""
        return e if len(e) > 1 else None

    def normalize(self, text: str) -> str:
        return self.normalize_with_mapping(text)[0]

    def normalize_with_mapping(self, text: str) -> tuple[str, list[int]]:
        """(normalized text, origins): origins[i] is the byte offset in `text` (UTF-8) that normalized byte i came
        from, plus one final entry = the number of input bytes consumed."""
        data = text.encode("utf-8")
        consumed = 0
        if self.remove_extra_whitespaces:
            while consumed < len(data) and data[consumed] == 0x20:
                consumed += 1
        if consumed == len(data):
            return "", []
        space = self.escaped_space() or b" "
        out = bytearray()
        origin_of: list[int] = []

        def add(piece: bytes, origin: int) -> None:
            out.extend(piece)
            origin_of.extend([origin] * len(piece))

        if self.add_dummy_prefix:
            add(space, consumed)
        prev_space, prev_word = True, False
        while consumed < len(data):
            b0 = data[consumed]
            n = 1 if b0 < 0x80 else 2 if b0 >> 5 == 0b110 else 3 if b0 >> 4 == 0b1110 else 4
            ch = data[consumed:consumed + n]
            origin = consumed
            consumed += n
            if self.remove_extra_whitespaces and prev_space and ch == b" ":
                continue
            prev_space = ch[-1] == 0x20
            if len(ch) == 1:
                byte = ch
                if self.escaped_space() is not None and byte == b" ":
                    add(space, origin)
                    prev_word = False
                    continue
                if self.split_on_punct_ascii and prev_word and _is_punct(ch):
                    add(space, origin)
                if self.lower_case_ascii:
                    byte = byte.lower()
                add(byte, origin)
            else:
                add(ch, origin)
            prev_word = not prev_space and not _is_punct(ch)
        if self.remove_extra_whitespaces:
            while out.endswith(space):
                cut = len(out) - len(space)
                consumed = origin_of[cut]
                del out[cut:]
                del origin_of[cut:]
        origin_of.append(consumed)
        if self.add_dummy_suffix:
            add(space, consumed)
        return out.decode("utf-8"), origin_of


@dataclass
class SpecialTokens:
    unk: int = 0
    bos: int = 1
    eos: int = 2
    pad: int = 0xFFFFFFFF
    hard_space: int = 0xFFFFFFFF


class ScoredTokenizer:
    def __init__(self, pieces: Sequence[bytes], scores: Sequence[float], normalizer: Optional[Normalizer] = None,
                 special: Optional[SpecialTokens] = None, byte_fallback: bool = True):
        self.tokens: list[bytes] = [bytes(p) for p in pieces]
        self.scores: list[float] = [float(s) for s in scores]
        self.normalizer = normalizer
        self.special = special or SpecialTokens()
        self.byte_fallback = False
        self.lookup: dict[bytes, int] = {}
        for i, p in enumerate(self.tokens):
            self.lookup.setdefault(p, i)            # the first piece of a spelling wins, as a hash map insert would
        self.max_token_len = max((len(p) for p in self.tokens), default=1)
        if byte_fallback:
            self.rewrite_byte_fallback_tokens()

    # ------------------------------------------------------------------ loading
    @staticmethod
    def from_tinyllama_file(path: str, vocab_size: int, normalizer: Optional[Normalizer] = None) -> "ScoredTokenizer":
        """`tokenizer.bin` of llama2.c: u32 max piece length, then per piece {f32 score, u32 length, bytes}
        (zml/tokenizer/homemade.zig:1206-1243).  Fewer pieces than `vocab_size` is accepted."""
        with open(path, "rb") as f:
            data = f.read()
        if len(data) < 4:
            raise ValueError(f"{path}: not a tokenizer.bin file")
        off = 4
        pieces, scores = [], []
        while len(pieces) < vocab_size and off + 8 <= len(data):
            score, n = struct.unpack_from("<fI", data, off)
            off += 8
            if off + n > len(data):
                break
            pieces.append(data[off:off + n])
            scores.append(score)
            off += n
        return ScoredTokenizer(pieces, scores, normalizer or Normalizer.well_known("sentencepiece"), SpecialTokens(0, 1, 2), True)

    def rewrite_byte_fallback_tokens(self) -> None:
        """Pieces spelled `<0xNN>` stand for byte NN: re-key them as that byte unless the byte already is a piece, so
        that the merge loop can start from raw bytes (zml/tokenizer/homemade.zig:340-374)."""
        found = 0
        for b in range(256):
            key = b"<0x%02X>" % b
            idx = self.lookup.get(key)
            if idx is None:
                continue
            found += 1
            single = bytes([b])
            if single in self.lookup:
                continue
            del self.lookup[key]
            self.tokens[idx] = single
            self.lookup[single] = idx
        self.byte_fallback = found == 256

    # ------------------------------------------------------------------ encode
    def _initial_tokens(self, data: bytes) -> list[int]:
        out = []
        i = 0
        while i < len(data):
            b0 = data[i]
            n = 1 if b0 < 0x80 else 2 if b0 >> 5 == 0b110 else 3 if b0 >> 4 == 0b1110 else 4
            ch = data[i:i + n]
            tid = self.lookup.get(ch)
            if tid is not None:
                out.append((tid, ch))
            elif self.byte_fallback:
                out.extend((self.lookup[bytes([b])], bytes([b])) for b in ch)
            else:
                out.append((self.special.unk, ch))
            i += n
        return out

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False, pad_to: int = 0) -> list[int]:
        if self.normalizer is not None:
            text = self.normalizer.normalize(text)
        toks = self._initial_tokens(text.encode("utf-8"))           # [(id, bytes it covers)]
        while len(toks) > 1:
            best_score, best_i, best_tok = -1e10, -1, 0
            for i in range(len(toks) - 1):
                if toks[i][0] == self.special.unk and toks[i][1] not in self.lookup:
                    continue
                merged = self.lookup.get(toks[i][1] + toks[i + 1][1])
                if merged is not None and self.scores[merged] > best_score:
                    best_score, best_i, best_tok = self.scores[merged], i, merged
            if best_i < 0:
                break
            toks[best_i:best_i + 2] = [(best_tok, toks[best_i][1] + toks[best_i + 1][1])]
        ids = [t for t, _ in toks]
        if add_bos:
            ids.insert(0, self.special.bos)
        if add_eos:
            ids.append(self.special.eos)
        if len(ids) < pad_to:
            ids.extend([self.special.pad] * (pad_to - len(ids)))
        return ids

    # ------------------------------------------------------------------ decode
    def lookup_piece(self, tid: int) -> bytes:
        """Bytes of a piece; bos / eos / pad decode to nothing, unknown to `<unk>`, an id outside the vocabulary to
        `<oob>` (zml/tokenizer/homemade.zig:293-302)."""
        if tid in (self.special.bos, self.special.eos, self.special.pad):
            return b""
        if tid == self.special.unk:
            return b"<unk>"
        if tid < 0 or tid >= len(self.tokens):
            return b"<oob>"
        return self.tokens[tid]

    token_bytes = lookup_piece

    def decode_bytes(self, ids: Iterable[int], sep: str = "") -> bytes:
        esc = self.normalizer.escaped_space() if self.normalizer is not None else None
        out = bytearray()
        first = True
        for tid in ids:
            piece = self.lookup_piece(int(tid))
            if esc is not None:
                while piece.startswith(esc):
                    piece = piece[len(esc):]
                    if not first:
                        out.extend(b" ")
            out.extend(piece)
            first = False
            out.extend(sep.encode("utf-8"))
        return bytes(out)

    def decode(self, ids: Iterable[int], skip_special: bool = False, sep: str = "") -> str:
        """`sep` is written after every piece (`decodeWithOpts`, zml/tokenizer/homemade.zig:311-338)."""
        ids = [int(i) for i in ids]
        if skip_special:
            ids = [i for i in ids if i != self.special.unk]
        return self.decode_bytes(ids, sep).decode("utf-8", errors="replace")

    def token_id(self, token: str) -> Optional[int]:
        return self.lookup.get(token.encode("utf-8"))

    def vocab_size(self) -> int:
        return len(self.tokens)
