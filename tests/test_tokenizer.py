"""The in-house BPE against the `tokenizers` library on a byte-level BPE trained in the test."""
import json

import pytest

from zml_b200.tokenizer import Tokenizer

tokenizers = pytest.importorskip("tokenizers")

TEXTS = ["Hello world!", "  multiple   spaces\nand\ttabs", "naïve café — 日本語のテキスト 🙂", "x = 3.14159 * (y+2)//7",
         "<|begin|>system prompt<|end|>The quick brown fox's 123 jumps", ""]


@pytest.fixture(scope="module")
def tok_json(tmp_path_factory):
    from tokenizers import Tokenizer as HfTok, decoders, models, pre_tokenizers, trainers
    t = HfTok(models.BPE())
    t.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    t.decoder = decoders.ByteLevel()
    corpus = ["the quick brown fox jumps over the lazy dog " * 3, "hello world hello tokenizer", "日本語 テキスト",
              "numbers 123 456 3.14159", "def f(x): return x * 2 // 7", "café naïve — emoji 🙂🙂"] * 20
    t.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, special_tokens=["<|begin|>", "<|end|>"],
                                                      initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    p = tmp_path_factory.mktemp("tok") / "tokenizer.json"
    t.save(str(p))
    return str(p)


def test_homemade_matches_hf(tok_json):
    hf = Tokenizer.from_file(tok_json, "hf")
    mine = Tokenizer.from_file(tok_json, "homemade")
    assert hf.backend == "hf" and mine.backend == "homemade"
    for text in TEXTS:
        want = hf.encode(text)
        got = mine.encode(text)
        assert got == want, text
        assert mine.decode(got) == text == hf.decode(want)
    assert mine.token_id("<|end|>") == hf.token_id("<|end|>") == 1
    assert mine.decode(mine.encode("<|begin|>hi"), skip_special=True) == "hi"
    assert mine.vocab_size() == hf.vocab_size()


def test_streaming_decoder_holds_incomplete_utf8(tok_json):
    for backend in ("homemade", "hf"):
        tok = Tokenizer.from_file(tok_json, backend)
        text = "日本語 🙂 ok"
        dec = tok.decoder()
        out = "".join(dec.next(i) for i in tok.encode(text))
        assert out == text
        assert "�" not in out
        assert dec.finalize() == ""
        # generation that stops inside a multi-byte character: the held-back bytes come out of finalize()
        ids = tok.encode("🙂")
        if len(ids) > 1:
            shown = "".join(dec.feed_one(i) for i in ids[:-1])
            assert shown == "" and dec.finalize() != "" and dec.finalize() == ""


def test_cli_checker(tok_json, capsys):
    from zml_b200.tokenizer.__main__ import main
    ids = Tokenizer.from_file(tok_json, "homemade").encode("hello world")
    assert main([f"--tokenizer={tok_json}", "--prompt=hello world", "--backend=homemade",
                 "--expected=" + ",".join(map(str, ids))]) == 0
    assert main([f"--tokenizer={tok_json}", "--prompt=hello world", "--expected=1,2"]) == 1


def test_sentencepiece_style_bpe_with_byte_fallback():
    vocab = {"<unk>": 0, "▁": 1, "h": 2, "i": 3, "▁h": 4, "▁hi": 5, "<0xE2>": 6, "<0x82>": 7, "<0xAC>": 8, "▁t": 9, "t": 10}
    spec = {"model": {"type": "BPE", "vocab": vocab, "merges": ["▁ h", "▁h i", "▁ t"], "byte_fallback": True, "unk_token": "<unk>"},
            "normalizer": {"type": "Sequence", "normalizers": [{"type": "Prepend", "prepend": "▁"},
                                                                {"type": "Replace", "pattern": {"String": " "}, "content": "▁"}]},
            "pre_tokenizer": None, "added_tokens": []}
    tok = Tokenizer.from_bytes(json.dumps(spec).encode(), "homemade")
    assert tok.encode("hi hi") == [5, 5]
    ids = tok.encode("hi €")
    assert ids == [5, 1, 6, 7, 8]
    assert tok.decode(ids) == "hi €"


def test_unigram_tokenizer_matches_hf():
    """The in-house Unigram tokenizer (Viterbi over piece log-probabilities, Metaspace, unknown fusion) against the
    `tokenizers` library on a model trained here."""
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer as HfTok, decoders, models, normalizers, pre_tokenizers, trainers
    from zml_b200.tokenizer import Tokenizer
    corpus = ["the quick brown fox jumps over the lazy dog", "a stitch in time saves nine", "hello world, hello tokens",
              "unigram language models segment text into pieces", "tokenization is fun and pieces are nice"] * 8
    t = HfTok(models.Unigram())
    t.normalizer = normalizers.NFKC()
    t.pre_tokenizer = pre_tokenizers.Metaspace()
    t.decoder = decoders.Metaspace()
    t.train_from_iterator(corpus, trainers.UnigramTrainer(vocab_size=120, special_tokens=["<unk>", "<s>"], unk_token="<unk>"))
    data = t.to_str().encode()
    ours = Tokenizer.from_bytes(data, backend="homemade")
    assert ours.backend == "homemade" and type(ours.impl).__name__ == "UnigramTokenizer"
    for text in ["the quick brown fox", "hello world", "time saves the lazy tokens", "pieces of text", "a dog in time",
                 "<s>hello world", "zebra quartz ωμέγα"]:
        want = t.encode(text, add_special_tokens=False).ids
        got = ours.encode(text)
        assert got == want, (text, got, want)
        assert ours.decode(got) == t.decode(want, skip_special_tokens=False)
    assert ours.vocab_size() == t.get_vocab_size() and ours.token_id("<s>") == t.token_to_id("<s>")


def test_normalizer_matches_the_reference_vectors():
    """The five cases of zml/tokenizer/homemade.zig `test Normalizer`."""
    from zml_b200.tokenizer.scored import Normalizer, SENTENCEPIECE_SPACE
    n = Normalizer(True, True, False, False, False)
    text, origin = n.normalize_with_mapping("Hellŏ  world!")
    assert text == " Hellŏ world!"
    assert origin == [0, 0, 1, 2, 3, 4, 4, 6, 8, 9, 10, 11, 12, 13, 14]
    assert Normalizer(True, True, True, False, False).normalize("Hello  world!") == " Hello world! "
    assert Normalizer(False, True, False, False, False, SENTENCEPIECE_SPACE).normalize("Hello  world!") == "▁Hello▁▁world!"
    assert Normalizer(True, False, True, True, False).normalize("Hello  world!") == "hello world! "
    assert Normalizer(True, False, True, False, True).normalize("Hello  world!") == "Hello world ! "
    assert Normalizer.well_known("sentencepiece").normalize("  a  b ") == "▁a▁b"
    assert Normalizer.well_known("llama3").normalize("   ") == ""


def test_scored_tokenizer_from_a_tinyllama_file(tmp_path):
    """A llama2.c tokenizer.bin: best-scoring merges first, byte pieces for characters outside the vocabulary."""
    import struct
    from zml_b200.tokenizer.scored import ScoredTokenizer
    pieces = [(b"<unk>", 0.0), (b"<s>", 0.0), (b"</s>", 0.0)] + [(b"<0x%02X>" % b, 0.0) for b in range(256)]
    base = len(pieces)
    words = [("▁", -1.0), ("h", -2.0), ("e", -2.0), ("l", -2.0), ("o", -2.0), ("w", -2.0), ("r", -2.0), ("d", -2.0),
             ("he", -3.0), ("ll", -4.0), ("hell", -5.0), ("hello", -0.5), ("▁hello", -0.2), ("wor", -6.0), ("or", -3.5),
             ("ld", -3.6), ("world", -0.6), ("▁world", -0.3), ("lo", -9.0)]
    pieces += [(w.encode(), s) for w, s in words]
    blob = struct.pack("<I", 8) + b"".join(struct.pack("<fI", s, len(p)) + p for p, s in pieces)
    path = tmp_path / "tokenizer.bin"
    path.write_bytes(blob)
    tok = Tokenizer.from_file(str(path))
    assert tok.backend == "scored" and tok.vocab_size() == len(pieces)
    ids = tok.encode("hello  world")
    assert ids == [base + 12, base + 17] and tok.decode(ids) == "hello world"
    # "held": of the pairs he (-3) and ld (-3.6) the better one merges first, then the other; "held" is no piece
    assert [tok.impl.tokens[i] for i in tok.encode("held")] == ["▁".encode(), b"he", b"ld"]
    # a character outside the vocabulary falls back to its bytes and decodes back
    ids = tok.encode("hé")
    assert [tok.impl.tokens[i] for i in ids] == ["▁".encode(), b"h", b"\xc3", b"\xa9"] and tok.decode(ids) == "hé"
    st = ScoredTokenizer.from_tinyllama_file(str(path), vocab_size=1 << 20)
    assert st.encode("hello", add_bos=True, add_eos=True, pad_to=5) == [1, base + 12, 2, st.special.pad, st.special.pad]
    assert st.decode([1, base + 12, base + 17, 2], sep="|") == "| hello| world||"       # only the very first id drops its space
    assert st.decode([base + 12, base + 17], sep="|") == "hello| world|"
    assert st.lookup_piece(10 ** 6) == b"<oob>" and st.lookup_piece(0) == b"<unk>"
    dec = tok.decoder()
    assert "".join(dec.feed_one(i) for i in tok.encode("hello world")) + dec.finalize() == "hello world"
