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
