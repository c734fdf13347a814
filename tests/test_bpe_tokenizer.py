"""In-tree byte-level BPE (``hippolm_b200/data/bpe.py``): training, round trips, files, and token-for-token equality with
the ``tokenizers`` library on the same vocabulary."""
import json

import pytest

from hippolm_b200.data import bpe
from hippolm_b200.data.tokenizer import ByteTokenizer, load_tokenizer

CORPUS = ["the quick brown fox jumps over the lazy dog " * 20,
          "tensor cores multiply tiles; tensor memory holds accumulators. " * 15,
          "def f(x):\n    return x + 1\n" * 10, "数据并行 与 张量并行 " * 10]
SAMPLES = ["the lazy tensor jumps!", "  def g(y):\n\treturn y", "naïve café 数据 🚀", "", "x", "<|im_start|>user\nhi<|im_end|>\n"]


def test_train_roundtrip_and_determinism():
    a = bpe.train_bpe(CORPUS, 600)
    b = bpe.train_bpe(list(reversed(CORPUS)), 600)
    assert a.merges == b.merges and a.vocab == b.vocab           # independent of input order
    assert 256 < a.vocab_size <= 600
    for s in SAMPLES:
        ids = a.encode(s)
        assert a.decode(ids, skip_special_tokens=False) == s
        assert all(0 <= i < a.vocab_size for i in ids)
    assert len(a.encode(CORPUS[0])) < len(CORPUS[0].encode()) // 2   # merges actually compress the training text
    assert a.encode("<|im_end|>") == [a.special["<|im_end|>"]]
    assert a.decode(a.encode("a<|im_end|>b")) == "ab"            # specials are dropped by default


def test_save_load_and_tokenizer_json(tmp_path):
    t = bpe.train_bpe(CORPUS, 500)
    t.save(tmp_path / "d")
    u = bpe.BPETokenizer.load(tmp_path / "d")
    assert [u.encode(s) for s in SAMPLES] == [t.encode(s) for s in SAMPLES]
    assert u.eos_token_id == t.eos_token_id == t.special["<|endoftext|>"]
    # the single-file layout with its own split pattern, normaliser and added tokens
    hf = {"added_tokens": [{"id": i, "content": c} for c, i in t.special.items()],
          "normalizer": {"type": "NFC"},
          "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
              {"type": "Split", "pattern": {"Regex": r"\p{N}|[^\s\p{N}]+|\s+"}, "behavior": "Isolated"},
              {"type": "ByteLevel", "use_regex": False}]},
          "model": {"type": "BPE", "vocab": t.vocab, "merges": [f"{a} {b}" for a, b in t.merges]}}
    (tmp_path / "j").mkdir()
    (tmp_path / "j" / "tokenizer.json").write_text(json.dumps(hf), encoding="utf-8")
    v = bpe.BPETokenizer.load(tmp_path / "j")
    assert v.pattern == r"\p{N}|[^\s\p{N}]+|\s+" and v.normalizer == "NFC"
    assert len(v.encode("12345")) == 5                           # digits split one by one under that pattern
    assert v.decode(v.encode("café 12")) == "café 12"  # NFC composed the accent
    w = load_tokenizer(str(tmp_path / "j"))
    assert isinstance(w, bpe.BPETokenizer) and w.encode("tensor 12") == v.encode("tensor 12")


def test_bundled_vocabulary_and_loader():
    t = load_tokenizer("builtin")
    assert isinstance(t, bpe.BPETokenizer) and t.vocab_size > 1000
    s = "tcgen05.mma accumulates into tensor memory"
    assert t.decode(t.encode(s)) == s and len(t.encode(s)) < len(s) // 2
    assert isinstance(load_tokenizer(None), ByteTokenizer)
    assert t("ab")["input_ids"] == t.encode("ab") and t(["ab", "c"])["input_ids"] == [t.encode("ab"), t.encode("c")]


def test_matches_the_tokenizers_library():
    tk = pytest.importorskip("tokenizers")
    from tokenizers import models, pre_tokenizers, Regex
    t = bpe.train_bpe(CORPUS, 700)
    ref = tk.Tokenizer(models.BPE(vocab=t.vocab, merges=[tuple(m) for m in t.merges]))
    pat = r"'(?:[sdmt]|ll|ve|re)| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"
    ref.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    for s in SAMPLES[:5] + CORPUS:
        assert t.encode(s) == ref.encode(s, add_special_tokens=False).ids, s
