"""Self-contained byte-level BPE tokenizer: train, encode, decode, save / load, no third-party tokenizer library.

The reference bundles a third-party vocabulary directory (``src/tokenizer/``: ``vocab`` + ``merges.txt`` of a byte-level
BPE) and loads it through ``transformers.AutoTokenizer`` (``src/training/tokenizer.py:12-28``). That vocabulary is not
redistributed here. Instead this module

* reads any byte-level BPE directory of that family (``vocab.json`` + ``merges.txt``, or a ``tokenizer.json`` with a
  ``model.vocab`` / ``model.merges`` section, plus the special tokens listed in ``added_tokens``) without
  ``transformers``, so the reference's directory, or any GPT-2 / Qwen style tokenizer on disk, loads as is;
* trains a vocabulary from an iterator of texts (``train_bpe``) and writes it in the same ``vocab.json`` +
  ``merges.txt`` format;
* ships a small vocabulary trained on this project's own documentation (``assets/bpe_small``), selected with
  ``--tokenizer_path builtin`` (the byte tokenizer stays the default when no tokenizer is named).

Byte-level BPE: text is split by a pre-tokenisation pattern, every piece is turned into UTF-8 bytes mapped to printable
unicode characters (the GPT-2 byte alphabet), and adjacent symbols are merged in rank order.
"""
from __future__ import annotations

import json
from collections import Counter
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

try:                                     # the `regex` module has \\p classes; plain `re` gets a simpler pattern
    import regex as _re
    _PRETOKENIZE = _re.compile(r"'(?:[sdmt]|ll|ve|re)| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+")
except ImportError:                      # pragma: no cover
    import re as _re
    _PRETOKENIZE = _re.compile(r"'(?:[sdmt]|ll|ve|re)| ?[^\W\d_]+| ?\d+| ?[^\s\w]+|\s+(?!\S)|\s+")

SPECIAL_TOKENS = ("<|endoftext|>", "<|im_start|>", "<|im_end|>")


def byte_alphabet() -> Dict[int, str]:
    """byte -> printable unicode character (printable latin-1 bytes map to themselves, the rest to U+0100...)."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


_B2U = byte_alphabet()
_U2B = {u: b for b, u in _B2U.items()}


def _to_symbols(piece: str) -> Tuple[str, ...]:
    return tuple(_B2U[b] for b in piece.encode("utf-8"))


class BPETokenizer:
    """Byte-level BPE with the small part of the HuggingFace tokenizer interface the data pipeline and the eval
    server use: ``encode``, ``__call__``, ``decode``, ``apply_chat_template``, ``vocab_size``, ``eos_token_id``,
    ``pad_token_id``."""

    def __init__(self, vocab: Dict[str, int], merges: Sequence[Tuple[str, str]],
                 special_tokens: Optional[Dict[str, int]] = None, pattern: Optional[str] = None,
                 normalizer: Optional[str] = None):
        self.pattern = pattern                         # pre-tokenisation regex of the vocabulary (None: the default one)
        self._split = _re.compile(pattern) if pattern else _PRETOKENIZE
        self.normalizer = normalizer                   # unicode normal form applied before splitting (e.g. "NFC")
        self.vocab = dict(vocab)
        self.ranks = {tuple(m): i for i, m in enumerate(merges)}
        self.merges = [tuple(m) for m in merges]
        self.special = dict(special_tokens or {})
        self.id_to_token = {i: t for t, i in self.vocab.items()}
        self.id_to_token.update({i: t for t, i in self.special.items()})
        self._cache: Dict[str, List[int]] = {}
        self._special_re = None
        if self.special:
            import re
            self._special_re = re.compile("(" + "|".join(re.escape(t) for t in sorted(self.special, key=len, reverse=True)) + ")")
        eos = self.special.get("<|endoftext|>", self.special.get("<|im_end|>"))
        self.eos_token_id = eos if eos is not None else max(self.id_to_token)
        self.pad_token_id = self.eos_token_id
        self.bos_token_id = self.special.get("<|im_start|>")

    @property
    def vocab_size(self) -> int:
        return max(self.id_to_token) + 1

    # ------------------------------------------------------------------ encode
    def _bpe(self, piece: str) -> List[int]:
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        word = list(_to_symbols(piece))
        while len(word) > 1:
            best, best_rank = -1, None
            for i in range(len(word) - 1):
                r = self.ranks.get((word[i], word[i + 1]))
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best_rank is None:
                break
            a, b = word[best], word[best + 1]
            out, i = [], 0
            while i < len(word):                       # merge every occurrence of the best pair, left to right
                if i + 1 < len(word) and word[i] == a and word[i + 1] == b:
                    out.append(a + b); i += 2
                else:
                    out.append(word[i]); i += 1
            word = out
        ids = []
        for sym in word:
            tid = self.vocab.get(sym)
            if tid is None:                            # a symbol outside the vocabulary: fall back to its bytes
                ids.extend(self.vocab[ch] for ch in sym if ch in self.vocab)
            else:
                ids.append(tid)
        if len(self._cache) < 1 << 20:
            self._cache[piece] = ids
        return ids

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids: List[int] = []
        parts = self._special_re.split(text) if self._special_re is not None else [text]
        for part in parts:
            if not part:
                continue
            if part in self.special:
                ids.append(self.special[part])
                continue
            if self.normalizer:
                import unicodedata
                part = unicodedata.normalize(self.normalizer, part)
            for piece in self._split.findall(part):
                ids.extend(self._bpe(piece))
        return ids

    def __call__(self, texts, add_special_tokens: bool = False, **kw):
        if isinstance(texts, str):
            return {"input_ids": self.encode(texts)}
        return {"input_ids": [self.encode(t) for t in texts]}

    # ------------------------------------------------------------------ decode
    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        out, buf = [], bytearray()
        for i in ids:
            tok = self.id_to_token.get(int(i))
            if tok is None:
                continue
            if tok in self.special:
                if not skip_special_tokens:
                    out.append(buf.decode("utf-8", errors="replace")); buf = bytearray(); out.append(tok)
                continue
            buf.extend(_U2B[ch] for ch in tok if ch in _U2B)
        out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    def apply_chat_template(self, messages, tokenize: bool = False, add_generation_prompt: bool = True):
        text = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
        if add_generation_prompt:
            text += "<|im_start|>assistant\n"
        return self.encode(text) if tokenize else text

    # ------------------------------------------------------------------ files
    def save(self, directory) -> None:
        """``vocab.json`` + ``merges.txt`` + ``special_tokens.json`` (the GPT-2 / Qwen family layout)."""
        d = Path(directory)
        d.mkdir(parents=True, exist_ok=True)
        (d / "vocab.json").write_text(json.dumps(self.vocab, ensure_ascii=False), encoding="utf-8")
        (d / "merges.txt").write_text("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in self.merges) + "\n",
                                      encoding="utf-8")
        (d / "special_tokens.json").write_text(json.dumps(self.special, ensure_ascii=False), encoding="utf-8")
        if self.pattern or self.normalizer:
            (d / "pretokenizer.json").write_text(json.dumps({"pattern": self.pattern, "normalizer": self.normalizer}),
                                                 encoding="utf-8")

    @classmethod
    def load(cls, directory) -> "BPETokenizer":
        d = Path(directory)
        vocab, merges, special, pattern, normalizer = None, None, {}, None, None
        tj = d / "tokenizer.json"
        if (d / "vocab.json").exists() and (d / "merges.txt").exists():
            vocab = json.loads((d / "vocab.json").read_text(encoding="utf-8"))
            merges = _read_merges((d / "merges.txt").read_text(encoding="utf-8").splitlines())
        elif tj.exists():
            model = json.loads(tj.read_text(encoding="utf-8"))
            vocab = model["model"]["vocab"]
            merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m) for m in model["model"]["merges"]]
        else:
            raise FileNotFoundError(f"{d}: neither vocab.json + merges.txt nor tokenizer.json")
        if (d / "special_tokens.json").exists():
            special = json.loads((d / "special_tokens.json").read_text(encoding="utf-8"))
        if (d / "pretokenizer.json").exists():
            pj = json.loads((d / "pretokenizer.json").read_text(encoding="utf-8"))
            pattern, normalizer = pj.get("pattern"), pj.get("normalizer")
        if tj.exists():                                     # special tokens, split pattern, normaliser of a tokenizer.json
            full = json.loads(tj.read_text(encoding="utf-8"))
            for t in full.get("added_tokens", []):
                special.setdefault(t["content"], int(t["id"]))
            pre = full.get("pre_tokenizer") or {}
            for sub in (pre.get("pretokenizers") or [pre]):
                rx = (sub.get("pattern") or {}).get("Regex") if sub.get("type") == "Split" else None
                if rx and pattern is None:
                    pattern = rx
            norm = full.get("normalizer") or {}
            if norm.get("type") in ("NFC", "NFD", "NFKC", "NFKD") and normalizer is None:
                normalizer = norm["type"]
        cfg = d / "tokenizer_config.json"
        if cfg.exists():
            for tid, t in (json.loads(cfg.read_text(encoding="utf-8")).get("added_tokens_decoder") or {}).items():
                special.setdefault(t["content"], int(tid))
        return cls(vocab, merges, special, pattern, normalizer)


def _read_merges(lines: Iterable[str]) -> List[Tuple[str, str]]:
    out = []
    for ln in lines:
        if not ln or ln.startswith("#version"):
            continue
        a, _, b = ln.partition(" ")
        if b:
            out.append((a, b))
    return out


def train_bpe(texts: Iterable[str], vocab_size: int, special_tokens: Sequence[str] = SPECIAL_TOKENS,
              min_frequency: int = 2) -> BPETokenizer:
    """Classic BPE training on pre-tokenised word counts: start from the 256 byte symbols, repeatedly merge the most
    frequent adjacent pair (ties broken by the pair's text, so the result does not depend on dict order) until the
    vocabulary reaches ``vocab_size`` (special tokens included) or no pair occurs ``min_frequency`` times. Pair
    counts are updated incrementally: only the words that contain the merged pair are revisited."""
    counts: Counter = Counter()
    for t in texts:
        counts.update(_PRETOKENIZE.findall(t))
    words = [list(_to_symbols(w)) for w in counts]
    freqs = [counts[w] for w in counts]
    vocab = {_B2U[b]: b for b in range(256)}
    merges: List[Tuple[str, str]] = []
    pair_freq: Counter = Counter()
    where: Dict[Tuple[str, str], set] = {}
    for wi, w in enumerate(words):
        for a, b in zip(w, w[1:]):
            pair_freq[(a, b)] += freqs[wi]
            where.setdefault((a, b), set()).add(wi)
    budget = vocab_size - len(special_tokens)
    while len(vocab) < budget and pair_freq:
        (a, b), f = max(pair_freq.items(), key=lambda kv: (kv[1], kv[0]))
        if f < min_frequency:
            break
        merges.append((a, b))
        vocab[a + b] = len(vocab)
        for wi in list(where.pop((a, b), ())):
            w, fr = words[wi], freqs[wi]
            for x, y in zip(w, w[1:]):                      # retract this word's pairs ...
                pair_freq[(x, y)] -= fr
                if pair_freq[(x, y)] <= 0:
                    del pair_freq[(x, y)]
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(a + b); i += 2
                else:
                    out.append(w[i]); i += 1
            words[wi] = out
            for x, y in zip(out, out[1:]):                  # ... and count the new ones
                pair_freq[(x, y)] += fr
                where.setdefault((x, y), set()).add(wi)
        pair_freq.pop((a, b), None)
    special = {t: len(vocab) + i for i, t in enumerate(special_tokens)}
    return BPETokenizer(vocab, merges, special)


DEFAULT_ASSET = Path(__file__).resolve().parent / "assets" / "bpe_small"


def load_default() -> BPETokenizer:
    """The bundled small vocabulary (trained on this project's documentation by ``python -m hippolm_b200.data.bpe``)."""
    return BPETokenizer.load(DEFAULT_ASSET)


def _main() -> None:                                        # pragma: no cover - asset generation
    import argparse
    ap = argparse.ArgumentParser(description="train a byte-level BPE vocabulary from text files")
    ap.add_argument("files", nargs="+")
    ap.add_argument("--vocab_size", type=int, default=4096)
    ap.add_argument("--out", type=str, default=str(DEFAULT_ASSET))
    a = ap.parse_args()
    texts = (Path(f).read_text(encoding="utf-8", errors="replace") for f in a.files)
    tok = train_bpe(texts, a.vocab_size)
    tok.save(a.out)
    print(f"{a.out}: vocab_size {tok.vocab_size}, {len(tok.merges)} merges")


if __name__ == "__main__":                                  # pragma: no cover
    _main()
