"""Tokenizer loading (``src/training/tokenizer.py:12-28``): a tokenizer directory (read by the in-tree byte-level BPE
of ``data/bpe.py`` or by ``transformers``), with ``pad = eos`` when the tokenizer has no pad token; ``builtin`` selects
the bundled small BPE vocabulary. A byte-level fallback keeps the text pipeline usable when no tokenizer is named."""
from __future__ import annotations

from typing import List, Optional


class ByteTokenizer:
    """UTF-8 bytes + 2 specials (256 = eos/pad, 257 = bos). vocab_size 258."""
    vocab_size = 258
    eos_token_id = 256
    pad_token_id = 256
    bos_token_id = 257

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        return list(text.encode("utf-8"))

    def __call__(self, texts, add_special_tokens: bool = False, **kw):
        if isinstance(texts, str):
            return {"input_ids": self.encode(texts)}
        return {"input_ids": [self.encode(t) for t in texts]}

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return bytes(i for i in ids if 0 <= int(i) < 256).decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, tokenize: bool = False, add_generation_prompt: bool = True):
        text = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
        if add_generation_prompt:
            text += "<|im_start|>assistant\n"
        return self.encode(text) if tokenize else text


def load_tokenizer(path: Optional[str]):
    """``None`` -> byte tokenizer; ``"builtin"`` -> the bundled small byte-level BPE vocabulary; a directory -> the
    in-tree BPE reader (``data/bpe.py``: ``vocab.json`` + ``merges.txt`` or ``tokenizer.json``, token-for-token equal
    to the HuggingFace tokenizer on such a directory), or ``transformers.AutoTokenizer`` when
    ``HIPPO_TOKENIZER_BACKEND=hf`` or the directory is not a byte-level BPE."""
    import os
    if not path:
        return ByteTokenizer()
    from . import bpe
    if path in ("builtin", "builtin:bpe_small"):
        return bpe.load_default()
    if os.environ.get("HIPPO_TOKENIZER_BACKEND", "native") != "hf":
        try:
            return bpe.BPETokenizer.load(path)
        except (FileNotFoundError, KeyError, ValueError):
            pass                                        # not a byte-level BPE directory: let transformers try
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(path, trust_remote_code=False)
    if tok.pad_token_id is None:
        tok.pad_token = tok.eos_token
    return tok
