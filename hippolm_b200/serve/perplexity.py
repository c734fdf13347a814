"""Offline perplexity of a checkpoint over local text: no server, no network, no external harness.

Documents (strings) are tokenised, packed by the training packer into ``[rows, seq_len]`` batches with ``cu_seqlens``
(documents never attend across their borders, the first token of a document is not a target) and run through the model's
own loss head; the result is the token-weighted mean negative log-likelihood and its exponential. Works under tensor
parallelism as well (every rank calls it with the same documents). The reference evaluates through an external harness
over its HTTP server only (``scripts/eval.py:67-357``)."""
from __future__ import annotations

import json
import math
from typing import Dict, Iterable, Iterator, List, Optional

import torch

from ..data.packing import pack_chunk_aligned


def iter_documents(files: Iterable[str], text_field: str = "content") -> Iterator[str]:
    """Documents of local files: ``.jsonl`` (one object per line, text under ``text_field`` or ``text``), ``.parquet``
    (same fields) and anything else as plain text (documents separated by blank lines)."""
    for f in files:
        f = str(f)
        if f.endswith(".parquet"):
            from ..data.streaming import iter_parquet_rows
            for row in iter_parquet_rows(f):
                t = row.get(text_field) or row.get("text")
                if t:
                    yield t
        elif f.endswith(".jsonl") or f.endswith(".json"):
            with open(f) as fh:
                for line in fh:
                    if line.strip():
                        row = json.loads(line)
                        t = row.get(text_field) or row.get("text")
                        if t:
                            yield t
        else:
            with open(f, errors="replace") as fh:
                for doc in fh.read().split("\n\n"):
                    if doc.strip():
                        yield doc


@torch.no_grad()
def evaluate_perplexity(model, tokenizer, documents: Iterable[str], seq_len: int = 1024, batch_rows: int = 4,
                        max_tokens: Optional[int] = None) -> Dict[str, float]:
    """``{"nll", "perplexity", "tokens", "documents"}`` over ``documents``. Documents longer than ``seq_len`` are cut into
    pieces of ``seq_len`` tokens (each piece is scored on its own context)."""
    cfg = model.cfg
    dev = next(model.parameters()).device
    eos = getattr(tokenizer, "eos_token_id", None)
    chunk = cfg.pack_chunk_size
    seq_len = max(chunk, seq_len // chunk * chunk)
    was_training = model.training
    model.eval()
    total_nll, total_tok, n_docs = 0.0, 0, 0
    pending: List[List[int]] = []

    def flush(final: bool):
        nonlocal total_nll, total_tok, pending
        while pending and (final or len(pending) >= 4 * batch_rows):
            take, pending = pending[:4 * batch_rows], pending[4 * batch_rows:]
            while take:
                # documents are placed largest first; whatever did not fit goes into the next batch
                ids, labels, cu, fitted = pack_chunk_aligned(take, seq_len, chunk, batch_rows, pad_id=0, eos_id=None,
                                                             return_placed=True)
                out = model(ids.to(dev), labels=labels.to(dev), cu_seqlens=cu.to(device=dev, dtype=torch.int32))
                n = int(out["n_valid"])
                if n > 0:
                    total_nll += float(out["loss"]) * n
                    total_tok += n
                fitted = set(fitted)
                take = [d for i, d in enumerate(take) if i not in fitted]
        return

    for text in documents:
        toks = tokenizer.encode(text, add_special_tokens=False)
        if eos is not None:
            toks = toks + [eos]
        if len(toks) < 2:
            continue
        n_docs += 1
        for s in range(0, len(toks), seq_len):
            piece = toks[s:s + seq_len]
            if len(piece) >= 2:
                pending.append(piece)
        flush(False)
        if max_tokens is not None and total_tok >= max_tokens:
            pending = []
            break
    flush(True)
    model.train(was_training)
    nll = total_nll / max(1, total_tok)
    return {"nll": nll, "perplexity": math.exp(min(nll, 700.0)), "tokens": total_tok, "documents": n_docs}
