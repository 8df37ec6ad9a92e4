"""Synthetic packed batches in the reference loader's format (src/dataloader.jl:241-274):
documents start with BOS, are concatenated into B columns of T tokens, continue across
batches, targets are the next token of the stream (a document's last token predicts BOS),
positions restart at 0 on BOS.  Token ids are Zipf(s) draws over 1..V-9, document lengths
geometric(mean) clipped to max_document_tokens; ids are 1-based like the reference's."""
from __future__ import annotations

import numpy as np


def bos_token_id(vocab_size: int) -> int:
    """src/tokenizers.jl:102-110: BOS = len(vocab) - 9 + 1 (1-based)."""
    return vocab_size - 9 + 1


class PackedBatches:
    def __init__(self, vocab_size: int, sequence_len: int, batch: int, max_document_tokens: int = 8192,
                 mean_doc_len: int = 512, zipf_s: float = 1.1, seed: int = 0x5EED0000, rank: int = 0):
        self.V, self.T, self.B = vocab_size, sequence_len, batch
        self.maxdoc, self.mean = max_document_tokens, mean_doc_len
        self.rng = np.random.default_rng(seed + 1000 * rank)
        self.bos = bos_token_id(vocab_size)
        nrank = vocab_size - 9
        w = 1.0 / np.power(np.arange(1, nrank + 1, dtype=np.float64), zipf_s)
        self.cdf = np.cumsum(w / w.sum())
        self.slots = [None] * batch   # (tokens, position) of the active document per column

    def _document(self):
        n = int(min(max(self.rng.geometric(1.0 / self.mean), 2), self.maxdoc))
        u = self.rng.random(n - 1)
        body = np.searchsorted(self.cdf, u).astype(np.int64) + 1
        return np.concatenate([[self.bos], body])

    def next(self):
        T, B = self.T, self.B
        tokens = np.full((B, T), self.bos, dtype=np.int32)
        targets = np.full((B, T), -1, dtype=np.int32)
        positions = np.zeros((B, T), dtype=np.int32)
        for col in range(B):
            doc = self.slots[col]
            row = 0
            while row < T:
                if doc is None:
                    doc = [self._document(), 0]
                toks, p = doc
                n = min(T - row, len(toks) - p)
                tokens[col, row:row + n] = toks[p:p + n]
                targets[col, row:row + n - 1] = toks[p + 1:p + n]
                positions[col, row:row + n] = p + np.arange(n)
                doc[1] = p + n
                if doc[1] == len(toks):
                    targets[col, row + n - 1] = self.bos
                    doc = None
                else:
                    targets[col, row + n - 1] = toks[doc[1]]
                row += n
            self.slots[col] = doc
        return tokens, targets, positions
