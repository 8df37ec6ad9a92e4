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


SEGMENT_DTYPE = np.dtype([("src", np.int64), ("col", np.int32), ("row", np.int32), ("n", np.int32), ("pos0", np.int32),
                          ("next", np.int32), ("reserved", np.int32)])   # femto_segment of include/femto.h


class DevicePackedBatches:
    """The same packed batches as `PackedBatches` (same seed -> same arrays, bit for bit), produced on the GPU: the
    documents of `batches` batches are drawn up front into one stream of 0-based 16-bit token ids that lives in device
    memory; per batch the host only walks the document lengths (model_batch!'s assignment of documents to columns,
    src/dataloader.jl:247-270) and emits a short segment list, and femto_pack_batch builds tokens / targets /
    positions from the stream on the device."""

    def __init__(self, vocab_size: int, sequence_len: int, batch: int, batches: int, max_document_tokens: int = 8192,
                 mean_doc_len: int = 512, zipf_s: float = 1.1, seed: int = 0x5EED0000, rank: int = 0):
        import torch
        if vocab_size > 65536:
            raise ValueError("16-bit wire format: vocab_size must be <= 65536")
        gen = PackedBatches(vocab_size, sequence_len, batch, max_document_tokens, mean_doc_len, zipf_s, seed, rank)
        self.V, self.T, self.B, self.bos = vocab_size, sequence_len, batch, gen.bos
        need = batches * batch * sequence_len + batch * max_document_tokens     # every column may end inside a document
        docs, total = [], 0
        while total < need:
            d = gen._document()
            docs.append(d)
            total += len(d)
        self.doc_off = np.concatenate([[0], np.cumsum([len(d) for d in docs])]).astype(np.int64)
        stream = (np.concatenate(docs) - 1).astype(np.uint16)                  # 0-based on the wire
        self._stream_host = stream
        self.stream = torch.from_numpy(stream.view(np.int16)).cuda()
        self.n_stream = int(stream.size)
        self.next_doc = 0
        self.slots = [None] * batch        # (document index, position) of the active document per column
        self.tokens = torch.empty(batch, sequence_len, dtype=torch.int32, device="cuda")
        self.targets = torch.empty_like(self.tokens)
        self.positions = torch.empty_like(self.tokens)
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def plan(self):
        """Segments of the next batch (host side, O(#documents))."""
        T, segs = self.T, []
        for col in range(self.B):
            doc, row = self.slots[col], 0
            while row < T:
                if doc is None:
                    if self.next_doc + 1 >= len(self.doc_off):
                        raise RuntimeError("token stream exhausted: construct with more `batches`")
                    doc = [self.next_doc, 0]
                    self.next_doc += 1
                d, p = doc
                off, length = int(self.doc_off[d]), int(self.doc_off[d + 1] - self.doc_off[d])
                n = min(T - row, length - p)
                doc[1] = p + n
                if doc[1] == length:
                    nxt = self.bos - 1                       # a document's last token predicts BOS
                    doc = None
                else:
                    nxt = int(self._stream_host[off + p + n])
                segs.append((off + p, col, row, n, p, nxt, 0))
                row += n
            self.slots[col] = doc
        return np.array(segs, dtype=SEGMENT_DTYPE)

    def next(self, stream_ptr=None):
        """Device tensors (tokens, targets, positions) of the next batch; they are overwritten by the following call."""
        import torch
        from . import _lib
        segs = self.plan()
        seg_dev = torch.from_numpy(segs.view(np.uint8).reshape(-1)).cuda()
        _lib.check(_lib.lib().femto_pack_batch(
            _lib.ptr(self.stream), self.n_stream, _lib.ptr(seg_dev), len(segs), self.B, self.T, self.bos - 1, 1,
            _lib.ptr(self.tokens), _lib.ptr(self.targets), _lib.ptr(self.positions), _lib.ptr(self.status),
            stream_ptr if stream_ptr is not None else _lib.stream_ptr()))
        self._keep = seg_dev                 # alive until the kernel has run
        return self.tokens, self.targets, self.positions


class Feeder:
    """Pinned, multi-buffered host-to-device feeder (femto_feeder_*): `submit` host int32 [B][T] arrays (numpy or CPU
    torch tensors) as they are produced, `next()` returns device tensors of the oldest submitted batch once its copy
    has been ordered before the current CUDA stream.  The copy of batch i+1 overlaps the step on batch i."""

    def __init__(self, batch: int, sequence_len: int, depth: int = 3):
        import ctypes as C
        from . import _lib
        self.B, self.T = batch, sequence_len
        f = C.c_void_p()
        _lib.check(_lib.lib().femto_feeder_create(batch, sequence_len, depth, C.byref(f)))
        self.f = f

    @staticmethod
    def _host_ptr(x):
        import ctypes as C
        if x is None:
            return None
        if isinstance(x, np.ndarray):
            assert x.dtype == np.int32 and x.flags["C_CONTIGUOUS"]
            return C.c_void_p(x.ctypes.data)
        assert x.dtype.is_floating_point is False and x.is_contiguous()
        return C.c_void_p(x.data_ptr())

    def submit(self, tokens, targets, positions=None):
        from . import _lib
        _lib.check(_lib.lib().femto_feeder_submit(self.f, self._host_ptr(tokens), self._host_ptr(targets),
                                                  self._host_ptr(positions)))

    def next(self):
        """(tokens, targets, positions) as raw device pointers wrapped for the ctypes calls of the step."""
        import ctypes as C
        from . import _lib
        a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
        _lib.check(_lib.lib().femto_feeder_next(self.f, _lib.stream_ptr(), C.byref(a), C.byref(b), C.byref(c)))
        return a, b, (c if c.value else None)

    def release(self):
        from . import _lib
        _lib.check(_lib.lib().femto_feeder_release(self.f, _lib.stream_ptr()))

    def close(self):
        from . import _lib
        if self.f:
            _lib.lib().femto_feeder_destroy(self.f)
            self.f = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
