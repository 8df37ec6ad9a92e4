"""Host mirror of femtochat's parameter storage (src/parameters.jl): GPTConfig, the flat
layout, Params(Θ, δ).  The layout itself is computed by the library (femto_layout) so the
Python and Julia hosts see exactly what the kernels use."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from . import _lib

KIND_NAMES = ["wte", "wq", "wk", "wv", "wo", "ve_gate", "fc", "proj", "ve_table", "lam_b", "lam_x0",
              "lm_head", "smear_gate", "lam_s", "lam_y"]


@dataclass
class GPTConfig:
    """src/parameters.jl:71-80 — same fields and defaults."""
    sequence_len: int = 2 ** 11
    max_document_tokens: int = 8192
    vocab_size: int = 2 ** 15
    n_layer: int = 12
    n_head: int = 6
    n_kv_head: int = 6
    n_embed: int = 768
    window_pattern: str = "SSSL"

    def c_struct(self, *, compute_dtype="float32", short_window=0, doc_mask=False, index_base=1, max_batch=1,
                 pad_vocab_size_to=64) -> _lib.FemtoConfig:
        c = _lib.FemtoConfig()
        c.sequence_len, c.max_document_tokens, c.vocab_size = self.sequence_len, self.max_document_tokens, self.vocab_size
        c.n_layer, c.n_head, c.n_kv_head, c.n_embed = self.n_layer, self.n_head, self.n_kv_head, self.n_embed
        c.window_pattern = self.window_pattern.encode()
        c.short_window = short_window
        c.compute_dtype = _lib.BF16 if str(compute_dtype).endswith("bfloat16") or compute_dtype == "bf16" else _lib.F32
        c.doc_mask = 1 if doc_mask else 0
        c.index_base = index_base
        c.max_batch = max_batch
        c.pad_vocab_size_to = pad_vocab_size_to
        return c


@dataclass
class ParamSpec:
    """src/parameters.jl:177-180: `offset` is 0-based, `shape` the Julia (column-major) shape."""
    offset: int
    shape: Tuple[int, ...]

    @property
    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def range(self) -> range:
        return range(self.offset, self.offset + self.size)


def paramview(buf, spec: ParamSpec):
    """src/parameters.jl:188-189 in row-major terms: a Julia (rows, cols) tensor is the
    row-major [cols][rows] view of its flat range."""
    flat = buf[spec.offset:spec.offset + spec.size]
    if len(spec.shape) == 2 and spec.shape != (1, 1):
        return flat.view(spec.shape[1], spec.shape[0])
    return flat


@dataclass
class Layout:
    embedding: ParamSpec
    blocks: List[Dict[str, Optional[ParamSpec]]]
    lm_head: ParamSpec
    smear_gate: ParamSpec
    lam_s: ParamSpec
    lam_y: ParamSpec
    padded_vocab_size: int
    nparams: int


def parameter_layout(config: GPTConfig, pad_vocab_size_to: int = 64) -> Layout:
    """src/parameters.jl:219-337."""
    L = _lib.lib()
    c = config.c_struct(pad_vocab_size_to=pad_vocab_size_to)
    n = L.femto_layout(c, None, 0)
    if n < 0:
        _lib.check(n)
    arr = (_lib.TensorDesc * n)()
    L.femto_layout(c, arr, n)
    blocks = [dict(wq=None, wk=None, wv=None, wo=None, ve_gate=None, fc=None, proj=None, ve_table=None,
                   lam_b=None, lam_x0=None) for _ in range(config.n_layer)]
    glob = {}
    for t in arr:
        name = KIND_NAMES[t.kind]
        shape = (int(t.rows), int(t.cols)) if name not in ("lam_b", "lam_x0", "lam_s", "lam_y") else (1,)
        spec = ParamSpec(int(t.offset), shape)
        if t.layer >= 0:
            blocks[t.layer][name] = spec
        else:
            glob[name] = spec
    nparams = int(L.femto_nparams(c))
    return Layout(glob["wte"], blocks, glob["lm_head"], glob["smear_gate"], glob["lam_s"], glob["lam_y"],
                  glob["wte"].shape[1], nparams)


def has_ve(layer_idx: int, n_layer: int) -> bool:
    """src/parameters.jl:197-198 (1-based layer index)."""
    return (layer_idx - 1) % 2 == (n_layer - 1) % 2


def window_sizes(config: GPTConfig, short_window: int = 0) -> List[Tuple[int, int]]:
    """src/parameters.jl:200-210 through femto_window_sizes."""
    import ctypes as C
    c = config.c_struct(short_window=short_window)
    left = (C.c_int32 * config.n_layer)()
    ve = (C.c_int32 * config.n_layer)()
    _lib.check(_lib.lib().femto_window_sizes(c, left, ve))
    return [(int(x), 0) for x in left]


class Params:
    """src/parameters.jl:31-62: flat parameter vector Θ and its fp32 gradient vector δ."""

    def __init__(self, theta, delta=None):
        import torch
        if theta.dim() != 1:
            raise ValueError("Θ must be a vector")
        if delta is None:
            delta = torch.zeros_like(theta, dtype=torch.float32)
        if delta.dtype != torch.float32:
            raise TypeError("δ must be Float32")
        if delta.numel() != theta.numel():
            raise ValueError("Θ and δ must have equal length")
        self.theta = theta
        self.delta = delta

    Θ = property(lambda self: self.theta)
    δ = property(lambda self: self.delta)
