"""Host mirror of femtochat's model call and gradient driver (src/gpt.jl, src/FemtoChat.jl:29-30,
ext/FemtoChatEnzymeExt.jl:27-44) over libfemto_sm100a.  All arithmetic runs in the library."""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

from . import _lib
from .parameters import GPTConfig, Layout, Params, parameter_layout, paramview


def initialize_(params, layout: Layout, seed: int = 123, all_nonzero: bool = False) -> None:
    """`initialize!` (src/gpt.jl:220-256): same distributions and draw order, drawn with torch's
    generator on Θ's device.  (The reference's own RNG stream exists only inside Julia.)
    `all_nonzero` also randomises the two zero-initialised projections and sets λₛ = 0.1."""
    import torch
    theta = params.theta if isinstance(params, Params) else params
    g = torch.Generator(device=theta.device).manual_seed(seed)
    d = layout.embedding.shape[0]
    n_layer = len(layout.blocks)
    s = math.sqrt(3.0 / d)

    def view(spec):
        return theta[spec.offset:spec.offset + spec.size]

    def normal(spec, std):
        view(spec).normal_(0.0, std, generator=g)

    def uniform(spec, lo, hi):
        view(spec).uniform_(lo, hi, generator=g)

    normal(layout.embedding, 0.8)
    normal(layout.lm_head, 0.001)
    for i, blk in enumerate(layout.blocks):
        uniform(blk["wq"], -s, s)
        uniform(blk["wk"], -s, s)
        uniform(blk["wv"], -s, s)
        if all_nonzero:
            uniform(blk["wo"], -s, s)
        else:
            view(blk["wo"]).zero_()
        if blk["ve_table"] is not None:
            uniform(blk["ve_table"], -s, s)
            uniform(blk["ve_gate"], 0.0, 0.02)
        uniform(blk["fc"], -0.4 * s, 0.4 * s)
        if all_nonzero:
            uniform(blk["proj"], -0.4 * s, 0.4 * s)
        else:
            view(blk["proj"]).zero_()
        depth = float(i) / max(n_layer - 1, 1)
        view(blk["lam_b"]).fill_(1.15 - 0.10 * depth)
        view(blk["lam_x0"]).fill_(0.20 - 0.15 * depth)
    view(layout.lam_y).fill_(0.2)
    view(layout.lam_s).fill_(0.1 if all_nonzero else 0.0)
    uniform(layout.smear_gate, 0.0, 0.02)


class GradientState:
    """What `gradient_state` returns (ext/FemtoChatEnzymeExt.jl:27-36): built once per
    (config, batch shape), reused for every batch.  Owns the library handle."""

    def __init__(self, config: GPTConfig, max_batch: int, compute_type="float32", short_window: int = 0,
                 doc_mask: bool = False, index_base: int = 1, rank: int = 0, world: int = 1, nccl_id: bytes = None):
        import torch
        self.config = config
        self.max_batch = max_batch
        self.compute_type = compute_type
        self.c = config.c_struct(compute_dtype=compute_type, short_window=short_window, doc_mask=doc_mask,
                                 index_base=index_base, max_batch=max_batch)
        h = C.c_void_p()
        idbuf = C.create_string_buffer(nccl_id, 128) if nccl_id is not None else None
        _lib.check(_lib.lib().femto_create(C.byref(self.c), rank, world, idbuf, C.byref(h)))
        self.h = h
        self.rank, self.world = rank, world
        self._loss = torch.zeros(1, dtype=torch.float32, device="cuda")
        self._nvalid = torch.zeros(1, dtype=torch.int32, device="cuda")
        self._weights_of = None

    def refresh_weights(self, theta) -> None:
        _lib.check(_lib.lib().femto_refresh_weights(self.h, _lib.ptr(theta), _lib.stream_ptr()))

    def status_word(self) -> int:
        out = C.c_int32(0)
        _lib.check(_lib.lib().femto_status_word(self.h, C.byref(out)))
        return out.value

    def launch_count(self) -> int:
        return int(_lib.lib().femto_launch_count(self.h))

    def close(self) -> None:
        if self.h:
            _lib.lib().femto_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def gradient_state(params: Params, config: GPTConfig, layout: Layout, tokens, targets, positions=None, **options):
    """`gradient_state(params, config, layout, tokens, targets; positions)`: the batch shape
    (T, B) fixes the workspace; Θ is cast into the compute-type weights once here."""
    B, T = tokens.shape
    if T != config.sequence_len:
        raise ValueError(f"tokens have T={T}, config.sequence_len={config.sequence_len}")
    st = GradientState(config, max_batch=options.pop("max_batch", B), **options)
    st.refresh_weights(params.theta)
    return st


def _dev_i32(x):
    import torch
    if x is None:
        return None
    if not x.is_cuda:
        x = x.cuda(non_blocking=True)
    return x.to(torch.int32).contiguous()


def loss_and_gradient_(params: Params, state: GradientState, layout: Layout, tokens, targets, positions=None,
                       reduction: str = "sum", accumulate: bool = False, sync: bool = True, batch: int = None):
    """`loss_and_gradient!` (ext/FemtoChatEnzymeExt.jl:38-44): fills params.δ (or adds to it, as
    the training script's later micro-steps do, scripts/train.jl:117-131) and returns the loss.
    With sync=False returns the device scalars (loss, n_valid) without waiting."""
    if isinstance(tokens, C.c_void_p):    # device pointers handed out by a Feeder: batch = the feeder's
        if batch is None:
            raise ValueError("pass batch= with raw device pointers")
        ptok, ptgt, ppos, B = tokens, targets, positions, batch
    else:
        tok, tgt, pos = _dev_i32(tokens), _dev_i32(targets), _dev_i32(positions)
        ptok, ptgt, ppos, B = _lib.ptr(tok), _lib.ptr(tgt), _lib.ptr(pos), tok.shape[0]
    _lib.check(_lib.lib().femto_loss_and_gradient(
        state.h, _lib.ptr(params.theta), _lib.ptr(params.delta), ptok, ptgt, ppos, B,
        _lib.REDUCTION[reduction], 1 if accumulate else 0, _lib.ptr(state._loss), _lib.ptr(state._nvalid),
        _lib.stream_ptr()))
    if not sync:
        return state._loss, state._nvalid
    return float(state._loss.item())


def loss_and_gradient_host_(params: Params, state: GradientState, tokens_pinned, targets_pinned, positions_pinned,
                            reduction: str = "sum", accumulate: bool = False):
    """End-to-end call with HOST int32 [B][T] buffers: host→device copies, the step, and the read
    back of (loss, n_valid) all happen inside the library call."""
    B = tokens_pinned.shape[0]
    loss, nv = C.c_float(0), C.c_int32(0)
    _lib.check(_lib.lib().femto_loss_and_gradient_host(
        state.h, _lib.ptr(params.theta), _lib.ptr(params.delta), _lib.ptr(tokens_pinned), _lib.ptr(targets_pinned),
        _lib.ptr(positions_pinned), B, _lib.REDUCTION[reduction], 1 if accumulate else 0, C.byref(loss),
        C.byref(nv), _lib.stream_ptr()))
    return loss.value, nv.value


class GPT:
    """The `🤖` model call (src/parameters.jl:438-503, src/gpt.jl:196-199):
    `GPT(params, config, layout, compute_type=...)(tokens, targets, positions=..., reduction=...)`."""

    def __init__(self, params: Params, config: GPTConfig, layout: Layout, compute_type="float32", **options):
        self.params, self.config, self.layout = params, config, layout
        self.compute_type = compute_type
        self.options = options
        self._state: Optional[GradientState] = None

    def state(self, B: int) -> GradientState:
        if self._state is None or self._state.max_batch < B:
            self._state = GradientState(self.config, max_batch=B, compute_type=self.compute_type, **self.options)
        return self._state

    def __call__(self, tokens, targets=None, positions=None, reduction: str = "mean"):
        """With targets: the loss (src/gpt.jl:196-199).  Without: the soft-capped logits as a float32
        [B][T][vocab_size] tensor, the reference's (V,T,B) array (src/gpt.jl:129-170)."""
        if targets is None:
            return self.logits(tokens, positions)
        tok, tgt, pos = _dev_i32(tokens), _dev_i32(targets), _dev_i32(positions)
        st = self.state(tok.shape[0])
        st.refresh_weights(self.params.theta)
        if reduction == "none":   # per-token losses [B][T] (src/gpt.jl:191-193)
            import torch
            out = torch.empty(tok.shape[0], tok.shape[1], device="cuda", dtype=torch.float32)
            _lib.check(_lib.lib().femto_forward_token_losses(
                st.h, _lib.ptr(self.params.theta), _lib.ptr(tok), _lib.ptr(tgt), _lib.ptr(pos), tok.shape[0],
                _lib.ptr(out), None, _lib.stream_ptr()))
            return out
        _lib.check(_lib.lib().femto_forward_loss(
            st.h, _lib.ptr(self.params.theta), _lib.ptr(tok), _lib.ptr(tgt), _lib.ptr(pos), tok.shape[0],
            _lib.REDUCTION[reduction], _lib.ptr(st._loss), _lib.ptr(st._nvalid), _lib.stream_ptr()))
        return float(st._loss.item())

    def logits(self, tokens, positions=None):
        import torch
        tok, pos = _dev_i32(tokens), _dev_i32(positions)
        st = self.state(tok.shape[0])
        st.refresh_weights(self.params.theta)
        out = torch.empty(tok.shape[0], tok.shape[1], self.config.vocab_size, device="cuda", dtype=torch.float32)
        _lib.check(_lib.lib().femto_forward_logits(st.h, _lib.ptr(self.params.theta), _lib.ptr(tok), _lib.ptr(pos),
                                                   tok.shape[0], _lib.ptr(out), _lib.stream_ptr()))
        return out
