"""CPU oracle for the femtochat GPT training step.  TEST INFRASTRUCTURE ONLY.

This file is a restatement, in plain torch-on-CPU arithmetic (fp32 or fp64), of the
reference's Julia code for the training-step path: parameter layout, forward,
hand-written reverse pass, AdamW, Muon (Polar Express + MuonEq/Muon+/NorMuon) and the
step semantics.  It is the checker for the CUDA library; nothing the library ships may
call into it.  Each function cites the reference file:line it follows (paths are inside
the femtochat project).

PARITY UNPINNED: the reference ships no tests, golden vectors or recorded outputs for
this path, and no Julia toolchain was available to run it, so this restatement could
not be checked against the reference's own outputs.  It is trusted through internal
cross-checks only: the hand-written reverse pass against torch autograd of the restated
forward, naive attention against the blockwise FlashAttention-1 restatement, fp32
against fp64, finite differences, and structural known-answers derived from the source
(tiny README config has 27 690 parameters; d20 has 947 651 226).

Memory-layout rule: Julia arrays are column-major, so a Julia `(d, T, B)` array is
byte-identical to a row-major `[B][T][d]` tensor, and a weight of Julia shape
`(out, in)` is a row-major `[in][out]` matrix.  All tensors below are row-major torch
tensors in that sense; the flat parameter vector uses the reference's offsets exactly.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

IGNORE_INDEX = -1          # src/gpt.jl:172
SOFTCAP = 15.0             # src/gpt.jl:12
QK_GAIN = 1.2              # src/gpt.jl:105-106
ROPE_BASE = 100000.0       # src/parameters.jl:413
EPS_F32 = 2.0 ** -23       # eps(Float32), src/gpt.jl:16
EPS_BF16 = 2.0 ** -7       # eps(BFloat16)


# --------------------------------------------------------------------------------------
# Configuration and flat layout  (src/parameters.jl:71-80, 197-210, 219-337)
# --------------------------------------------------------------------------------------
@dataclass
class GPTConfig:
    """src/parameters.jl:71-80 (same field names and defaults)."""
    sequence_len: int = 2 ** 11
    max_document_tokens: int = 8192
    vocab_size: int = 2 ** 15
    n_layer: int = 12
    n_head: int = 6
    n_kv_head: int = 6
    n_embed: int = 768
    window_pattern: str = "SSSL"


@dataclass
class Spec:
    """One tensor of the flat vector: 0-based offset and the Julia (column-major) shape."""
    offset: int
    shape: Tuple[int, ...]

    @property
    def size(self) -> int:
        return int(math.prod(self.shape))


def has_ve(layer_idx: int, n_layer: int) -> bool:
    """src/parameters.jl:197-198; `layer_idx` is 1-based."""
    return (layer_idx - 1) % 2 == (n_layer - 1) % 2


def window_sizes(cfg: GPTConfig, short_window: int = 0) -> List[Tuple[int, int]]:
    """src/parameters.jl:200-210.  `short_window=0` keeps the reference rule
    S = min(L, cld(L, 512)*128); a positive value overrides S (benchmark configs)."""
    L = cfg.sequence_len
    S = min(L, -(-L // 512) * 128) if short_window <= 0 else min(L, short_window)
    pat = cfg.window_pattern
    w = [(S, 0) if pat[i % len(pat)] == "S" else (L, 0) for i in range(cfg.n_layer)]
    w[-1] = (L, 0)
    return w


@dataclass
class Layout:
    embedding: Spec
    blocks: List[Dict[str, Optional[Spec]]]
    lm_head: Spec
    smear_gate: Spec
    lam_s: Spec
    lam_y: Spec
    padded_vocab_size: int
    nparams: int


def parameter_layout(cfg: GPTConfig, pad_vocab_size_to: int = 64) -> Layout:
    """src/parameters.jl:219-337: the order in which tensors are taken from Θ."""
    assert cfg.n_embed % cfg.n_head == 0
    assert cfg.n_kv_head <= cfg.n_head and cfg.n_head % cfg.n_kv_head == 0
    pos = 0

    def take(*shape):
        nonlocal pos
        s = Spec(pos, tuple(shape))
        pos += s.size
        return s

    d = cfg.n_embed
    hd = d // cfg.n_head
    kv = cfg.n_kv_head * hd
    vp = -(-cfg.vocab_size // pad_vocab_size_to) * pad_vocab_size_to
    embedding = take(d, vp)
    blocks = []
    for li in range(1, cfg.n_layer + 1):
        ve = has_ve(li, cfg.n_layer)
        blk: Dict[str, Optional[Spec]] = {}
        blk["wq"] = take(d, d)
        blk["wk"] = take(kv, d)
        blk["wv"] = take(kv, d)
        blk["wo"] = take(d, d)
        blk["ve_gate"] = take(cfg.n_kv_head, 12) if ve else None
        blk["fc"] = take(4 * d, d)
        blk["proj"] = take(d, 4 * d)
        blk["ve_table"] = take(kv, vp) if ve else None
        blk["lam_b"] = take(1)
        blk["lam_x0"] = take(1)
        blocks.append(blk)
    lm_head = take(vp, d)
    smear_gate = take(1, 24)
    lam_s = take(1)
    lam_y = take(1)
    return Layout(embedding, blocks, lm_head, smear_gate, lam_s, lam_y, vp, pos)


def rm(theta: torch.Tensor, s: Spec) -> torch.Tensor:
    """Row-major view of a Julia `(rows, cols)` tensor: shape [cols][rows]."""
    flat = theta[s.offset:s.offset + s.size]
    if len(s.shape) == 1:
        return flat
    return flat.view(s.shape[1], s.shape[0])


def rotary_tables(seq_len: int, head_dim: int, dtype=torch.float32, base: float = ROPE_BASE):
    """src/parameters.jl:409-428: returns (sin, cos), each [seq_len][head_dim/2].
    The reference builds them in Float32 when Θ is Float32."""
    ch = torch.arange(0, head_dim, 2, dtype=torch.float32)
    t = torch.arange(seq_len, dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(base, dtype=torch.float32), ch / head_dim)
    freqs = t[:, None] * inv_freq[None, :]
    return torch.sin(freqs).to(dtype), torch.cos(freqs).to(dtype)


# --------------------------------------------------------------------------------------
# Initialisation  (src/gpt.jl:201-256)
# --------------------------------------------------------------------------------------
def initialize(theta: torch.Tensor, cfg: GPTConfig, layout: Layout, seed: int = 123,
               all_nonzero: bool = False) -> None:
    """Distributions and draw order of src/gpt.jl:220-256.  The reference's RNG stream
    cannot be regenerated outside Julia, so callers hand the SAME buffer to the oracle
    and to the library.  `all_nonzero=True` additionally randomises the two zero-init
    projections and sets λₛ = 0.1 so every gradient path carries signal."""
    g = torch.Generator().manual_seed(seed)
    d = layout.embedding.shape[0]
    n_layer = len(layout.blocks)
    s = math.sqrt(3.0 / d)

    def normal(spec, std):
        theta[spec.offset:spec.offset + spec.size] = (
            torch.randn(spec.size, generator=g, dtype=torch.float32) * std).to(theta.dtype)

    def uniform(spec, lo, hi):
        theta[spec.offset:spec.offset + spec.size] = (
            lo + (hi - lo) * torch.rand(spec.size, generator=g, dtype=torch.float32)).to(theta.dtype)

    def fill(spec, v):
        theta[spec.offset:spec.offset + spec.size] = v

    normal(layout.embedding, 0.8)
    normal(layout.lm_head, 0.001)
    for i, blk in enumerate(layout.blocks):
        uniform(blk["wq"], -s, s)
        uniform(blk["wk"], -s, s)
        uniform(blk["wv"], -s, s)
        if all_nonzero:
            uniform(blk["wo"], -s, s)
        else:
            fill(blk["wo"], 0.0)
        if blk["ve_table"] is not None:
            uniform(blk["ve_table"], -s, s)
            uniform(blk["ve_gate"], 0.0, 0.02)
        uniform(blk["fc"], -0.4 * s, 0.4 * s)
        if all_nonzero:
            uniform(blk["proj"], -0.4 * s, 0.4 * s)
        else:
            fill(blk["proj"], 0.0)
        depth = float(i) / max(n_layer - 1, 1)
        fill(blk["lam_b"], 1.15 - 0.10 * depth)
        fill(blk["lam_x0"], 0.20 - 0.15 * depth)
    fill(layout.lam_y, 0.2)
    fill(layout.lam_s, 0.1 if all_nonzero else 0.0)
    uniform(layout.smear_gate, 0.0, 0.02)


# --------------------------------------------------------------------------------------
# Element-level pieces of the forward  (src/gpt.jl:7-77)
# --------------------------------------------------------------------------------------
def norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    """src/gpt.jl:16-20: x / sqrt(mean(x²) + eps) over the embedding axis, no gain."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_backward(dy: torch.Tensor, x: torch.Tensor, eps: float) -> torch.Tensor:
    """ext/FemtoChatMooncakeExt.jl:248-255: dx = dy/r − x·(Σ dy·x)/(D r³)."""
    D = x.shape[-1]
    r = torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    dot = (dy * x).sum(dim=-1, keepdim=True)
    return dy / r - x * dot / (D * r ** 3)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """src/gpt.jl:55-77 (half-split rotation).  x: [B,T,H,hd]; cos/sin: [B,T,1,hd/2]."""
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat([x1 * cos + x2 * sin, -x1 * sin + x2 * cos], dim=-1)


def rope_backward(dy: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """ext/FemtoChatEnzymeExt.jl:168-169."""
    h = dy.shape[-1] // 2
    d1, d2 = dy[..., :h], dy[..., h:]
    return torch.cat([d1 * cos - d2 * sin, d1 * sin + d2 * cos], dim=-1)


def document_starts(positions: torch.Tensor) -> torch.Tensor:
    """Start row (0-based, within its batch column) of the document each token belongs
    to, derived from the positions reset: start = t − positions[t], clipped to 0 for a
    document that continues from an earlier batch (src/dataloader.jl:241-274)."""
    T = positions.shape[1]
    t = torch.arange(T, dtype=positions.dtype)[None, :]
    return torch.clamp(t - positions, min=0)


def attention_mask(T: int, window: Tuple[int, int], doc_start: Optional[torch.Tensor] = None):
    """src/kernels.jl:30-42.  Returns bool [T(query)][T(key)] (or [B,T,T] with documents):
    key allowed iff q−left ≤ k ≤ q+right; (-1,0) is plain causal.  With `doc_start`
    (not in the reference; benchmark option) also k ≥ start-of-document(q)."""
    left, right = window
    q = torch.arange(T)[:, None]
    k = torch.arange(T)[None, :]
    if window == (-1, 0):
        m = k <= q
    else:
        m = (q - left <= k) & (k <= q + right)
    if doc_start is not None:
        m = m[None] & (k[None] >= doc_start[:, :, None])
    return m


def naive_attention(Q, K, V, window, doc_start=None):
    """src/kernels.jl:59-96.  Q: [B,T,H,hd], K,V: [B,T,Hkv,hd].  kv head of head h
    (1-based) is cld(h, H/Hkv) (:69), i.e. 0-based h // group."""
    B, T, H, hd = Q.shape
    Hkv = K.shape[2]
    g = H // Hkv
    Kx = K.repeat_interleave(g, dim=2)
    Vx = V.repeat_interleave(g, dim=2)
    S = torch.einsum("bqhd,bkhd->bhqk", Q, Kx) / math.sqrt(hd)
    m = attention_mask(T, window, doc_start)
    m = m[None, None] if m.dim() == 2 else m[:, None]
    S = torch.where(m, S, torch.full_like(S, torch.finfo(S.dtype).min))
    P = torch.softmax(S, dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", P, Vx)


def flash_attention_forward(Q, K, V, window, doc_start=None, block: int = 512):
    """src/kernels.jl:131-219 (FlashAttention-1 blockwise forward), vectorised over
    batch and heads.  Returns O [B,T,H,hd] and the saved row statistics ℓ (running sum)
    and m (running max, natural-log units) as [B,H,T] — Julia's (1,T,H,B)."""
    B, T, H, hd = Q.shape
    Hkv = K.shape[2]
    g = H // Hkv
    Bc = Br = min(T, block)
    scale = 1.0 / math.sqrt(hd)
    F = Q.dtype
    fmax = torch.finfo(F).max
    O = torch.zeros_like(Q)
    l = torch.zeros(B, H, T, dtype=F)
    m = torch.full((B, H, T), -math.inf, dtype=F)
    full_mask = attention_mask(T, window, doc_start)   # [T,T] or [B,T,T], (q,k)
    for j0 in range(0, T, Bc):
        j1 = min(j0 + Bc, T)
        Kj = K[:, j0:j1].repeat_interleave(g, dim=2)
        Vj = V[:, j0:j1].repeat_interleave(g, dim=2)
        for i0 in range(0, T, Br):
            i1 = min(i0 + Br, T)
            Mij = full_mask[..., i0:i1, j0:j1]
            Mij = Mij[None, None] if Mij.dim() == 2 else Mij[:, None]
            S = torch.einsum("bqhd,bkhd->bhqk", Q[:, i0:i1], Kj) * scale
            S = torch.where(Mij, S, torch.full_like(S, -fmax))
            mt = S.max(dim=-1).values
            P = torch.where(Mij, torch.exp(S - mt[..., None]), torch.zeros_like(S))
            lt = P.sum(dim=-1)
            mi, li = m[:, :, i0:i1], l[:, :, i0:i1]
            mnew = torch.maximum(mi, mt)
            em = torch.exp(mi - mnew)
            emt = torch.exp(mt - mnew)
            lnew = em * li + emt * lt
            Ot = torch.einsum("bhqk,bkhd->bqhd", P, Vj)
            Oi = O[:, i0:i1]
            num = Oi * (li * em).permute(0, 2, 1)[..., None] + Ot * emt.permute(0, 2, 1)[..., None]
            O[:, i0:i1] = num / torch.clamp(lnew, min=torch.finfo(F).eps).permute(0, 2, 1)[..., None]
            m[:, :, i0:i1] = mnew
            l[:, :, i0:i1] = lnew
    return O, l, m


def flash_attention_backward(dO, Q, K, V, O, l, m, window, doc_start=None, block: int = 512):
    """src/kernels.jl:287-379 (FlashAttention-1 backward): returns dQ, dK, dV."""
    B, T, H, hd = Q.shape
    Hkv = K.shape[2]
    g = H // Hkv
    Bc = Br = min(T, block)
    scale = 1.0 / math.sqrt(hd)
    F = Q.dtype
    fmax = torch.finfo(F).max
    dQ = torch.zeros_like(Q)
    dK = torch.zeros_like(K)
    dV = torch.zeros_like(V)
    full_mask = attention_mask(T, window, doc_start)
    Dall = (dO * O).sum(dim=-1).permute(0, 2, 1)            # [B,H,T]  (:363-364)
    for j0 in range(0, T, Bc):
        j1 = min(j0 + Bc, T)
        Kj = K[:, j0:j1].repeat_interleave(g, dim=2)
        Vj = V[:, j0:j1].repeat_interleave(g, dim=2)
        for i0 in range(0, T, Br):
            i1 = min(i0 + Br, T)
            Mij = full_mask[..., i0:i1, j0:j1]
            Mij = Mij[None, None] if Mij.dim() == 2 else Mij[:, None]
            S = torch.einsum("bqhd,bkhd->bhqk", Q[:, i0:i1], Kj) * scale
            S = torch.where(Mij, S, torch.full_like(S, -fmax))
            li = torch.clamp(l[:, :, i0:i1], min=torch.finfo(F).eps)
            P = torch.where(Mij, torch.exp(S - m[:, :, i0:i1, None]) / li[..., None],
                            torch.zeros_like(S))
            dOi = dO[:, i0:i1]
            dVt = torch.einsum("bhqk,bqhd->bkhd", P, dOi)
            dP = torch.einsum("bqhd,bkhd->bhqk", dOi, Vj)
            dS = P * (dP - Dall[:, :, i0:i1, None])
            dQ[:, i0:i1] += scale * torch.einsum("bhqk,bkhd->bqhd", dS, Kj)
            dKt = scale * torch.einsum("bhqk,bqhd->bkhd", dS, Q[:, i0:i1])
            dK[:, j0:j1] += dKt.reshape(B, j1 - j0, Hkv, g, hd).sum(dim=3)
            dV[:, j0:j1] += dVt.reshape(B, j1 - j0, Hkv, g, hd).sum(dim=3)
    return dQ, dK, dV


# --------------------------------------------------------------------------------------
# Whole-model forward + hand-written reverse pass
# --------------------------------------------------------------------------------------
@dataclass
class StepOptions:
    eps: float = EPS_F32          # eps(activation type): 2^-23 for fp32, 2^-7 for bf16 runs
    short_window: int = 0         # 0 = reference rule
    doc_mask: bool = False        # False = reference (attention crosses documents)
    reduction: str = "sum"        # "sum" (training script) | "mean" (model call default)
    index_base: int = 1           # tokens/targets are 1-based in the reference


class Model:
    """Restated `🤖` (src/parameters.jl:438-503, src/gpt.jl:129-199) over a flat Θ."""

    def __init__(self, cfg: GPTConfig, opts: Optional[StepOptions] = None):
        self.cfg = cfg
        self.opts = opts or StepOptions()
        self.layout = parameter_layout(cfg)
        self.windows = window_sizes(cfg, self.opts.short_window)
        self.hd = cfg.n_embed // cfg.n_head
        self.backout_layer = cfg.n_layer // 2 + 1          # 1-based, src/gpt.jl:145
        self._rope = {}

    def rope(self, dtype):
        if dtype not in self._rope:
            self._rope[dtype] = rotary_tables(self.cfg.max_document_tokens, self.hd, dtype)
        return self._rope[dtype]

    # -- forward, written with differentiable torch ops so autograd can cross-check ----
    def forward(self, theta, tokens, targets, positions=None, attention="flash", cache=None):
        cfg, lay, o = self.cfg, self.layout, self.opts
        B, T = tokens.shape
        d, H, Hkv, hd = cfg.n_embed, cfg.n_head, cfg.n_kv_head, self.hd
        F = theta.dtype
        tok = (tokens - o.index_base).long()
        if positions is None:
            positions = torch.arange(T, dtype=torch.int64)[None, :].expand(B, T)
        positions = positions.long()
        sin_t, cos_t = self.rope(F)
        sin = sin_t[positions][:, :, None, :]                  # src/gpt.jl:44-49
        cos = cos_t[positions][:, :, None, :]
        doc_start = document_starts(positions) if o.doc_mask else None
        c = cache if cache is not None else {}
        c.update(tok=tok, sin=sin, cos=cos, doc_start=doc_start, B=B, T=T)

        E = rm(theta, lay.embedding)[tok]                      # src/gpt.jl:34,134
        xe = norm(E, o.eps)                                    # :136
        w_s = rm(theta, lay.smear_gate)                        # [24][1]
        lam_s = theta[lay.lam_s.offset]
        sg = torch.sigmoid(xe[:, 1:, :24] @ w_s)[..., 0]       # :139
        gate = lam_s * sg
        x0 = torch.cat([xe[:, :1], xe[:, 1:] + gate[..., None] * xe[:, :-1]], dim=1)  # :118-122
        c.update(E=E, xe=xe, sg=sg, gate=gate, x0=x0, layers=[])
        x = x0
        xb = None
        for i, blk in enumerate(lay.blocks):
            L = {}
            lam_b = theta[blk["lam_b"].offset]
            lam_x0 = theta[blk["lam_x0"].offset]
            xin = x
            xm = lam_b * xin + lam_x0 * x0                      # :148
            xn1 = norm(xm, o.eps)                               # :114
            q = (xn1 @ rm(theta, blk["wq"])).view(B, T, H, hd)  # :86-88
            k = (xn1 @ rm(theta, blk["wk"])).view(B, T, Hkv, hd)
            v = (xn1 @ rm(theta, blk["wv"])).view(B, T, Hkv, hd)
            if blk["ve_table"] is not None:
                VE = rm(theta, blk["ve_table"])[tok].view(B, T, Hkv, hd)   # :152
                sv = torch.sigmoid(xn1[..., :12] @ rm(theta, blk["ve_gate"]))  # :97
                v = v + (3.0 * sv)[..., None] * VE              # :98
                L.update(VE=VE, sv=sv)
            qr = apply_rope(q, cos, sin)                        # :103-104
            kr = apply_rope(k, cos, sin)
            qn = QK_GAIN * norm(qr, o.eps)                      # :105-106
            kn = QK_GAIN * norm(kr, o.eps)
            if attention == "naive":
                att = naive_attention(qn, kn, v, self.windows[i], doc_start)
            else:
                att, l_, m_ = flash_attention_forward(qn, kn, v, self.windows[i], doc_start)
                L.update(l=l_, m=m_)
            xa = xm + att.reshape(B, T, d) @ rm(theta, blk["wo"])   # :110,114
            xn2 = norm(xa, o.eps)                               # :115
            u = xn2 @ rm(theta, blk["fc"])                      # :36-40
            a = torch.clamp(u, min=0) ** 2
            xo = xa + a @ rm(theta, blk["proj"])
            L.update(xin=xin, xm=xm, xn1=xn1, qr=qr, kr=kr, qn=qn, kn=kn, v=v, att=att,
                     xa=xa, xn2=xn2, u=u, a=a)
            c["layers"].append(L)
            x = xo
            if i + 1 == self.backout_layer:
                xb = x                                          # :155-157
        lam_y = theta[lay.lam_y.offset]
        xf = x - lam_y * xb                                     # :160-162
        xnf = norm(xf, o.eps)                                   # :165
        Wlm = rm(theta, lay.lm_head)[:, :cfg.vocab_size]        # [d][V], padded rows sliced (:168)
        z = SOFTCAP * torch.tanh((xnf @ Wlm) / SOFTCAP)         # :169
        valid = targets != IGNORE_INDEX                         # :177
        tgt = torch.where(valid, targets - o.index_base, torch.zeros_like(targets)).long()
        lse = torch.logsumexp(z, dim=-1)
        losses = lse - torch.gather(z, -1, tgt[..., None])[..., 0]
        losses = torch.where(valid, losses, torch.zeros_like(losses))
        nvalid = int(valid.sum())
        if o.reduction == "mean":
            loss = losses.sum() / nvalid
        elif o.reduction == "sum":
            loss = losses.sum()
        else:
            loss = losses
        c.update(xb=xb, xlast=x, xf=xf, xnf=xnf, z=z, lse=lse, valid=valid, tgt=tgt, nvalid=nvalid,
                 losses=losses)
        return loss

    # -- hand-written reverse pass (the schedule the CUDA library implements) ----------
    @torch.no_grad()
    def loss_and_gradient(self, theta, tokens, targets, positions=None, delta=None,
                          accumulate=False):
        """`loss_and_gradient!` (ext/FemtoChatEnzymeExt.jl:38-44): returns the loss and
        fills δ with its gradient.  With `accumulate` δ is added to, as the training
        script's later micro-steps do (scripts/train.jl:117-131)."""
        cfg, lay, o = self.cfg, self.layout, self.opts
        assert o.reduction in ("sum", "mean")
        c = {}
        loss = self.forward(theta, tokens, targets, positions, attention="flash", cache=c)
        B, T = c["B"], c["T"]
        d, H, Hkv, hd = cfg.n_embed, cfg.n_head, cfg.n_kv_head, self.hd
        V = cfg.vocab_size
        if delta is None:
            delta = torch.zeros(lay.nparams, dtype=torch.float32)
        g = torch.zeros(lay.nparams, dtype=theta.dtype)
        tok, sin, cos = c["tok"], c["sin"], c["cos"]
        x0 = c["x0"]

        # cross-entropy and softcap reverse  (src/kernels.jl:16-28, EnzymeExt:175-189)
        w = 1.0 if o.reduction == "sum" else 1.0 / c["nvalid"]
        z = c["z"]
        p = torch.exp(z - c["lse"][..., None])
        dz = p
        dz.scatter_add_(-1, c["tgt"][..., None], -torch.ones_like(c["tgt"][..., None], dtype=z.dtype))
        dz = torch.where(c["valid"][..., None], w * dz, torch.zeros_like(dz))
        dlog = dz * (1.0 - (z / SOFTCAP) ** 2)
        Wlm_full = rm(theta, lay.lm_head)
        gW = rm(g, lay.lm_head)
        gW[:, :V] += c["xnf"].reshape(-1, d).T @ dlog.reshape(-1, V)      # EnzymeExt:100
        dxnf = dlog @ Wlm_full[:, :V].T                                   # :101
        dxf = norm_backward(dxnf, c["xf"], o.eps)
        lam_y = theta[lay.lam_y.offset]
        g[lay.lam_y.offset] += -(dxf * c["xb"]).sum()
        dx = dxf.clone()
        dxb = -lam_y * dxf
        dx0 = torch.zeros_like(x0)
        for i in reversed(range(cfg.n_layer)):
            blk, L = lay.blocks[i], c["layers"][i]
            if i + 1 == self.backout_layer:
                dx = dx + dxb
            # MLP reverse  (ext/FemtoChatEnzymeExt.jl:121-134)
            rm(g, blk["proj"]).add_(L["a"].reshape(-1, 4 * d).T @ dx.reshape(-1, d))
            da = dx @ rm(theta, blk["proj"]).T
            du = da * 2.0 * torch.clamp(L["u"], min=0)
            rm(g, blk["fc"]).add_(L["xn2"].reshape(-1, d).T @ du.reshape(-1, 4 * d))
            dxn2 = du @ rm(theta, blk["fc"]).T
            dxa = dx + norm_backward(dxn2, L["xa"], o.eps)
            # attention output projection
            rm(g, blk["wo"]).add_(L["att"].reshape(-1, d).T @ dxa.reshape(-1, d))
            datt = (dxa @ rm(theta, blk["wo"]).T).view(B, T, H, hd)
            dqn, dkn, dv = flash_attention_backward(
                datt, L["qn"], L["kn"], L["v"], L["att"], L["l"], L["m"], self.windows[i],
                c["doc_start"])
            dq = rope_backward(norm_backward(QK_GAIN * dqn, L["qr"], o.eps), cos, sin)
            dk = rope_backward(norm_backward(QK_GAIN * dkn, L["kr"], o.eps), cos, sin)
            xn1 = L["xn1"]
            dxn1 = torch.zeros_like(xn1)
            if blk["ve_table"] is not None:
                sv, VE = L["sv"], L["VE"]
                dgate = (dv * VE).sum(dim=-1)                    # [B,T,Hkv]
                dVE = (3.0 * sv)[..., None] * dv
                rm(g, blk["ve_table"]).index_add_(0, tok.reshape(-1), dVE.reshape(-1, Hkv * hd))
                dpre = dgate * 3.0 * sv * (1.0 - sv)
                rm(g, blk["ve_gate"]).add_(xn1[..., :12].reshape(-1, 12).T @ dpre.reshape(-1, Hkv))
                dxn1[..., :12] += dpre @ rm(theta, blk["ve_gate"]).T
            x2 = xn1.reshape(-1, d)
            rm(g, blk["wq"]).add_(x2.T @ dq.reshape(-1, d))
            rm(g, blk["wk"]).add_(x2.T @ dk.reshape(-1, Hkv * hd))
            rm(g, blk["wv"]).add_(x2.T @ dv.reshape(-1, Hkv * hd))
            dxn1 += (dq.reshape(B, T, d) @ rm(theta, blk["wq"]).T
                     + dk.reshape(B, T, -1) @ rm(theta, blk["wk"]).T
                     + dv.reshape(B, T, -1) @ rm(theta, blk["wv"]).T)
            dxm = dxa + norm_backward(dxn1, L["xm"], o.eps)
            g[blk["lam_b"].offset] += (dxm * L["xin"]).sum()
            g[blk["lam_x0"].offset] += (dxm * x0).sum()
            dx0 += theta[blk["lam_x0"].offset] * dxm
            dx = theta[blk["lam_b"].offset] * dxm
        dx0 += dx
        # smear reverse  (ext/FemtoChatMooncakeExt.jl:57-73) and its gate
        xe, sg, gate = c["xe"], c["sg"], c["gate"]
        dxe = dx0.clone()
        dxe[:, :-1] += gate[..., None] * dx0[:, 1:]
        dgate = (dx0[:, 1:] * xe[:, :-1]).sum(dim=-1)
        lam_s = theta[lay.lam_s.offset]
        g[lay.lam_s.offset] += (dgate * sg).sum()
        dpre = dgate * lam_s * sg * (1.0 - sg)
        rm(g, lay.smear_gate).add_((xe[:, 1:, :24].reshape(-1, 24).T @ dpre.reshape(-1, 1)))
        dxe[:, 1:, :24] += dpre[..., None] * rm(theta, lay.smear_gate)[:, 0]
        dE = norm_backward(dxe, c["E"], o.eps)
        # embedding scatter  (src/kernels.jl:8-14)
        rm(g, lay.embedding).index_add_(0, tok.reshape(-1), dE.reshape(-1, d))
        if accumulate:
            delta += g.to(torch.float32)
        else:
            delta.copy_(g.to(torch.float32))
        return float(loss), delta, c

    def loss_and_gradient_autograd(self, theta, tokens, targets, positions=None):
        """Independent check: torch autograd through the restated forward with the
        naive attention of src/kernels.jl:59-96."""
        th = theta.clone().requires_grad_(True)
        loss = self.forward(th, tokens, targets, positions, attention="naive")
        loss.backward()
        return float(loss.detach()), th.grad.detach().to(torch.float32)


# --------------------------------------------------------------------------------------
# Optimiser  (src/optim.jl)
# --------------------------------------------------------------------------------------
POLAR_EXPRESS_COEFFS = (                       # src/optim.jl:90-96
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)
QUINTIC_COEFFS = tuple((3.4445, -4.7750, 2.0315) for _ in range(5))


def polar_express(G: torch.Tensor, coeffs=POLAR_EXPRESS_COEFFS, compute_dtype=None):
    """src/optim.jl:131-149 on a stack [k][rows][cols] given in the JULIA orientation
    (rows = Julia dim 1).  Normalise by 1.01‖G‖_F + 1e-6, orient so rows ≤ cols, then
    X ← aX + (bA + cA²)X with A = XXᵀ, per step."""
    m, n = G.shape[-2], G.shape[-1]
    transposed = m > n
    scale = 1.01 * torch.sqrt((G.float() ** 2).sum(dim=(-2, -1), keepdim=True)) + 1e-6
    X = (G.transpose(-1, -2) if transposed else G) / scale
    if compute_dtype is not None:
        X = X.to(compute_dtype)
    for a, b, c in coeffs:
        A = X @ X.transpose(-1, -2)
        Bm = b * A + c * (A @ A)
        X = a * X + Bm @ X
    X = X.to(G.dtype)
    return X.transpose(-1, -2) if transposed else X


def julia_stack(vec: torch.Tensor, specs: List[Spec]) -> torch.Tensor:
    """Gather same-shape matrices into [k][m][n] in the Julia orientation
    (src/optim.jl:259-265): Julia (m,n) column-major = row-major [n][m], transposed."""
    m, n = specs[0].shape
    return torch.stack([vec[s.offset:s.offset + s.size].view(n, m).T for s in specs])


class AdamWState:
    def __init__(self, spec, alpha, b1, b2, eps, lam):
        self.spec, self.alpha, self.b1, self.b2, self.eps, self.lam = spec, alpha, b1, b2, eps, lam
        self.m = torch.zeros(spec.size, dtype=torch.float32)
        self.v = torch.zeros(spec.size, dtype=torch.float32)
        self.t = 0


class MuonState:
    def __init__(self, specs, alpha, mu, b2, lam, steps=5):
        self.specs, self.alpha, self.mu, self.b2, self.lam, self.steps = specs, alpha, mu, b2, lam, steps
        m, n = specs[0].shape
        k = len(specs)
        self.m = torch.zeros(k, m, n, dtype=torch.float32)
        self.v = torch.zeros((k, m, 1) if m >= n else (k, 1, n), dtype=torch.float32)   # :180


class MuonAdamW:
    """src/optim.jl:318-440: group construction order and the step."""

    def __init__(self, layout: Layout, unembedding_lr=0.004, embedding_lr=0.2, matrix_lr=0.02,
                 weight_decay=0.0, scalar_lr=0.5, smear_lr=0.2, coeffs=POLAR_EXPRESS_COEFFS,
                 compute_dtype=None):
        D = layout.embedding.shape[0]
        scale = math.sqrt(768.0 / D)
        A = AdamWState
        self.adamw = [A(layout.lm_head, unembedding_lr * scale, 0.8, 0.96, 1e-10, 0.01),
                      A(layout.embedding, embedding_lr * scale, 0.8, 0.995, 1e-10, 0.001)]
        for blk in layout.blocks:
            if blk["ve_table"] is not None:
                self.adamw.append(A(blk["ve_table"], 0.5 * embedding_lr * scale, 0.8, 0.995, 1e-10, 0.01))
            self.adamw.append(A(blk["lam_b"], 0.01 * scalar_lr, 0.8, 0.95, 1e-10, 0.05))
            self.adamw.append(A(blk["lam_x0"], scalar_lr, 0.96, 0.95, 1e-10, 0.0))
        for spec in (layout.smear_gate, layout.lam_s, layout.lam_y):
            self.adamw.append(A(spec, smear_lr, 0.8, 0.95, 1e-10, 0.0))
        muon_specs = []
        for blk in layout.blocks:
            muon_specs += [blk["wq"], blk["wk"], blk["wv"], blk["wo"], blk["fc"], blk["proj"]]
            if blk["ve_gate"] is not None:
                muon_specs.append(blk["ve_gate"])
        shapes = []
        for s in muon_specs:
            if s.shape not in shapes:
                shapes.append(s.shape)
        self.muon = [MuonState([s for s in muon_specs if s.shape == shp], matrix_lr, 0.95, 0.9,
                               weight_decay) for shp in shapes]
        self.coeffs = coeffs
        self.compute_dtype = compute_dtype

    @torch.no_grad()
    def step(self, theta, delta, eta=1.0, mu=None, lam=None, Nt=1.0):
        f32 = torch.float32
        for st in self.adamw:                                   # :431-433 → :75-87
            sl = slice(st.spec.offset, st.spec.offset + st.spec.size)
            g = delta[sl].to(f32) / Nt
            st.t += 1
            st.m.mul_(st.b1).add_((1 - st.b1) * g)
            st.v.mul_(st.b2).add_((1 - st.b2) * g * g)
            alpha = eta * st.alpha
            th = theta[sl].to(f32) * (1.0 - alpha * st.lam)
            th = th - alpha * (st.m / (1 - st.b1 ** st.t)) / (torch.sqrt(st.v / (1 - st.b2 ** st.t)) + st.eps)
            theta[sl] = th.to(theta.dtype)
        for st in self.muon:                                    # :434-438
            self._muon_group(st, theta, delta, eta * st.alpha, st.mu if mu is None else mu,
                             st.lam if lam is None else lam, Nt)

    def muon_direction(self, st: MuonState, G: torch.Tensor, mu: float, Nt: float):
        """src/optim.jl:198-236; G is [k][m][n] (Julia orientation), fp32."""
        k, m, n = G.shape
        g = G / Nt
        st.m.mul_(mu).add_((1 - mu) * g)                         # Nesterov (:206-207)
        X = (1 - mu) * g + mu * st.m
        old = (X ** 2).sum(dim=(1, 2), keepdim=True)             # MuonEq (:210-212)
        row = (X ** 2).sum(dim=2, keepdim=True)
        X = X * (torch.sqrt(old / m) / torch.clamp(torch.sqrt(row), min=1e-6))
        X = polar_express(X, self.coeffs, self.compute_dtype)    # :215
        old = (X ** 2).sum(dim=(1, 2), keepdim=True)             # Muon+ (:218-219)
        X = X * (math.sqrt(float(min(m, n))) / torch.clamp(torch.sqrt(old), min=1e-6))
        dim = 2 if m >= n else 1                                 # NorMuon (:222-233)
        dsize = X.shape[dim]
        v_mean = (X ** 2).sum(dim=dim, keepdim=True) / dsize
        st.v.mul_(st.b2).add_((1 - st.b2) * v_mean)
        step_size = 1.0 / torch.sqrt(torch.clamp(st.v, min=1e-10))
        old = (X ** 2).sum(dim=(1, 2), keepdim=True)
        new = (dsize * v_mean * step_size ** 2).sum(dim=(1, 2), keepdim=True)
        X = X * (step_size * torch.sqrt(old) / torch.clamp(torch.sqrt(new), min=1e-10))
        return X

    def _muon_group(self, st, theta, delta, alpha, mu, lam, Nt):
        G = julia_stack(delta.to(torch.float32), st.specs)
        X = self.muon_direction(st, G, mu, Nt)
        m, n = st.specs[0].shape
        eta = alpha * math.sqrt(max(1.0, m / n))                 # :244
        for j, s in enumerate(st.specs):
            th = theta[s.offset:s.offset + s.size].view(n, m).T.to(torch.float32)
            x = X[j]
            th = th - (eta * x + eta * lam * th * ((x * th) >= 0))   # :245 cautious decay
            theta[s.offset:s.offset + s.size] = th.T.contiguous().view(-1).to(theta.dtype)


# --------------------------------------------------------------------------------------
# Schedules and the FLOP model  (src/scaling.jl)
# --------------------------------------------------------------------------------------
def num_scaling_params(layout: Layout):
    """src/scaling.jl:7-28."""
    n = lambda s: 0 if s is None else s.size
    ve = sum(n(b["ve_table"]) for b in layout.blocks)
    mats = sum(n(b[k]) for b in layout.blocks for k in ("wq", "wk", "wv", "wo", "ve_gate", "fc", "proj"))
    scalars = layout.smear_gate.size + layout.lam_s.size + layout.lam_y.size + 2 * len(layout.blocks)
    wte, lm = layout.embedding.size, layout.lm_head.size
    return dict(wte=wte, value_embeds=ve, lm_head=lm, transformer_matrices=mats, scalars=scalars,
                total=wte + ve + lm + mats + scalars)


def num_matmul_params(layout: Layout) -> int:
    """src/scaling.jl:30-33."""
    c = num_scaling_params(layout)
    return c["transformer_matrices"] + c["lm_head"] + layout.smear_gate.size


def estimate_flops(cfg: GPTConfig, short_window: int = 0) -> int:
    """src/scaling.jl:33-43: FLOPs per token = 6·matmul params + Σ 12·n_embed·min(window,T)."""
    layout = parameter_layout(cfg)
    att = sum(12 * cfg.n_embed * (cfg.sequence_len if w < 0 else min(w, cfg.sequence_len))
              for w, _ in window_sizes(cfg, short_window))
    return 6 * num_matmul_params(layout) + att


def training_schedule(step: int, steps: int, warmup_steps=40, warmdown_ratio=0.65, final_lr_frac=0.05):
    """src/scaling.jl:59-78; `step` counts completed updates from zero."""
    warmdown = round(warmdown_ratio * steps)
    start = steps - warmdown
    if step < warmup_steps:
        eta = (step + 1) / warmup_steps
    elif step <= start:
        eta = 1.0
    else:
        p = (steps - step) / warmdown
        eta = p + (1 - p) * final_lr_frac
    if step < 400:
        mu = 0.85 + (0.97 - 0.85) * step / 400
    elif step >= start and warmdown > 0:
        mu = 0.97 + (0.90 - 0.97) * (step - start) / warmdown
    else:
        mu = 0.97
    lam = (1 + math.cos(math.pi * step / steps)) / 2
    return eta, mu, lam
