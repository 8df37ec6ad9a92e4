"""Host mirror of MuonAdamW (src/optim.jl:318-440).  The moments live in caller-owned torch
tensors, exposed per group in the reference's order so checkpoints round-trip
(src/checkpoints.jl:9-12); the update itself runs in the library."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

from . import _lib
from .gpt import GradientState
from .parameters import Layout, Params

POLAR_EXPRESS_COEFFS = (                       # src/optim.jl:90-96
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)
QUINTIC_COEFFS = tuple((3.4445, -4.7750, 2.0315) for _ in range(5))


SHARD_MIN_TABLE = 1 << 20


def shard_plan(layout, world: int, min_table: int = SHARD_MIN_TABLE):
    """The partition `MuonAdamW.shard` uses, as sorted (offset, count, owner) triplets: every AdamW table of at
    least 2^20 elements whose size divides by 4*world is cut into `world` equal slices (slice r to rank r); the Muon
    matrices of block i (of at least 1024 elements: the value-embedding gates are excepted) belong to rank
    i*world // n_layer, adjacent matrices of one owner merged into one range.
    Everything else (scalars, gates, small or indivisible tables) is updated by every rank (`min_table` is the
    library's fixed 2^20; tests lower it to cut small tables).  The reference has no
    data-parallel path (scripts/train.jl:13); the ranges follow its parameter layout (src/parameters.jl:219-337)."""
    if world <= 1:
        return []
    def size(sp):
        n = 1
        for x in sp.shape:
            n *= int(x)
        return n
    out = []
    tables = [layout.lm_head, layout.embedding] + [b["ve_table"] for b in layout.blocks if b["ve_table"] is not None]
    for sp in tables:
        n = size(sp)
        if n >= min_table and n % (4 * world) == 0:
            out += [(int(sp.offset) + r * (n // world), n // world, r) for r in range(world)]
    L = len(layout.blocks)
    mats = []
    for i, b in enumerate(layout.blocks):
        for k in ("wq", "wk", "wv", "wo", "fc", "proj", "ve_gate"):
            if b[k] is not None and size(b[k]) >= 1024:      # the tiny value-embedding gates stay with every rank
                mats.append((int(b[k].offset), size(b[k]), i * world // L))
    merged = []
    for off, n, owner in sorted(mats):
        if merged and merged[-1][2] == owner and merged[-1][0] + merged[-1][1] == off:
            merged[-1] = (merged[-1][0], merged[-1][1] + n, owner)
        else:
            merged.append((off, n, owner))
    return sorted(out + merged)


class _AdamGroupView:
    def __init__(self, owner, index, spec, m, v):
        self._owner, self._index, self.spec, self.m, self.v = owner, index, spec, m, v

    @property
    def t(self) -> int:
        return self._owner.get_t()[self._index]


class _MuonGroupView:
    def __init__(self, specs, m, v):
        self.specs, self.m, self.v = specs, m, v


class MuonAdamW:
    """`MuonAdamW(params, layout; unembedding_lr, embedding_lr, matrix_lr, weight_decay, scalar_lr,
    smear_lr, compute_type, t)` then `ω(; η, μ, λ, Nₜ)` as `.step(eta, mu, lam, Nt)`."""

    def __init__(self, params: Params, layout: Layout, state: GradientState, unembedding_lr=0.004, embedding_lr=0.2,
                 matrix_lr=0.02, weight_decay=0.0, scalar_lr=0.5, smear_lr=0.2, compute_type="float32", t: int = 0,
                 coeffs=POLAR_EXPRESS_COEFFS):
        import torch
        self.params, self.layout, self.state = params, layout, state
        L = _lib.lib()
        sizes = (C.c_int64 * 4)()
        _lib.check(L.femto_optimizer_state_sizes(state.h, sizes))
        dev = params.theta.device
        self.adam_m = torch.zeros(sizes[0], dtype=torch.float32, device=dev)
        self.adam_v = torch.zeros(sizes[1], dtype=torch.float32, device=dev)
        self.muon_m = torch.zeros(sizes[2], dtype=torch.float32, device=dev)
        self.muon_v = torch.zeros(sizes[3], dtype=torch.float32, device=dev)
        cfg = _lib.OptimizerConfig()
        cfg.unembedding_lr, cfg.embedding_lr, cfg.matrix_lr = unembedding_lr, embedding_lr, matrix_lr
        cfg.weight_decay, cfg.scalar_lr, cfg.smear_lr = weight_decay, scalar_lr, smear_lr
        cfg.ns_steps = len(coeffs)
        flat = [x for abc in coeffs for x in abc] + [0.0] * (15 - 3 * len(coeffs))
        cfg.ns_coeffs = (C.c_float * 15)(*flat)
        cfg.compute_dtype = _lib.BF16 if str(compute_type).endswith("bfloat16") or compute_type == "bf16" else _lib.F32
        o = C.c_void_p()
        _lib.check(L.femto_optimizer_create(state.h, C.byref(cfg), _lib.ptr(self.adam_m), _lib.ptr(self.adam_v),
                                            _lib.ptr(self.muon_m), _lib.ptr(self.muon_v), C.byref(o)))
        self.o = o
        # per-group views, in the reference's order (src/optim.jl:333-403, :405-425)
        specs = [layout.lm_head, layout.embedding]
        for blk in layout.blocks:
            if blk["ve_table"] is not None:
                specs.append(blk["ve_table"])
            specs += [blk["lam_b"], blk["lam_x0"]]
        specs += [layout.smear_gate, layout.lam_s, layout.lam_y]
        self.adamw: List[_AdamGroupView] = []
        off = 0
        for i, sp in enumerate(specs):
            self.adamw.append(_AdamGroupView(self, i, sp, self.adam_m[off:off + sp.size], self.adam_v[off:off + sp.size]))
            off += sp.size
        mspecs = []
        for blk in layout.blocks:
            mspecs += [blk["wq"], blk["wk"], blk["wv"], blk["wo"], blk["fc"], blk["proj"]]
            if blk["ve_gate"] is not None:
                mspecs.append(blk["ve_gate"])
        shapes = []
        for sp in mspecs:
            if sp.shape not in shapes:
                shapes.append(sp.shape)
        self.muon: List[_MuonGroupView] = []
        mo = vo = 0
        for shp in shapes:
            grp = [sp for sp in mspecs if sp.shape == shp]
            k, (m, n) = len(grp), shp
            # stacked Julia (m,n,k) column-major == row-major [k][n][m]
            mview = self.muon_m[mo:mo + k * m * n].view(k, n, m)
            vlen = m if m >= n else n
            vview = self.muon_v[vo:vo + k * vlen].view(k, vlen)
            self.muon.append(_MuonGroupView(grp, mview, vview))
            mo += k * m * n
            vo += k * vlen
        if t:
            self.set_t([t] * len(self.adamw))

    def step(self, eta: float = 1.0, mu: Optional[float] = None, lam: Optional[float] = None, Nt: float = 1.0):
        _lib.check(_lib.lib().femto_optimizer_step(
            self.o, _lib.ptr(self.params.theta), _lib.ptr(self.params.delta), float(eta), 0 if mu is None else 1,
            0.0 if mu is None else float(mu), 0 if lam is None else 1, 0.0 if lam is None else float(lam), float(Nt),
            _lib.stream_ptr()))

    __call__ = step

    def shard(self, rank: int, world: int):
        """Owner-sharded update for data parallelism (the reference is single-GPU, scripts/train.jl:13): this rank
        updates slice `rank` of every large AdamW table and the Muon matrices of its share of the blocks, and `step`
        exchanges the results over the handle's communicator.  `world == 1` restores the full update."""
        _lib.check(_lib.lib().femto_optimizer_set_shard(self.o, int(rank), int(world)))

    def set_exchange(self, mode: int):
        """What a sharded `step` exchanges: 0 = the fp32 Theta (complete on every rank after every update), 1 = only the
        model's compute-type weights (cheaper; call `gather_theta` before reading Theta on the host)."""
        _lib.check(_lib.lib().femto_optimizer_set_exchange(self.o, int(mode)))

    def gather_theta(self):
        """Under `shard` with exchange mode 1: complete the fp32 Theta on every rank."""
        _lib.check(_lib.lib().femto_optimizer_gather_theta(self.o, _lib.ptr(self.params.theta), _lib.stream_ptr()))

    def grad_sync(self, loss=None, n_valid=None):
        """Sum `params.delta` (and the device scalars `loss`, `n_valid`) over the ranks before `step`.  Under `shard`
        a range that one rank alone consumes is summed only onto that rank (half the bytes of an all-reduce)."""
        _lib.check(_lib.lib().femto_optimizer_grad_sync(
            self.o, _lib.ptr(self.params.delta), None if loss is None else _lib.ptr(loss),
            None if n_valid is None else _lib.ptr(n_valid), _lib.stream_ptr()))

    def gather_state(self):
        """Under `shard`: make the moment buffers complete on every rank (before `optimizer_state` for a checkpoint,
        src/checkpoints.jl:9-12, or before changing the sharding)."""
        _lib.check(_lib.lib().femto_optimizer_gather_state(self.o, _lib.stream_ptr()))

    def state_ranges(self, which: int):
        """(offset, count, owner) cover of a state buffer: 0 adam_m, 1 adam_v, 2 muon_m, 3 muon_v."""
        n = _lib.lib().femto_optimizer_state_ranges(self.o, int(which), None, 0)
        buf = (C.c_int64 * (3 * max(n, 1)))()
        _lib.lib().femto_optimizer_state_ranges(self.o, int(which), buf, n)
        return [(int(buf[3 * i]), int(buf[3 * i + 1]), int(buf[3 * i + 2])) for i in range(n)]

    def shard_ranges(self):
        """(offset, count, owner) of every range of Theta that a single rank updates under the current sharding."""
        n = _lib.lib().femto_optimizer_shard_ranges(self.o, None, 0)
        buf = (C.c_int64 * (3 * max(n, 1)))()
        _lib.lib().femto_optimizer_shard_ranges(self.o, buf, n)
        return [(int(buf[3 * i]), int(buf[3 * i + 1]), int(buf[3 * i + 2])) for i in range(n)]

    def get_t(self):
        n = len(self.adamw)
        buf = (C.c_int32 * n)()
        _lib.lib().femto_optimizer_get_t(self.o, buf, n)
        return list(buf)

    def set_t(self, ts):
        buf = (C.c_int32 * len(ts))(*ts)
        _lib.check(_lib.lib().femto_optimizer_set_t(self.o, buf, len(ts)))

    def close(self):
        if self.o:
            _lib.lib().femto_optimizer_destroy(self.o)
            self.o = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
