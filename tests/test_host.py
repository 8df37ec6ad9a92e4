"""CPU checks of the host mirror and of the C ABI surface (no GPU compute)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import femtochat_b200 as fb
from femtochat_b200 import _lib
from oracle import femto_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CONFIGS = [
    dict(sequence_len=4, max_document_tokens=64, vocab_size=16, n_layer=2, n_head=2, n_kv_head=1, n_embed=32, window_pattern="L"),
    dict(sequence_len=2048, vocab_size=65536, n_layer=12, n_head=6, n_kv_head=6, n_embed=768, window_pattern="L"),
    dict(sequence_len=2048, vocab_size=65536, n_layer=20, n_head=10, n_kv_head=5, n_embed=1280, window_pattern="SSSL"),
    dict(sequence_len=2048, vocab_size=65536, n_layer=26, n_head=13, n_kv_head=13, n_embed=1664, window_pattern="SSSL"),
    dict(sequence_len=96, vocab_size=100, n_layer=3, n_head=4, n_kv_head=2, n_embed=64, window_pattern="SL"),
]


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "femto.h")).read()
    declared = set(re.findall(r"\b(femto_[a-z0-9_]+)\s*\(", hdr))
    declared -= {"femto_handle", "femto_optimizer"}
    L = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in include/femto.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert _lib.lib().femto_version() == 100


@pytest.mark.parametrize("kw", CONFIGS)
def test_layout_matches_oracle(kw):
    lay = fb.parameter_layout(fb.GPTConfig(**kw))
    ref = fo.parameter_layout(fo.GPTConfig(**kw))
    assert lay.nparams == ref.nparams and lay.padded_vocab_size == ref.padded_vocab_size
    assert (lay.embedding.offset, lay.embedding.shape) == (ref.embedding.offset, ref.embedding.shape)
    assert (lay.lm_head.offset, lay.lm_head.shape) == (ref.lm_head.offset, ref.lm_head.shape)
    assert lay.smear_gate.offset == ref.smear_gate.offset and lay.lam_s.offset == ref.lam_s.offset
    assert lay.lam_y.offset == ref.lam_y.offset
    for a, b in zip(lay.blocks, ref.blocks):
        for k in a:
            if b[k] is None:
                assert a[k] is None
            else:
                assert a[k].offset == b[k].offset and a[k].size == b[k].size, k
    assert fb.window_sizes(fb.GPTConfig(**kw)) == fo.window_sizes(fo.GPTConfig(**kw))
    assert fb.window_sizes(fb.GPTConfig(**kw), short_window=1024) == fo.window_sizes(fo.GPTConfig(**kw), 1024)
    assert fb.estimate_flops(fb.GPTConfig(**kw)) == fo.estimate_flops(fo.GPTConfig(**kw))


def test_bad_configs_are_rejected_with_messages():
    with pytest.raises(_lib.FemtoError, match="n_head"):
        fb.parameter_layout(fb.GPTConfig(n_embed=100, n_head=3))
    with pytest.raises(_lib.FemtoError, match="window_pattern"):
        fb.parameter_layout(fb.GPTConfig(window_pattern="SX"))


def test_no_cpu_fallback():
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    cfg = fb.GPTConfig(**CONFIGS[0])
    with pytest.raises(_lib.FemtoError, match="no CUDA device"):
        fb.GradientState(cfg, 2)


def test_schedules_match_oracle():
    for step, steps in ((0, 100), (39, 100), (40, 100), (77, 100), (399, 1000), (400, 1000), (999, 1000)):
        s = fb.training_schedule(step, steps)
        assert (s["eta"], s["mu"], s["lam"]) == pytest.approx(fo.training_schedule(step, steps))


def test_packed_batches_follow_loader_format():
    V, T, B = 4096, 256, 4
    pk = fb.PackedBatches(V, T, B, max_document_tokens=300, mean_doc_len=40, seed=1)
    bos = fb.bos_token_id(V)
    assert bos == V - 8
    prev = None
    for _ in range(3):
        tok, tgt, pos = pk.next()
        assert tok.shape == (B, T) and tok.dtype == np.int32
        assert tok.min() >= 1 and tok.max() <= bos and (tgt != -1).all()
        assert (tgt[:, :-1] == tok[:, 1:]).all()                  # targets are the next token of the stream
        starts = tok == bos
        assert (pos[starts] == 0).all()                             # positions restart on BOS
        cont = ~starts[:, 1:]
        assert (pos[:, 1:][cont] == pos[:, :-1][cont] + 1).all()
        assert pos.max() < 300
        if prev is not None:                                        # documents continue across batches
            ptok, ptgt, ppos = prev
            assert (ptgt[:, -1] == tok[:, 0]).all()
            c = tok[:, 0] != bos
            assert (pos[c, 0] == ppos[c, -1] + 1).all()
        prev = (tok, tgt, pos)
    # determinism by seed, rank-dependent streams
    a = fb.PackedBatches(V, T, B, seed=5).next()[0]
    b = fb.PackedBatches(V, T, B, seed=5).next()[0]
    c = fb.PackedBatches(V, T, B, seed=5, rank=1).next()[0]
    assert (a == b).all() and (a != c).any()


def _header_prototypes():
    """name -> (return kind, [argument kinds]) of every function declared in include/femto.h; a kind is
    'ptr', 'i32', 'i64', 'f32' or 'f64'."""
    hdr = open(os.path.join(ROOT, "include", "femto.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)

    def kind(decl):
        decl = decl.strip()
        if "*" in decl:
            return "ptr"
        for pat, k in (("int32_t", "i32"), ("int64_t", "i64"), ("float", "f32"), ("double", "f64")):
            if re.search(rf"\b{pat}\b", decl):
                return k
        raise AssertionError(f"unknown C type in {decl!r}")

    out = {}
    for m in re.finditer(r"([A-Za-z_][A-Za-z0-9_ ]*?[\s\*]+)(femto_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", hdr):
        ret, name, args = m.group(1), m.group(2), m.group(3).strip()
        out[name] = (kind(ret), [] if args in ("", "void") else [kind(a) for a in args.split(",")])
    return out


def test_ctypes_table_matches_the_header():
    """Every signature in femtochat_b200/_lib.py has the header's argument count and kinds."""
    protos = _header_prototypes()
    kinds = {ctypes.c_int32: "i32", ctypes.c_int64: "i64", ctypes.c_float: "f32", ctypes.c_double: "f64"}

    def kind(t):
        return kinds.get(t, "ptr")

    for name, (res, args) in _lib.SIGNATURES.items():
        assert name in protos, name
        assert [kind(a) for a in args] == protos[name][1], name
        assert kind(res) == protos[name][0], name


def test_julia_shim_ccalls_match_the_header():
    """julia/FemtoChatCUDAExt.jl cannot be executed here (no Julia toolchain), so each of its ccall signatures is
    parsed and compared with include/femto.h: same entry point name, same number of arguments, and each Julia
    argument type the right width (Int32 / Int64 / Float32 / pointer-like)."""
    src = open(os.path.join(ROOT, "julia", "FemtoChatCUDAExt.jl")).read()
    protos = _header_prototypes()

    def jl_kind(t):
        t = t.strip()
        if t.startswith(("Ptr{", "CuPtr{", "Ref{")) or t == "Cstring":
            return "ptr"
        return {"Int32": "i32", "Int64": "i64", "Float32": "f32", "Float64": "f64"}[t]

    def split_top(s):
        parts, depth, cur = [], 0, ""
        for ch in s:
            if ch in "({[":
                depth += 1
            elif ch in ")}]":
                depth -= 1
            if ch == "," and depth == 0:
                parts.append(cur)
                cur = ""
            else:
                cur += ch
        if cur.strip():
            parts.append(cur)
        return [p.strip() for p in parts]

    seen = set()
    for m in re.finditer(r"ccall\(\(:(femto_[a-z0-9_]+), libfemto\),\s*([A-Za-z0-9]+),\s*\(", src):
        name, ret = m.group(1), m.group(2)
        i, depth = m.end(), 1                        # scan the argument-type tuple to its closing parenthesis
        while depth:
            depth += {"(": 1, ")": -1}.get(src[i], 0)
            i += 1
        types = [t for t in split_top(src[m.end():i - 1]) if t]
        assert name in protos, f"{name} is not declared in include/femto.h"
        want_ret, want_args = protos[name]
        assert jl_kind(ret) == want_ret, name
        assert [jl_kind(t) for t in types] == want_args, (name, types, want_args)
        # the call passes as many values as the tuple has types
        j, depth = i, 0
        while True:
            depth += {"(": 1, ")": -1}.get(src[j], 0)
            if depth < 0:
                break
            j += 1
        values = [v for v in split_top(src[i:j]) if v]
        assert len(values) == len(types), (name, len(values), len(types))
        seen.add(name)
    # every seam that INTEGRATION.md maps is bound
    for name in ("femto_create", "femto_destroy", "femto_refresh_weights", "femto_loss_and_gradient", "femto_forward_loss",
                 "femto_forward_logits", "femto_forward_token_losses", "femto_optimizer_state_sizes",
                 "femto_optimizer_create", "femto_optimizer_step", "femto_optimizer_set_t", "femto_optimizer_destroy",
                 "femto_attention_fwd", "femto_attention_bwd", "femto_embedding_gradient", "femto_embed_gather",
                 "femto_rmsnorm_fwd", "femto_rmsnorm_bwd", "femto_gemm_bf16", "femto_newton_schulz",
                 "femto_muon_direction", "femto_adamw", "femto_cross_entropy", "femto_cross_entropy_gradient",
                 "femto_status_word", "femto_last_error"):
        assert name in seen, f"{name} is not bound in the Julia shim"
    # the methods the reference's extension defines are defined here too
    for method in ("function gradient_state(", "function loss_and_gradient!(", "function MuonAdamW(", "function attention!(",
                   "function Δattention!(", "function embedding_gradient!(", "function batched_mul!(", "function gather!(",
                   "function scatter!("):
        assert method in src, method
    assert "accumulate::Bool=true" in src          # the reference's default for Δattention!
    assert "reduction=:mean" in src                # the reference drivers differentiate the mean loss


@pytest.mark.parametrize("world", [2, 3, 8, 32])
def test_shard_plan_tiles_the_parameter_vector(world):
    """Owner-sharded update: the single-owner ranges are disjoint, lie inside [0, nparams), give every Muon matrix
    (the tiny value-embedding gates excepted) exactly one owner and every divisible large table `world` equal slices; the rest is replicated.  Also with more
    ranks than layers (some ranks then own no block)."""
    kw = dict(sequence_len=64, max_document_tokens=64, vocab_size=32768, n_layer=5, n_head=2, n_kv_head=1, n_embed=128,
              window_pattern="SL")
    lay = fb.parameter_layout(fb.GPTConfig(**kw))
    plan = fb.shard_plan(lay, world)
    at = 0
    owned = 0
    for off, n, owner in plan:
        assert off >= at and n > 0 and 0 <= owner < world       # sorted and disjoint
        at = off + n
        owned += n
    assert at <= lay.nparams
    mats = sum(b[k].size for b in lay.blocks for k in ("wq", "wk", "wv", "wo", "fc", "proj") if b[k] is not None)
    assert all(b["ve_gate"] is None or b["ve_gate"].size < 1024 for b in lay.blocks)   # the gates stay with every rank
    tables = [lay.lm_head, lay.embedding] + [b["ve_table"] for b in lay.blocks if b["ve_table"] is not None]
    big = sum(t.size for t in tables if t.size >= fb.optim.SHARD_MIN_TABLE and t.size % (4 * world) == 0)
    assert owned == mats + big
    # every Muon matrix lies inside exactly one range of one owner
    for b in lay.blocks:
        for k in ("wq", "wk", "wv", "wo", "fc", "proj"):
            sp = b[k]
            if sp is None:
                continue
            inside = [(o, n, r) for o, n, r in plan if o <= sp.offset and sp.offset + sp.size <= o + n]
            assert len(inside) == 1, k
    # table slices: rank r owns slice r
    for t in tables:
        if t.size >= fb.optim.SHARD_MIN_TABLE and t.size % (4 * world) == 0:
            for r in range(world):
                assert (t.offset + r * (t.size // world), t.size // world, r) in plan
