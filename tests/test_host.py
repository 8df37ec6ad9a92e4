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
