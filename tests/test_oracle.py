"""CPU checks of the oracle itself: internal cross-checks and the committed golden vectors.
(The reference ships no golden vectors for this path; see the header of oracle/femto_oracle.py.)"""
import math
import os

import pytest
import torch

from oracle import femto_oracle as fo

GOLD = os.path.join(os.path.dirname(__file__), "golden")
TINY = dict(sequence_len=4, max_document_tokens=64, vocab_size=16, n_layer=2, n_head=2, n_kv_head=1, n_embed=32,
            window_pattern="L")
D20 = dict(sequence_len=2048, vocab_size=65536, n_layer=20, n_head=10, n_kv_head=5, n_embed=1280, window_pattern="SSSL")


def test_structural_known_answers():
    # derived from src/parameters.jl:219-337 by hand
    assert fo.parameter_layout(fo.GPTConfig(**TINY)).nparams == 27690
    lay = fo.parameter_layout(fo.GPTConfig(**D20))
    assert lay.nparams == 947651226
    assert fo.num_matmul_params(lay) == 444334704
    assert fo.estimate_flops(fo.GPTConfig(**D20)) == 2941259424
    assert fo.estimate_flops(fo.GPTConfig(**D20), 1024) == 3059224224
    w = fo.window_sizes(fo.GPTConfig(**D20))
    assert w[:4] == [(512, 0), (512, 0), (512, 0), (2048, 0)] and w[-1] == (2048, 0)
    assert sum(1 for x in w if x[0] == 512) == 15
    tiny = fo.parameter_layout(fo.GPTConfig(**TINY))
    assert tiny.blocks[0]["ve_table"] is None and tiny.blocks[1]["ve_table"] is not None
    assert fo.window_sizes(fo.GPTConfig(**TINY)) == [(4, 0), (4, 0)]


def _inputs(cfg, B, seed=0):
    g = torch.Generator().manual_seed(seed)
    T = cfg.sequence_len
    tok = torch.randint(1, cfg.vocab_size + 1, (B, T), generator=g, dtype=torch.int32)
    tgt = torch.randint(1, cfg.vocab_size + 1, (B, T), generator=g, dtype=torch.int32)
    tgt[0, T // 2] = -1
    pos = ((torch.arange(T)[None, :].repeat(B, 1) + 3 * torch.arange(B)[:, None]) % max(5, T // 2 + 1)).int()
    return tok, tgt, pos


@pytest.mark.parametrize("doc_mask,reduction", [(False, "sum"), (True, "mean")])
def test_hand_reverse_matches_autograd(doc_mask, reduction):
    cfg = fo.GPTConfig(sequence_len=48, max_document_tokens=64, vocab_size=50, n_layer=3, n_head=4, n_kv_head=2,
                       n_embed=32, window_pattern="SL")
    lay = fo.parameter_layout(cfg)
    th = torch.zeros(lay.nparams, dtype=torch.float64)
    fo.initialize(th, cfg, lay, 1, all_nonzero=True)
    tok, tgt, pos = _inputs(cfg, 2)
    M = fo.Model(cfg, fo.StepOptions(eps=fo.EPS_BF16, short_window=16, doc_mask=doc_mask, reduction=reduction))
    assert M.windows[0] == (16, 0) and M.windows[-1] == (48, 0)
    l1, g1, _ = M.loss_and_gradient(th, tok, tgt, pos)
    l2, g2 = M.loss_and_gradient_autograd(th, tok, tgt, pos)   # naive attention, autograd
    assert abs(l1 - l2) < 1e-10 * abs(l2)
    assert float((g1 - g2).abs().max()) < 1e-6 * float(g2.abs().max())


def test_fp32_matches_fp64():
    cfg = fo.GPTConfig(**TINY)
    lay = fo.parameter_layout(cfg)
    th = torch.zeros(lay.nparams, dtype=torch.float32)
    fo.initialize(th, cfg, lay, 123, all_nonzero=True)
    tok, tgt, pos = _inputs(cfg, 2)
    M = fo.Model(cfg)
    l32, g32, _ = M.loss_and_gradient(th, tok, tgt, pos)
    l64, g64, _ = M.loss_and_gradient(th.double(), tok, tgt, pos)
    assert abs(l32 - l64) < 1e-5 * abs(l64)
    cos = torch.dot(g32.double(), g64.double()) / (g32.double().norm() * g64.double().norm())
    assert cos > 0.999999


def test_finite_difference_spot_check():
    cfg = fo.GPTConfig(**TINY)
    lay = fo.parameter_layout(cfg)
    th = torch.zeros(lay.nparams, dtype=torch.float64)
    fo.initialize(th, cfg, lay, 5, all_nonzero=True)
    tok, tgt, pos = _inputs(cfg, 2)
    M = fo.Model(cfg)
    _, g, _ = M.loss_and_gradient(th, tok, tgt, pos)
    for idx in (lay.lam_y.offset, lay.blocks[0]["lam_b"].offset, lay.blocks[1]["ve_gate"].offset + 3,
                lay.smear_gate.offset + 2, lay.blocks[0]["wq"].offset + 17, lay.lm_head.offset + 5):
        e = 1e-6
        tp, tm = th.clone(), th.clone()
        tp[idx] += e
        tm[idx] -= e
        fd = (float(M.forward(tp, tok, tgt, pos)) - float(M.forward(tm, tok, tgt, pos))) / (2 * e)
        assert abs(fd - float(g[idx])) < 1e-4 * max(1.0, abs(fd)), (idx, fd, float(g[idx]))


def test_zero_gradient_invariants():
    cfg = fo.GPTConfig(**TINY)
    lay = fo.parameter_layout(cfg)
    th = torch.zeros(lay.nparams, dtype=torch.float64)
    fo.initialize(th, cfg, lay, 123)            # reference init: both projections zero, lam_s zero
    tok, tgt, pos = _inputs(cfg, 2)
    _, g, _ = fo.Model(cfg).loss_and_gradient(th, tok, tgt, pos)
    for blk in lay.blocks:
        for k in ("wq", "wk", "wv", "fc"):
            s = blk[k]
            assert float(g[s.offset:s.offset + s.size].abs().max()) == 0.0
    # padded vocabulary rows of lm_head and never-seen token rows of wte get exactly zero
    glm = fo.rm(g, lay.lm_head)
    assert float(glm[:, cfg.vocab_size:].abs().max()) == 0.0
    gw = fo.rm(g, lay.embedding)
    seen = set((tok - 1).flatten().tolist())
    unseen = [r for r in range(lay.padded_vocab_size) if r not in seen]
    assert float(gw[unseen].abs().max()) == 0.0


def test_naive_vs_blockwise_attention():
    g = torch.Generator().manual_seed(3)
    Q = torch.randn(2, 40, 4, 16, generator=g, dtype=torch.float64)
    K = torch.randn(2, 40, 2, 16, generator=g, dtype=torch.float64)
    V = torch.randn(2, 40, 2, 16, generator=g, dtype=torch.float64)
    for window in ((40, 0), (7, 0), (-1, 0)):
        a = fo.naive_attention(Q, K, V, window)
        b, l, m = fo.flash_attention_forward(Q, K, V, window, block=16)
        assert float((a - b).abs().max()) < 1e-12


def test_polar_express_orthogonalises():
    g = torch.Generator().manual_seed(4)
    G = torch.randn(2, 24, 48, generator=g, dtype=torch.float64)
    X = fo.polar_express(G)
    s = torch.linalg.svdvals(X)
    assert float(s.min()) > 0.5 and float(s.max()) < 1.3
    Xt = fo.polar_express(G.transpose(1, 2).contiguous())
    assert float((Xt.transpose(1, 2) - X).abs().max()) < 1e-9


def test_schedule_known_points():
    eta, mu, lam = fo.training_schedule(0, 1000)
    assert eta == pytest.approx(1 / 40) and mu == pytest.approx(0.85) and lam == pytest.approx(1.0)
    eta, mu, lam = fo.training_schedule(999, 1000)
    assert eta == pytest.approx(1 / 650 + (1 - 1 / 650) * 0.05)


def test_golden_readme_tiny():
    gold = torch.load(os.path.join(GOLD, "readme_tiny.pt"))
    cfg = fo.GPTConfig(**TINY)
    M = fo.Model(cfg, fo.StepOptions(eps=fo.EPS_F32, reduction="sum"))
    for name in ("ref_init", "all_nonzero"):
        c = gold[name]
        loss, delta, _ = M.loss_and_gradient(c["theta0"].double(), gold["tokens"], gold["targets"], gold["positions"])
        assert loss / 8 == pytest.approx(float(c["losses"][0]), rel=1e-12)
        assert float((delta - c["delta_step1"]).abs().max()) < 1e-6 * float(c["delta_step1"].abs().max())
        assert float(c["losses"][-1]) < float(c["losses"][0])     # SGD on the sum loss goes down


def test_golden_optimizer_small():
    gold = torch.load(os.path.join(GOLD, "optimizer_small.pt"))
    cfg = fo.GPTConfig(sequence_len=32, max_document_tokens=64, vocab_size=96, n_layer=2, n_head=4, n_kv_head=2,
                       n_embed=64, window_pattern="SL")
    lay = fo.parameter_layout(cfg)
    th = gold["theta0"].clone()
    opt = fo.MuonAdamW(lay, weight_decay=0.1)
    assert [len(g.specs) for g in opt.muon] == [4, 4, 2, 2, 1]      # (64,64) (32,64) (256,64) (64,256) (2,12)
    assert len(opt.adamw) == 2 + 1 + 2 * 2 + 3
    for i, d in enumerate(gold["deltas"]):
        opt.step(th, d, eta=0.5 + 0.25 * i, mu=0.9, lam=0.05, Nt=64.0)
        assert float((th - gold["thetas"][i]).abs().max()) < 1e-5
