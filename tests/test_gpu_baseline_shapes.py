"""GPU parity against the CPU oracle at the benchmark models' own widths: d20 (1280 wide, 10 query / 5 kv heads),
d26 (1664 wide, 13/13) and d12 (768 wide, 6/6), sequence length 2048, "SSSL" with a 1024-token short window,
per-document masking, a 65 536-entry vocabulary, packed BOS / geometric(512) batches -- with fewer layers and
one or two batch columns so that the oracle finishes in seconds.  Every tensor of the layout is compared on
its own (a whole-delta cosine cannot see a wrong scalar gradient)."""
import math

import pytest
import torch

import femtochat_b200 as fb
from oracle import femto_oracle as fo

pytestmark = pytest.mark.gpu

MATS = ("wq", "wk", "wv", "wo", "fc", "proj")
SCALARS = ("lam_b", "lam_x0")


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-300))


def per_tensor_report(lay, g0, g1):
    """(name, layer, cosine, |g1|/|g0|, relative error) for every tensor of the layout."""
    rows = []

    def add(name, layer, sp):
        if sp is None:
            return
        a, b = g0[sp.offset:sp.offset + sp.size].double(), g1[sp.offset:sp.offset + sp.size].double()
        na, nb = float(a.norm()), float(b.norm())
        rows.append((name, layer, cosine(a, b), nb / (na + 1e-300), float((a - b).norm()) / (na + 1e-300), na))

    add("wte", -1, lay.embedding)
    for i, blk in enumerate(lay.blocks):
        for k in MATS + ("ve_gate", "ve_table") + SCALARS:
            add(k, i, blk[k])
    add("lm_head", -1, lay.lm_head)
    add("smear_gate", -1, lay.smear_gate)
    add("lam_s", -1, lay.lam_s)
    add("lam_y", -1, lay.lam_y)
    return rows


def check_every_tensor(lay, g0, g1, g0r=None, cos_min=0.995, norm_tol=0.03, scalar_tol=0.05):
    """Matrices, tables and gate vectors: cosine >= cos_min and norm ratio within norm_tol.  One-element
    tensors (the lambda scalars): each is a sum over every activation element in which positive and negative
    terms largely cancel, so its bf16 error is judged against its own sensitivity: the change of the ORACLE's
    value when the weights are rounded to bf16 (`g0r`, what the bf16 build multiplies with).  A scalar passes
    when it is within scalar_tol of the oracle, or within four times that sensitivity of it."""
    bad = []
    for name, layer, c, ratio, rel, n0 in per_tensor_report(lay, g0, g1):
        assert n0 > 0, (name, layer, "oracle gradient is zero: the case does not exercise this tensor")
        if name in SCALARS or name in ("lam_s", "lam_y"):
            sp = {"lam_s": lay.lam_s, "lam_y": lay.lam_y}.get(name) or lay.blocks[layer][name]
            a, b = float(g0[sp.offset]), float(g1[sp.offset])
            noise = abs(float(g0r[sp.offset]) - a) if g0r is not None else 0.0
            if abs(b - a) > max(scalar_tol * abs(a), 4.0 * noise):
                bad.append((name, layer, "oracle", a, "library", b, "oracle with bf16 weights", a + noise))
        elif c < cos_min or abs(ratio - 1.0) > norm_tol:
            bad.append((name, layer, "cos", c, "norm ratio", ratio))
    assert not bad, bad


def round_weights_to_bf16(lay, th):
    """Theta with every matrix and table rounded to bf16 (the values the bf16 build computes with); scalars and the
    small gate vectors stay fp32 there and here."""
    out = th.clone()
    specs = [lay.embedding, lay.lm_head]
    for blk in lay.blocks:
        specs += [blk[k] for k in MATS + ("ve_table",) if blk[k] is not None]
    for sp in specs:
        out[sp.offset:sp.offset + sp.size] = out[sp.offset:sp.offset + sp.size].bfloat16().float()
    return out


def packed_inputs(cfgkw, B, seed_rank=0):
    pk = fb.PackedBatches(cfgkw["vocab_size"], cfgkw["sequence_len"], B, max_document_tokens=cfgkw["max_document_tokens"],
                          rank=seed_rank)
    pk.next()                       # skip the first batch: later ones start mid-document (positions > 0 at t = 0)
    return tuple(torch.from_numpy(x) for x in pk.next())


def run_case(cfgkw, B, short_window, doc_mask, seed=123, sensitivity=True):
    cfg, ocfg = fb.GPTConfig(**cfgkw), fo.GPTConfig(**cfgkw)
    lay, olay = fb.parameter_layout(cfg), fo.parameter_layout(ocfg)
    tok, tgt, pos = packed_inputs(cfgkw, B)
    tgt = tgt.clone()
    tgt[0, 5] = -1                  # an ignored slot
    th = torch.zeros(lay.nparams, dtype=torch.float32)
    fo.initialize(th, ocfg, olay, seed, all_nonzero=True)
    M = fo.Model(ocfg, fo.StepOptions(eps=fo.EPS_BF16, short_window=short_window, doc_mask=doc_mask))
    l0, g0, _ = M.loss_and_gradient(th, tok, tgt, pos)
    g0r = None
    if sensitivity:
        _, g0r, _ = M.loss_and_gradient(round_weights_to_bf16(lay, th), tok, tgt, pos)
    params = fb.Params(th.cuda())
    st = fb.gradient_state(params, cfg, lay, tok, tgt, pos, compute_type="bfloat16", short_window=short_window,
                           doc_mask=doc_mask)
    l1 = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos)
    g1 = params.delta.cpu().clone()
    assert st.status_word() == 0
    st.close()
    return lay, float(l0), l1, g0, g1, g0r


BASE = dict(sequence_len=2048, max_document_tokens=8192, vocab_size=65536, window_pattern="SSSL")


@pytest.mark.parametrize("name,kw,B", [
    ("d20", dict(n_layer=4, n_head=10, n_kv_head=5, n_embed=1280), 2),     # GQA 10/5, backout after block 3
    # three layers, not two: with two the backed-out block is the last one, the head's input is then a multiple of
    # that block's output and d loss / d lam_y vanishes (the gradient of norm is orthogonal to its input)
    ("d26", dict(n_layer=3, n_head=13, n_kv_head=13, n_embed=1664), 1),    # 1664 = 6.5 GEMM tiles of 256
    ("d12", dict(n_layer=3, n_head=6, n_kv_head=6, n_embed=768), 1)])
def test_step_at_benchmark_widths(name, kw, B):
    """Loss within 1e-2 relative, whole-delta cosine >= 0.999, and every tensor on its own."""
    lay, l0, l1, g0, g1, g0r = run_case({**BASE, **kw}, B, short_window=1024, doc_mask=True)
    assert abs(l1 - l0) <= 1e-2 * abs(l0), (l0, l1)
    assert cosine(g0, g1) >= 0.999
    check_every_tensor(lay, g0, g1, g0r)


def test_step_d20_reference_window_rule_no_doc_mask():
    """The reference's own options at the d20 width: short window 512 (src/parameters.jl:204), attention
    crossing document boundaries (src/dataloader.jl:165-166)."""
    lay, l0, l1, g0, g1, g0r = run_case({**BASE, **dict(n_layer=4, n_head=10, n_kv_head=5, n_embed=1280)}, 1,
                                        short_window=0, doc_mask=False, seed=7)
    assert abs(l1 - l0) <= 1e-2 * abs(l0), (l0, l1)
    assert cosine(g0, g1) >= 0.999
    check_every_tensor(lay, g0, g1, g0r)


TC = dict(sequence_len=256, max_document_tokens=512, vocab_size=1000, n_layer=4, n_head=4, n_kv_head=2, n_embed=512,
          window_pattern="SL")


@pytest.mark.parametrize("doc_mask", [False, True])
def test_small_tensor_core_step_every_tensor(doc_mask, monkeypatch):
    """The smallest shape that runs every tensor-core kernel, all fifteen tensor kinds checked one by one.  The lm_head
    tail is cut into chunks of 768 tokens here (1024 tokens: one full chunk and a short one, the second on the other
    d-logit buffer and adding to the first one's weight gradient), as the full-size step cuts its 65 536."""
    monkeypatch.setenv("FEMTO_XENT_CHUNK", "768")
    cfg, ocfg = fb.GPTConfig(**TC), fo.GPTConfig(**TC)
    lay, olay = fb.parameter_layout(cfg), fo.parameter_layout(ocfg)
    g = torch.Generator().manual_seed(4)
    B, T = 4, TC["sequence_len"]
    tok = torch.randint(1, TC["vocab_size"] + 1, (B, T), generator=g, dtype=torch.int32)
    tgt = torch.randint(1, TC["vocab_size"] + 1, (B, T), generator=g, dtype=torch.int32)
    tgt[1, 7] = -1
    pos = ((torch.arange(T)[None, :].repeat(B, 1) + 5 * torch.arange(B)[:, None]) % 97).int()
    th = torch.zeros(lay.nparams)
    fo.initialize(th, ocfg, olay, 11, all_nonzero=True)
    M = fo.Model(ocfg, fo.StepOptions(eps=fo.EPS_BF16, short_window=128, doc_mask=doc_mask))
    l0, g0, _ = M.loss_and_gradient(th, tok, tgt, pos)
    _, g0r, _ = M.loss_and_gradient(round_weights_to_bf16(lay, th), tok, tgt, pos)
    params = fb.Params(th.cuda())
    st = fb.gradient_state(params, cfg, lay, tok, tgt, pos, compute_type="bfloat16", short_window=128, doc_mask=doc_mask)
    l1 = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos)
    assert abs(l1 - float(l0)) <= 1e-2 * abs(float(l0))
    check_every_tensor(lay, g0, params.delta.cpu(), g0r)
    # the same streaming kernels in the fp32 build (they are templates over the activation type): every scalar tight
    st32 = fb.gradient_state(params, cfg, lay, tok, tgt, pos, compute_type="float32", short_window=128, doc_mask=doc_mask)
    M32 = fo.Model(ocfg, fo.StepOptions(eps=fo.EPS_F32, short_window=128, doc_mask=doc_mask))
    _, g32, _ = M32.loss_and_gradient(th.double(), tok, tgt, pos)
    fb.loss_and_gradient_(params, st32, lay, tok, tgt, pos)
    check_every_tensor(lay, g32.float(), params.delta.cpu(), None, cos_min=0.99999, norm_tol=1e-4, scalar_tol=1e-3)


def test_external_theta_write_needs_refresh_and_changes_the_loss():
    """The library keeps a compute-type copy of the weights: after Theta is written from outside, the next loss
    must change once refresh_weights has run (a host that forgets it would train on stale weights)."""
    cfg = fb.GPTConfig(**TC)
    lay = fb.parameter_layout(cfg)
    th = torch.zeros(lay.nparams)
    fo.initialize(th, fo.GPTConfig(**TC), fo.parameter_layout(fo.GPTConfig(**TC)), 3, all_nonzero=True)
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(1, 1001, (2, 256), generator=g, dtype=torch.int32)
    tgt = torch.randint(1, 1001, (2, 256), generator=g, dtype=torch.int32)
    params = fb.Params(th.cuda())
    st = fb.gradient_state(params, cfg, lay, tok, tgt, compute_type="bfloat16")
    l0 = fb.loss_and_gradient_(params, st, lay, tok, tgt)
    params.theta -= 0.5 * params.delta / 512
    st.refresh_weights(params.theta)
    l1 = fb.loss_and_gradient_(params, st, lay, tok, tgt)
    assert l1 < l0 and math.isfinite(l1)
