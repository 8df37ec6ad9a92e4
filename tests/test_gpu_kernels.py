"""GPU parity of the kernel-level C-ABI entry points against the CPU oracle (oracle/femto_oracle.py)."""
import ctypes as C
import math
import os

import pytest
import torch

import femtochat_b200 as fb
from femtochat_b200 import _lib
from oracle import femto_oracle as fo

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def cosine(a, b):
    a, b = a.double().flatten().cpu(), b.double().flatten().cpu()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-300))


# ---- GEMM -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("ak", [True, False])
@pytest.mark.parametrize("bk", [True, False])
@pytest.mark.parametrize("shape", [(256, 512, 320, 1), (264, 264, 136, 1), (384, 640, 1280, 3)])
def test_gemm_bf16_all_operand_layouts(ak, bk, shape):
    """Every combination of K-contiguous / MN-contiguous operands, ragged tails, batches."""
    M, N, K, batch = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    A = torch.randn(batch, M, K, generator=g, device="cuda").bfloat16()
    B = torch.randn(batch, K, N, generator=g, device="cuda").bfloat16()
    As = A.contiguous() if ak else A.transpose(1, 2).contiguous()
    Bs = B.transpose(1, 2).contiguous() if bk else B.contiguous()
    Cc = torch.empty(batch, M, N, device="cuda", dtype=torch.bfloat16)
    _lib.check(_lib.lib().femto_gemm_bf16(_lib.ptr(As), int(ak), K if ak else M, _lib.ptr(Bs), int(bk), K if bk else N,
                                          _lib.ptr(Cc), N, M, N, K, batch, M * K, K * N, M * N, 0, 0, None))
    torch.cuda.synchronize()
    ref = torch.bmm(A.double().cpu(), B.double().cpu())      # exact products of the bf16 inputs
    err = (Cc.double().cpu() - ref).abs().max()
    assert err <= 2.0 ** -8 * ref.abs().max()               # one bf16 rounding of the result


def test_gemm_split_k_fp32_accumulate_is_deterministic():
    """Weight-gradient form: both operands MN-contiguous, K = tokens, fp32 C += ; split-K reduce in fixed order."""
    M, N, K = 1280, 1280, 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    A = torch.randn(K, M, generator=g, device="cuda").bfloat16()
    B = torch.randn(K, N, generator=g, device="cuda").bfloat16()
    outs = []
    for _ in range(2):
        Cc = torch.ones(M, N, device="cuda")
        _lib.check(_lib.lib().femto_gemm_bf16(_lib.ptr(A), 0, M, _lib.ptr(B), 0, N, _lib.ptr(Cc), N, M, N, K, 1, 0, 0, 0,
                                              1, 1, None))
        torch.cuda.synchronize()
        outs.append(Cc.cpu())
    ref = 1.0 + A.double().cpu().T @ B.double().cpu()
    assert (outs[0].double() - ref).abs().max() <= 1e-5 * ref.abs().max()
    assert torch.equal(outs[0], outs[1])


# ---- attention ----------------------------------------------------------------------------------------
def _attn_inputs(dtype, B, T, H, Hkv, hd, seed, docs):
    g = torch.Generator().manual_seed(seed)
    td = torch.bfloat16 if dtype == _lib.BF16 else torch.float32
    mk = lambda *s: torch.randn(*s, generator=g).to(td)
    Q, K, V, dO = mk(B, T, H, hd), mk(B, T, Hkv, hd), mk(B, T, Hkv, hd), mk(B, T, H, hd)
    ds = None
    if docs:
        pos = (torch.arange(T)[None, :].repeat(B, 1) + 7 * torch.arange(B)[:, None]) % 61
        ds = fo.document_starts(pos).int().contiguous()
    return Q, K, V, dO, ds


@pytest.mark.parametrize("dtype,B,T,H,Hkv,hd,left,docs", [
    (_lib.F32, 2, 40, 4, 2, 16, 40, False), (_lib.F32, 2, 40, 4, 1, 16, 7, True), (_lib.F32, 1, 33, 2, 2, 64, 33, False),
    (_lib.BF16, 2, 256, 4, 2, 128, 256, False), (_lib.BF16, 2, 512, 4, 2, 128, 100, True),
    (_lib.BF16, 1, 1024, 10, 5, 128, 300, True), (_lib.BF16, 2, 96, 2, 1, 64, 30, False),
    # one query head per kv head (the single-head forward kernel) and four per kv head (two CTAs per group)
    (_lib.BF16, 2, 384, 3, 3, 128, 200, True), (_lib.BF16, 1, 512, 8, 2, 128, 512, False),
    # three query heads per kv head: the forward pairs adjacent query tiles of one head instead of two heads
    (_lib.BF16, 1, 512, 6, 2, 128, 150, True)])
def test_attention_forward_and_reverse(dtype, B, T, H, Hkv, hd, left, docs):
    """attention! / Δattention! against naive_attention (src/kernels.jl:59-96) and the blockwise reverse."""
    Q, K, V, dO, ds = _attn_inputs(dtype, B, T, H, Hkv, hd, seed=T + hd, docs=docs)
    Qd, Kd, Vd, dOd = (x.double() for x in (Q, K, V, dO))
    O_ref = fo.naive_attention(Qd, Kd, Vd, (left, 0), ds.long() if ds is not None else None)
    _, l_ref, m_ref = fo.flash_attention_forward(Qd, Kd, Vd, (left, 0), ds.long() if ds is not None else None)
    dq_ref, dk_ref, dv_ref = fo.flash_attention_backward(dOd, Qd, Kd, Vd, O_ref, l_ref, m_ref, (left, 0),
                                                         ds.long() if ds is not None else None)
    dev = [x.cuda() for x in (Q, K, V, dO)]
    dsd = ds.cuda() if ds is not None else None
    O = torch.zeros_like(dev[0])
    lse, l, m = (torch.zeros(B, H, T, device="cuda") for _ in range(3))
    L = _lib.lib()
    _lib.check(L.femto_attention_fwd(dtype, _lib.ptr(O), _lib.ptr(l), _lib.ptr(m), _lib.ptr(lse), _lib.ptr(dev[0]),
                                     _lib.ptr(dev[1]), _lib.ptr(dev[2]), B, T, H, Hkv, hd, left, _lib.ptr(dsd), None))
    dQ, dK, dV = torch.zeros_like(dev[0]), torch.zeros_like(dev[1]), torch.zeros_like(dev[2])
    _lib.check(L.femto_attention_bwd(dtype, _lib.ptr(dQ), _lib.ptr(dK), _lib.ptr(dV), _lib.ptr(dev[3]), _lib.ptr(dev[0]),
                                     _lib.ptr(dev[1]), _lib.ptr(dev[2]), _lib.ptr(O), _lib.ptr(lse), None, None, B, T, H, Hkv, hd,
                                     left, _lib.ptr(dsd), 0, None))
    torch.cuda.synchronize()
    tol = 2e-2 if dtype == _lib.BF16 else 2e-5
    assert (O.double().cpu() - O_ref).abs().max() <= tol
    lse_ref = m_ref + torch.log(l_ref)
    assert (lse.double().cpu() - lse_ref).abs().max() <= (1e-3 if dtype == _lib.BF16 else 1e-5)
    assert ((m + torch.log(l)).double().cpu() - lse_ref).abs().max() <= (1e-3 if dtype == _lib.BF16 else 1e-5)
    for got, ref in ((dQ, dq_ref), (dK, dk_ref), (dV, dv_ref)):
        rel = (got.double().cpu() - ref).norm() / ref.norm()
        assert rel <= (1e-2 if dtype == _lib.BF16 else 1e-5), rel


def test_attention_at_benchmark_shape_geometric_documents():
    """The benchmark's attention shape: T=2048, 10 query / 5 kv heads, head_dim 128, short window 1024, documents of
    geometric(512) length (B=1 so that the fp64 naive reference stays small)."""
    import numpy as np
    B, T, H, Hkv, hd, left = 1, 2048, 10, 5, 128, 1024
    Q, K, V, dO, _ = _attn_inputs(_lib.BF16, B, T, H, Hkv, hd, seed=1, docs=False)
    rng = np.random.default_rng(2)
    starts, t = [], 0
    while t < T:
        n = int(min(max(rng.geometric(1.0 / 512), 2), T - t))
        starts += [t] * n
        t += n
    ds = torch.tensor(starts, dtype=torch.int32)[None, :].contiguous()
    Qd, Kd, Vd, dOd = (x.double() for x in (Q, K, V, dO))
    O_ref = fo.naive_attention(Qd, Kd, Vd, (left, 0), ds.long())
    _, l_ref, m_ref = fo.flash_attention_forward(Qd, Kd, Vd, (left, 0), ds.long())
    dq_ref, dk_ref, dv_ref = fo.flash_attention_backward(dOd, Qd, Kd, Vd, O_ref, l_ref, m_ref, (left, 0), ds.long())
    dev = [x.cuda() for x in (Q, K, V, dO)]
    dsd = ds.cuda()
    O = torch.zeros_like(dev[0])
    lse = torch.zeros(B, H, T, device="cuda")
    L = _lib.lib()
    _lib.check(L.femto_attention_fwd(_lib.BF16, _lib.ptr(O), None, None, _lib.ptr(lse), _lib.ptr(dev[0]), _lib.ptr(dev[1]),
                                     _lib.ptr(dev[2]), B, T, H, Hkv, hd, left, _lib.ptr(dsd), None))
    dQ, dK, dV = torch.zeros_like(dev[0]), torch.zeros_like(dev[1]), torch.zeros_like(dev[2])
    _lib.check(L.femto_attention_bwd(_lib.BF16, _lib.ptr(dQ), _lib.ptr(dK), _lib.ptr(dV), _lib.ptr(dev[3]), _lib.ptr(dev[0]),
                                     _lib.ptr(dev[1]), _lib.ptr(dev[2]), _lib.ptr(O), _lib.ptr(lse), None, None, B, T, H, Hkv,
                                     hd, left, _lib.ptr(dsd), 0, None))
    torch.cuda.synchronize()
    assert (O.double().cpu() - O_ref).abs().max() <= 2e-2
    assert (lse.double().cpu() - (m_ref + torch.log(l_ref))).abs().max() <= 1e-3
    for got, ref in ((dQ, dq_ref), (dK, dk_ref), (dV, dv_ref)):
        rel = (got.double().cpu() - ref).norm() / ref.norm()
        assert rel <= 1e-2, rel


@pytest.mark.parametrize("dtype,T,hd", [(_lib.BF16, 256, 128), (_lib.F32, 40, 16)])
def test_attention_reverse_accumulates_and_takes_l_m(dtype, T, hd):
    """The reference's call form (ext/FemtoChatCUDAExt.jl:1771-1776): the saved statistics are the row sum l and
    the row max m, and accumulate=true (its default) adds to dQ / dK / dV."""
    B, H, Hkv, left = 2, 4, 2, T // 2
    Q, K, V, dO, ds = _attn_inputs(dtype, B, T, H, Hkv, hd, seed=5, docs=True)
    dev = [x.cuda() for x in (Q, K, V, dO)]
    dsd = ds.cuda()
    O = torch.zeros_like(dev[0])
    lse, l, m = (torch.zeros(B, H, T, device="cuda") for _ in range(3))
    L = _lib.lib()
    _lib.check(L.femto_attention_fwd(dtype, _lib.ptr(O), _lib.ptr(l), _lib.ptr(m), _lib.ptr(lse), _lib.ptr(dev[0]),
                                     _lib.ptr(dev[1]), _lib.ptr(dev[2]), B, T, H, Hkv, hd, left, _lib.ptr(dsd), None))

    def bwd(dQ, dK, dV, use_lm, acc):
        _lib.check(L.femto_attention_bwd(dtype, _lib.ptr(dQ), _lib.ptr(dK), _lib.ptr(dV), _lib.ptr(dev[3]), _lib.ptr(dev[0]),
                                         _lib.ptr(dev[1]), _lib.ptr(dev[2]), _lib.ptr(O), None if use_lm else _lib.ptr(lse),
                                         _lib.ptr(l) if use_lm else None, _lib.ptr(m) if use_lm else None, B, T, H, Hkv,
                                         hd, left, _lib.ptr(dsd), acc, None))
        torch.cuda.synchronize()

    base = [torch.zeros_like(dev[0]), torch.zeros_like(dev[1]), torch.zeros_like(dev[2])]
    bwd(*base, False, 0)
    via_lm = [torch.full_like(x, 7.0) for x in base]          # accumulate=0 overwrites whatever was there
    bwd(*via_lm, True, 0)
    tol = 2e-2 if dtype == _lib.BF16 else 1e-5
    for a, b in zip(base, via_lm):
        assert (a.float() - b.float()).abs().max() <= tol * max(1.0, float(a.float().abs().max()))
    g = torch.Generator().manual_seed(8)
    init = [torch.randn(x.shape, generator=g).to(x.dtype).cuda() for x in base]
    acc = [x.clone() for x in init]
    bwd(*acc, False, 1)
    for a, i0, b in zip(acc, init, base):
        want = i0.float() + b.float()
        assert (a.float() - want).abs().max() <= (3e-2 if dtype == _lib.BF16 else 1e-5) * max(1.0, float(want.abs().max()))
    # neither form of the statistics given -> argument error, nothing launched
    assert L.femto_attention_bwd(dtype, _lib.ptr(acc[0]), _lib.ptr(acc[1]), _lib.ptr(acc[2]), _lib.ptr(dev[3]),
                                 _lib.ptr(dev[0]), _lib.ptr(dev[1]), _lib.ptr(dev[2]), _lib.ptr(O), None, None, None, B, T, H,
                                 Hkv, hd, left, _lib.ptr(dsd), 0, None) == -1


# ---- embedding gradient ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [_lib.F32, _lib.BF16])
def test_embedding_gradient_segmented_scatter(dtype):
    """embedding_gradient! (src/kernels.jl:8-14) with a Zipf-like token list (one id 3000 times, BOS
    runs, unseen rows): fixed summation order -> repeatable bit for bit; unseen rows untouched."""
    N, D, rows = 8192, 256, 4096
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, rows, (N,), generator=g, dtype=torch.int32)
    tok[:3000] = 17
    tok[3000:3100] = rows - 1
    tok = tok[torch.randperm(N, generator=g)]
    td = torch.bfloat16 if dtype == _lib.BF16 else torch.float32
    dy = torch.randn(N, D, generator=g).to(td)
    ref = torch.full((rows, D), 0.5, dtype=torch.float64)
    ref.index_add_(0, tok.long(), dy.double())
    outs = []
    for _ in range(2):
        table = torch.full((rows, D), 0.5, device="cuda")
        dyd, tokd = dy.cuda(), tok.cuda()          # keep the device copies alive across the call
        _lib.check(_lib.lib().femto_embedding_gradient(dtype, _lib.ptr(table), _lib.ptr(dyd), _lib.ptr(tokd), N, D, rows,
                                                       None))
        outs.append(table.cpu())
    assert (outs[0].double() - ref).abs().max() <= 1e-3
    assert torch.equal(outs[0], outs[1])
    unseen = torch.ones(rows, dtype=torch.bool)
    unseen[tok.long()] = False
    assert torch.equal(outs[0][unseen], torch.full_like(outs[0][unseen], 0.5))


# ---- lm_head tail -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,N,D,V,ldw", [(_lib.F32, 70, 32, 50, 64), (_lib.BF16, 512, 256, 1000, 1024),
                                              (_lib.BF16, 300, 64, 100, 128),
                                              # more tokens than one chunk of 8192: later chunks offset every row
                                              # buffer, add to dW, and the last one is short
                                              (_lib.BF16, 8192 + 300, 128, 1000, 1024), (_lib.F32, 8192 + 300, 32, 50, 64),
                                              (_lib.BF16, 20000, 256, 1000, 1024)])
def test_xent_fused_tail(dtype, N, D, V, ldw):
    g = torch.Generator().manual_seed(9)
    td = torch.bfloat16 if dtype == _lib.BF16 else torch.float32
    x = fo.norm(torch.randn(N, D, generator=g), 1e-6).to(td)
    W = (torch.randn(D, ldw, generator=g) * 0.5).to(td)
    tgt = torch.randint(0, V, (N,), generator=g, dtype=torch.int32)
    tgt[::13] = -1
    xd, Wd = x.double().requires_grad_(True), W.double().requires_grad_(True)
    z = fo.SOFTCAP * torch.tanh(xd @ Wd[:, :V] / fo.SOFTCAP)
    valid = tgt >= 0
    losses = torch.logsumexp(z, -1) - z.gather(1, tgt.clamp(min=0).long()[:, None])[:, 0]
    loss_ref = losses[valid].sum()
    loss_ref.backward()
    dx = torch.zeros(N, D, device="cuda", dtype=td)
    dw = torch.ones(D, ldw, device="cuda")
    loss = torch.zeros(1, device="cuda")
    nv = torch.zeros(1, device="cuda", dtype=torch.int32)
    xg, Wg, tg = x.cuda(), W.cuda(), tgt.cuda()   # keep the device copies alive across the call
    _lib.check(_lib.lib().femto_xent_fused(dtype, _lib.ptr(xg), _lib.ptr(Wg), ldw, _lib.ptr(tg), N, D, V, 1.0, _lib.ptr(dx),
                                           _lib.ptr(dw), _lib.ptr(loss), _lib.ptr(nv), None))
    torch.cuda.synchronize()
    assert int(nv.item()) == int(valid.sum())
    tol = 1e-2 if dtype == _lib.BF16 else 1e-5
    assert abs(float(loss.item()) - float(loss_ref.detach())) <= tol * abs(float(loss_ref.detach()))
    assert cosine(dx, xd.grad) >= (0.999 if dtype == _lib.BF16 else 0.999999)
    assert cosine(dw[:, :V] - 1.0, Wd.grad[:, :V]) >= (0.999 if dtype == _lib.BF16 else 0.999999)
    assert torch.equal(dw[:, V:].cpu(), torch.ones(D, ldw - V))      # padded vocabulary columns untouched


# ---- optimiser ------------------------------------------------------------------------------------------------
def test_adamw_matches_oracle_three_steps():
    n = 10007
    g = torch.Generator().manual_seed(2)
    theta = torch.randn(n, generator=g)
    spec = fo.Spec(0, (n,))
    st = fo.AdamWState(spec, 0.03, 0.8, 0.95, 1e-10, 0.05)
    th_ref = theta.clone()
    th, m, v = theta.cuda(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for t in range(1, 4):
        d = torch.randn(n, generator=g) * 4
        gg = d / 64.0
        st.t += 1
        st.m.mul_(st.b1).add_((1 - st.b1) * gg)
        st.v.mul_(st.b2).add_((1 - st.b2) * gg * gg)
        th_ref = th_ref * (1 - st.alpha * st.lam) - st.alpha * (st.m / (1 - st.b1 ** st.t)) / (
            torch.sqrt(st.v / (1 - st.b2 ** st.t)) + st.eps)
        dd = d.cuda()
        _lib.check(_lib.lib().femto_adamw(_lib.ptr(th), _lib.ptr(dd), _lib.ptr(m), _lib.ptr(v), n, 0.03, 0.8, 0.95, 1e-10,
                                          0.05, t, 64.0, None))
        torch.cuda.synchronize()
    torch.cuda.synchronize()
    assert (th.cpu() - th_ref).abs().max() <= 1e-5


@pytest.mark.parametrize("dtype,k,rows,cols", [(_lib.F32, 3, 24, 48), (_lib.F32, 2, 48, 24), (_lib.F32, 2, 32, 32),
                                                (_lib.BF16, 2, 256, 512), (_lib.BF16, 2, 512, 256)])
def test_newton_schulz_matches_polar_express(dtype, k, rows, cols):
    """polar_express! (src/optim.jl:131-149) with the reference's five coefficient triples."""
    g = torch.Generator().manual_seed(rows + cols)
    G = torch.randn(k, rows, cols, generator=g)
    ref = fo.polar_express(G.double())
    X = G / (1.01 * G.pow(2).sum(dim=(1, 2), keepdim=True).sqrt() + 1e-6)
    td = torch.bfloat16 if dtype == _lib.BF16 else torch.float32
    Xd = X.to(td).cuda().contiguous()
    coeffs = (C.c_float * 15)(*[c for abc in fo.POLAR_EXPRESS_COEFFS for c in abc])
    _lib.check(_lib.lib().femto_newton_schulz(dtype, _lib.ptr(Xd), k, rows, cols, coeffs, 5, None))
    torch.cuda.synchronize()
    if dtype == _lib.F32:
        assert (Xd.double().cpu() - ref).abs().max() <= 1e-4
    else:
        assert cosine(Xd, ref) >= 0.995


def test_muon_adamw_three_steps_against_golden():
    """The whole MuonAdamW step (group order, MuonEq, Polar Express, Muon+, NorMuon, cautious decay)
    in fp32 against the oracle fixture."""
    gold = torch.load(os.path.join(GOLD, "optimizer_small.pt"))
    kw = dict(sequence_len=32, max_document_tokens=64, vocab_size=96, n_layer=2, n_head=4, n_kv_head=2, n_embed=64,
              window_pattern="SL")
    cfg = fb.GPTConfig(**kw)
    lay = fb.parameter_layout(cfg)
    params = fb.Params(gold["theta0"].clone().cuda())
    st = fb.GradientState(cfg, max_batch=2)
    st.refresh_weights(params.theta)
    opt = fb.MuonAdamW(params, lay, st, weight_decay=0.1)
    assert len(opt.adamw) == 10 and [len(g.specs) for g in opt.muon] == [4, 4, 2, 2, 1]
    for i, d in enumerate(gold["deltas"]):
        params.delta.copy_(d.cuda())
        opt.step(eta=0.5 + 0.25 * i, mu=0.9, lam=0.05, Nt=64.0)
        err = (params.theta.cpu() - gold["thetas"][i]).abs().max()
        assert err <= 2e-4, (i, float(err))
    assert opt.get_t() == [3] * 10
    assert float(opt.adamw[0].m.abs().max()) > 0 and float(opt.muon[0].m.abs().max()) > 0


@pytest.mark.parametrize("reduction", ["sum", "mean", "none"])
def test_cross_entropy_on_materialised_logits(reduction):
    """cross_entropy / cross_entropy_gradient! on a (V,T,B) logits array (src/gpt.jl:175-193,
    src/kernels.jl:16-28): fp32, ignored targets contribute nothing, delta is accumulated into."""
    L = _lib.lib()
    N, V, ld = 70, 50, 56
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(N, ld, generator=g) * 3
    tgt = torch.randint(0, V, (N,), generator=g, dtype=torch.int32)
    tgt[::9] = -1
    valid = tgt >= 0
    z = logits[:, :V].double()
    losses = torch.where(valid, torch.logsumexp(z, -1) - z.gather(1, tgt.clamp(min=0).long()[:, None])[:, 0], torch.zeros(N, dtype=torch.float64))
    red = {"sum": 0, "mean": 1, "none": 2}[reduction]
    lg, tg = logits.cuda(), tgt.cuda()
    out = torch.zeros(N if reduction == "none" else 1, device="cuda")
    nv = torch.zeros(1, device="cuda", dtype=torch.int32)
    _lib.check(L.femto_cross_entropy(_lib.ptr(lg), ld, _lib.ptr(tg), N, V, red, _lib.ptr(out), _lib.ptr(nv), None))
    torch.cuda.synchronize()
    assert int(nv) == int(valid.sum())
    ref = {"sum": losses.sum(), "mean": losses.sum() / valid.sum(), "none": losses}[reduction]
    assert torch.allclose(out.double().cpu().reshape(ref.shape), ref, rtol=1e-5, atol=1e-5)
    # gradient, accumulated into a non-zero delta
    dy = 0.7
    dy_rows = torch.rand(N, generator=g) + 0.5
    scale = {"sum": torch.full((N,), dy, dtype=torch.float64), "mean": torch.full((N,), dy / int(valid.sum()), dtype=torch.float64),
             "none": dy_rows.double()}[reduction]
    onehot = torch.zeros(N, V, dtype=torch.float64)
    onehot[valid, tgt[valid].long()] = 1.0
    d_ref = torch.where(valid[:, None], scale[:, None] * (torch.softmax(z, -1) - onehot), torch.zeros(N, V, dtype=torch.float64))
    delta0 = torch.randn(N, ld, generator=g)
    delta = delta0.clone().cuda()
    dyr = dy_rows.cuda()
    _lib.check(L.femto_cross_entropy_gradient(_lib.ptr(delta), ld, _lib.ptr(lg), ld, _lib.ptr(tg), N, V, red, dy,
                                              _lib.ptr(dyr) if reduction == "none" else None, None))
    torch.cuda.synchronize()
    got = delta.double().cpu()
    assert torch.allclose(got[:, :V], delta0[:, :V].double() + d_ref, rtol=1e-5, atol=1e-6)
    assert torch.equal(got[:, V:], delta0[:, V:].double())   # padded columns untouched


# ---- streaming kernels behind their own entry points --------------------------------------------------------------
@pytest.mark.parametrize("dtype,N,D", [(_lib.F32, 37, 40), (_lib.F32, 9, 33), (_lib.BF16, 300, 1280), (_lib.BF16, 65, 128)])
def test_rmsnorm_forward_and_reverse(dtype, N, D):
    """norm (src/gpt.jl:16-20) and its reverse (ext/FemtoChatMooncakeExt.jl:248-255) with eps = eps(eltype)."""
    td = torch.bfloat16 if dtype == _lib.BF16 else torch.float32
    eps = fo.EPS_BF16 if dtype == _lib.BF16 else fo.EPS_F32
    g = torch.Generator().manual_seed(N + D)
    x = (torch.randn(N, D, generator=g) * 2).to(td)
    dy = torch.randn(N, D, generator=g).to(td)
    y_ref = fo.norm(x.double(), eps)
    dx_ref = fo.norm_backward(dy.double(), x.double(), eps)
    xd, dyd = x.cuda(), dy.cuda()
    y, dx = torch.zeros_like(xd), torch.zeros_like(xd)
    r = torch.zeros(N, device="cuda")
    L = _lib.lib()
    _lib.check(L.femto_rmsnorm_fwd(dtype, _lib.ptr(xd), _lib.ptr(y), _lib.ptr(r), N, D, eps, None))
    _lib.check(L.femto_rmsnorm_bwd(dtype, _lib.ptr(dyd), _lib.ptr(y), _lib.ptr(r), _lib.ptr(dx), N, D, None))
    torch.cuda.synchronize()
    tol = 2e-2 if dtype == _lib.BF16 else 1e-5
    assert (y.double().cpu() - y_ref).abs().max() <= tol
    assert (r.double().cpu() - torch.sqrt(x.double().pow(2).mean(-1) + eps)).abs().max() <= 1e-5 * float(r.max())
    assert (dx.double().cpu() - dx_ref).abs().max() <= tol * max(1.0, float(dx_ref.abs().max()))


@pytest.mark.parametrize("dtype,D", [(_lib.F32, 36), (_lib.BF16, 640), (_lib.BF16, 30)])
def test_embed_gather_is_bit_exact(dtype, D):
    """E[:, tokens] (src/gpt.jl:34): a pure row copy, so bit-exact; a bad id is clamped and flagged, not a fault."""
    td = torch.bfloat16 if dtype == _lib.BF16 else torch.float32
    rows, N = 500, 1000
    g = torch.Generator().manual_seed(D)
    table = torch.randn(rows, D, generator=g).to(td)
    tok = torch.randint(0, rows, (N,), generator=g, dtype=torch.int32)
    L = _lib.lib()
    tb, tk = table.cuda(), tok.cuda()
    out = torch.zeros(N, D, device="cuda", dtype=td)
    _lib.check(L.femto_embed_gather(dtype, _lib.ptr(out), _lib.ptr(tb), _lib.ptr(tk), N, D, rows, None))
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), table[tok.long()])
    w = C.c_int32(-1)
    _lib.check(L.femto_status_word(None, C.byref(w)))
    assert w.value == 0
    bad = tok.clone()
    bad[3] = rows + 7
    bd = bad.cuda()
    _lib.check(L.femto_embed_gather(dtype, _lib.ptr(out), _lib.ptr(tb), _lib.ptr(bd), N, D, rows, None))
    _lib.check(L.femto_status_word(None, C.byref(w)))
    assert w.value & 1


@pytest.mark.parametrize("dtype,k,m,n", [(_lib.F32, 3, 48, 24), (_lib.F32, 2, 24, 48), (_lib.F32, 2, 5, 12),
                                          (_lib.BF16, 2, 512, 256), (_lib.BF16, 2, 256, 512), (_lib.BF16, 2, 256, 256)])
def test_muon_direction_matches_oracle_two_steps(dtype, k, m, n):
    """muon_direction! (src/optim.jl:198-236) on a stack of k Julia (m, n) matrices, two consecutive calls so that
    the momentum and the NorMuon second moment carried between steps are compared as well."""
    g = torch.Generator().manual_seed(m * 3 + n)
    specs = [fo.Spec(i * m * n, (m, n)) for i in range(k)]
    st = fo.MuonState(specs, 0.02, 0.95, 0.9, 0.0)
    ora = fo.MuonAdamW.__new__(fo.MuonAdamW)
    ora.coeffs, ora.compute_dtype = fo.POLAR_EXPRESS_COEFFS, (torch.bfloat16 if dtype == _lib.BF16 else None)
    coeffs = (C.c_float * 15)(*[c for abc in fo.POLAR_EXPRESS_COEFFS for c in abc])
    mom = torch.zeros(k, n, m, device="cuda")
    v = torch.zeros(k, max(m, n), device="cuda")
    out = torch.zeros(k, n, m, device="cuda")
    L = _lib.lib()
    for step in range(2):
        G = torch.randn(k, m, n, generator=g) * 3                      # Julia orientation
        X_ref = ora.muon_direction(st, G.clone(), 0.9, 64.0)
        Gs = G.transpose(1, 2).contiguous().cuda()                     # stored orientation [k][n][m]
        _lib.check(L.femto_muon_direction(dtype, _lib.ptr(out), _lib.ptr(Gs), _lib.ptr(mom), _lib.ptr(v), k, n, m, 0.9, 0.9,
                                          64.0, coeffs, 5, None))
        got = out.cpu().transpose(1, 2)
        if dtype == _lib.F32:
            assert (got - X_ref).abs().max() <= 2e-4 * max(1.0, float(X_ref.abs().max())), step
        else:
            assert cosine(got, X_ref) >= 0.995, step
            assert abs(float(got.norm() / X_ref.norm()) - 1.0) <= 2e-2
        assert (mom.cpu().transpose(1, 2) - st.m).abs().max() <= 1e-6 * max(1.0, float(st.m.abs().max()))
        assert (v.cpu().reshape(st.v.shape) - st.v).abs().max() <= (6e-2 if dtype == _lib.BF16 else 1e-5) * float(st.v.abs().max())


def test_muon_adamw_three_steps_bf16_against_oracle():
    """The whole MuonAdamW step with the Polar-Express chain in bf16 (the training configuration) against the oracle
    run with compute_dtype=bfloat16, on 256- and 512-wide matrices that take the tensor-core GEMM.  bf16 Newton-Schulz
    amplifies rounding differences, so the comparison is on the update Theta_t - Theta_0: cosine >= 0.99 per step
    over the Muon matrices, and 1e-5 absolute on everything AdamW owns (fp32 on both sides)."""
    kw = dict(sequence_len=32, max_document_tokens=64, vocab_size=512, n_layer=2, n_head=2, n_kv_head=1, n_embed=256,
              window_pattern="SL")
    cfg, ocfg = fb.GPTConfig(**kw), fo.GPTConfig(**kw)
    lay, olay = fb.parameter_layout(cfg), fo.parameter_layout(ocfg)
    th0 = torch.zeros(lay.nparams)
    fo.initialize(th0, ocfg, olay, 17, all_nonzero=True)
    g = torch.Generator().manual_seed(21)
    deltas = [torch.randn(lay.nparams, generator=g) * 0.5 for _ in range(3)]
    oopt = fo.MuonAdamW(olay, weight_decay=0.1, compute_dtype=torch.bfloat16)
    th_ref = th0.clone()
    params = fb.Params(th0.clone().cuda())
    st = fb.GradientState(cfg, max_batch=1, compute_type="bfloat16")
    st.refresh_weights(params.theta)
    opt = fb.MuonAdamW(params, lay, st, weight_decay=0.1, compute_type="bfloat16")
    muon_mask = torch.zeros(lay.nparams, dtype=torch.bool)
    for grp in opt.muon:
        for sp in grp.specs:
            muon_mask[sp.offset:sp.offset + sp.size] = True
    prev_ref, prev = th0.clone(), th0.clone()
    for i, d in enumerate(deltas):
        kwargs = dict(eta=0.5 + 0.25 * i, mu=0.9, lam=0.05, Nt=64.0)
        oopt.step(th_ref, d, **kwargs)
        params.delta.copy_(d.cuda())
        opt.step(**kwargs)
        got = params.theta.cpu()
        assert (got[~muon_mask] - th_ref[~muon_mask]).abs().max() <= 1e-5
        for grp in opt.muon:
            for sp in grp.specs:
                sl = slice(sp.offset, sp.offset + sp.size)
                c = cosine(got[sl] - prev[sl], th_ref[sl] - prev_ref[sl])
                assert c >= (0.99 if min(sp.shape) >= 128 else 0.95), (i, sp.shape, c)
        prev_ref, prev = th_ref.clone(), got.clone()
        params.theta.copy_(th_ref.cuda())      # keep both sides on the same trajectory
        st.refresh_weights(params.theta)
    assert st.status_word() == 0


# ---- batch producer ---------------------------------------------------------------------------------------------------
def test_device_batch_producer_is_bit_exact_against_the_host_packer():
    """model_batch! (src/dataloader.jl:241-274) on the device: tokens, targets and positions of five consecutive
    batches equal the host packer's arrays bit for bit (documents continuing across batches, a document's last token
    predicting BOS, positions restarting on BOS); padding rows and a bad segment follow the documented rules."""
    V, T, B = 4096, 256, 6
    host = fb.PackedBatches(V, T, B, max_document_tokens=300, mean_doc_len=40, seed=9)
    dev = fb.DevicePackedBatches(V, T, B, batches=5, max_document_tokens=300, mean_doc_len=40, seed=9)
    for _ in range(5):
        want = host.next()
        got = dev.next()
        torch.cuda.synchronize()
        for w, g in zip(want, got):
            assert torch.equal(torch.from_numpy(w), g.cpu())
    assert int(dev.status.item()) == 0
    # padding: a batch with a single short segment
    import numpy as np
    from femtochat_b200.data import SEGMENT_DTYPE
    segs = np.array([(0, 1, 3, 5, 7, -1, 0), (10, 9, 0, 4, 0, 2, 0)], dtype=SEGMENT_DTYPE)   # the second one is outside the batch
    sd = torch.from_numpy(segs.view(np.uint8).reshape(-1)).cuda()
    tok, tgt, pos = (torch.empty(B, T, dtype=torch.int32, device="cuda") for _ in range(3))
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(_lib.lib().femto_pack_batch(_lib.ptr(dev.stream), dev.n_stream, _lib.ptr(sd), 2, B, T, dev.bos - 1, 1,
                                           _lib.ptr(tok), _lib.ptr(tgt), _lib.ptr(pos), _lib.ptr(st), None))
    torch.cuda.synchronize()
    s16 = torch.from_numpy(dev._stream_host.astype(np.int32))
    assert int(st.item()) & 1                                   # the out-of-range segment was flagged and skipped
    assert torch.equal(tok[1, 3:8].cpu(), s16[0:5] + 1) and torch.equal(pos[1, 3:8].cpu(), torch.arange(7, 12, dtype=torch.int32))
    assert torch.equal(tgt[1, 3:7].cpu(), s16[1:5] + 1) and int(tgt[1, 7]) == -1
    mask = torch.ones(B, T, dtype=torch.bool)
    mask[1, 3:8] = False
    assert (tok.cpu()[mask] == dev.bos).all() and (tgt.cpu()[mask] == -1).all() and (pos.cpu()[mask] == 0).all()


def test_feeder_delivers_batches_in_order_and_a_step_runs_from_it():
    """The pinned multi-buffered feeder: batches come out in submission order with the submitted contents, a full
    feeder and an empty one are refused with FEMTO_ERR_STATE, and a training step fed from it gives the loss of the
    same step fed directly."""
    kw = dict(sequence_len=96, max_document_tokens=64, vocab_size=100, n_layer=3, n_head=4, n_kv_head=2, n_embed=64,
              window_pattern="SL")
    cfg = fb.GPTConfig(**kw)
    lay = fb.parameter_layout(cfg)
    B, T = 3, 96
    pk = fb.PackedBatches(100, T, B, max_document_tokens=64, mean_doc_len=20, seed=4)
    batches = [pk.next() for _ in range(5)]
    fd = fb.Feeder(B, T, depth=2)
    fd.submit(*batches[0])
    fd.submit(*batches[1])
    L = _lib.lib()
    assert L.femto_feeder_submit(fd.f, fd._host_ptr(batches[2][0]), fd._host_ptr(batches[2][1]), None) == -4   # full
    theta = torch.zeros(lay.nparams)
    fo.initialize(theta, fo.GPTConfig(**kw), fo.parameter_layout(fo.GPTConfig(**kw)), 3, all_nonzero=True)
    params = fb.Params(theta.cuda())
    st = fb.GradientState(cfg, max_batch=B)
    st.refresh_weights(params.theta)
    for i in range(5):
        a, b, c = fd.next()
        got = fb.loss_and_gradient_(params, st, lay, a, b, c, batch=B)
        fd.release()
        if i + 2 < 5:
            fd.submit(*batches[i + 2])
        want = fb.loss_and_gradient_(params, st, lay, *(torch.from_numpy(x) for x in batches[i]))
        assert got == want, i
    a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
    assert L.femto_feeder_next(fd.f, None, C.byref(a), C.byref(b), C.byref(c)) == -4                       # empty
    fd.close()


@pytest.mark.parametrize("ak", [True, False])
@pytest.mark.parametrize("bk", [True, False])
def test_gemm_cta_pairs_equal_single_ctas(ak, bk):
    """256 x 256 tiles computed by CTA pairs (tcgen05.mma.cta_group::2) against 128 x 256 tiles by single CTAs: the
    same products summed in the same order, so bf16 results are bit-identical; ragged M (the last pair has an empty
    half), ragged N and K, a batch, and the fp32 split-K form."""
    L = _lib.lib()
    M, N, K, batch = 648, 520, 1288, 2
    g = torch.Generator(device="cuda").manual_seed(17)
    A = torch.randn(batch, M, K, generator=g, device="cuda").bfloat16()
    B = torch.randn(batch, K, N, generator=g, device="cuda").bfloat16()
    As = A.contiguous() if ak else A.transpose(1, 2).contiguous()
    Bs = B.transpose(1, 2).contiguous() if bk else B.contiguous()
    outs = []
    for mode in (0, 1):
        L.femto_gemm_pair_mode(mode)
        Cc = torch.zeros(batch, M, N, device="cuda", dtype=torch.bfloat16)
        _lib.check(L.femto_gemm_bf16(_lib.ptr(As), int(ak), K if ak else M, _lib.ptr(Bs), int(bk), K if bk else N,
                                     _lib.ptr(Cc), N, M, N, K, batch, M * K, K * N, M * N, 0, 0, None))
        torch.cuda.synchronize()
        outs.append(Cc.cpu())
    L.femto_gemm_pair_mode(1)
    ref = torch.bmm(A.double().cpu(), B.double().cpu())
    assert (outs[1].double() - ref).abs().max() <= 2.0 ** -8 * ref.abs().max()
    assert torch.equal(outs[0], outs[1])
    # fp32 accumulate with split-K (one matrix, long K)
    Kl = 8192
    A2 = torch.randn(Kl, 512, generator=g, device="cuda").bfloat16()
    B2 = torch.randn(Kl, 768, generator=g, device="cuda").bfloat16()
    res = []
    for mode in (0, 1):
        L.femto_gemm_pair_mode(mode)
        Cf = torch.ones(512, 768, device="cuda")
        _lib.check(L.femto_gemm_bf16(_lib.ptr(A2), 0, 512, _lib.ptr(B2), 0, 768, _lib.ptr(Cf), 768, 512, 768, Kl, 1, 0, 0, 0, 1, 1,
                                     None))
        torch.cuda.synchronize()
        res.append(Cf.cpu())
    L.femto_gemm_pair_mode(1)
    ref2 = 1.0 + A2.double().cpu().T @ B2.double().cpu()
    assert (res[1].double() - ref2).abs().max() <= 1e-5 * ref2.abs().max()
    assert (res[0] - res[1]).abs().max() <= 1e-5 * ref2.abs().max()   # split counts may differ between the modes


def test_bounded_wait_runs_out_cleanly():
    """Every mbarrier wait in the tensor-core kernels is bounded.  The self test waits 1024 polls on a barrier nobody
    arrives at: the waiter gives up and raises status bit 2, a second role waiting without a small limit unwinds
    through the abort flag, the kernel returns by itself and the context stays usable."""
    L = _lib.lib()
    status, res = C.c_int32(-1), (C.c_int32 * 2)()
    _lib.check(L.femto_selftest_bounded_wait(1024, C.byref(status), res))
    assert status.value == 2 and list(res) == [1, 1]
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum()) == 16.0                      # the device still answers
    w = C.c_int32(-1)
    _lib.check(L.femto_status_word(None, C.byref(w)))
    assert w.value == 0                                      # the self test cleared the word it raised
