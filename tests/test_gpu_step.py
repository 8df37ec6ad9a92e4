"""GPU parity of the whole training step through the C ABI against the CPU oracle."""
import os

import pytest
import torch

import femtochat_b200 as fb
from oracle import femto_oracle as fo

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TINY = dict(sequence_len=4, max_document_tokens=64, vocab_size=16, n_layer=2, n_head=2, n_kv_head=1, n_embed=32,
            window_pattern="L")
MID = dict(sequence_len=96, max_document_tokens=64, vocab_size=100, n_layer=3, n_head=4, n_kv_head=2, n_embed=64,
           window_pattern="SL")
# smallest shape that runs every tensor-core kernel: head_dim 128, GEMM tiles 128x256x64
TC = dict(sequence_len=256, max_document_tokens=512, vocab_size=1000, n_layer=4, n_head=4, n_kv_head=2, n_embed=512,
          window_pattern="SL")


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-300))


def inputs(cfg, B, seed=0, ignore=True):
    g = torch.Generator().manual_seed(seed)
    T = cfg["sequence_len"]
    tok = torch.randint(1, cfg["vocab_size"] + 1, (B, T), generator=g, dtype=torch.int32)
    tgt = torch.randint(1, cfg["vocab_size"] + 1, (B, T), generator=g, dtype=torch.int32)
    if ignore:
        tgt[0, T // 2] = -1
        tgt[B - 1, T - 3:] = -1
    pos = ((torch.arange(T)[None, :].repeat(B, 1) + 3 * torch.arange(B)[:, None]) % max(5, T // 2 + 1)).int()
    return tok, tgt, pos


def run_both(cfgkw, B, dtype, short_window=0, doc_mask=False, reduction="sum", nz=True, seed=0):
    cfg, ocfg = fb.GPTConfig(**cfgkw), fo.GPTConfig(**cfgkw)
    lay, olay = fb.parameter_layout(cfg), fo.parameter_layout(ocfg)
    tok, tgt, pos = inputs(cfgkw, B, seed)
    th = torch.zeros(lay.nparams, dtype=torch.float32)
    fo.initialize(th, ocfg, olay, 123, all_nonzero=nz)
    eps = fo.EPS_BF16 if dtype == "bfloat16" else fo.EPS_F32
    M = fo.Model(ocfg, fo.StepOptions(eps=eps, short_window=short_window, doc_mask=doc_mask, reduction=reduction))
    l0, g0, _ = M.loss_and_gradient(th.double() if dtype == "float32" else th, tok, tgt, pos)
    params = fb.Params(th.cuda())
    st = fb.gradient_state(params, cfg, lay, tok, tgt, pos, compute_type=dtype, short_window=short_window,
                           doc_mask=doc_mask)
    l1 = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos, reduction=reduction)
    g1 = params.delta.cpu().clone()
    l2 = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos, reduction=reduction)
    assert st.status_word() == 0
    bitwise = torch.equal(g1, params.delta.cpu()) and l1 == l2
    return dict(l0=l0, l1=l1, g0=g0, g1=g1, lay=lay, st=st, params=params, bitwise=bitwise, inputs=(tok, tgt, pos))


@pytest.mark.parametrize("nz", [False, True])
def test_readme_tiny_fp32(nz):
    """Config 1: loss within 1e-5 relative, delta cosine >= 0.999 (and far tighter in fp32)."""
    r = run_both(TINY, 2, "float32", nz=nz)
    assert abs(r["l1"] - r["l0"]) <= 1e-5 * abs(r["l0"])
    assert cosine(r["g0"], r["g1"]) >= 0.999999
    assert float((r["g0"] - r["g1"]).abs().max()) <= 2e-5 * float(r["g0"].abs().max())
    assert r["bitwise"]            # deterministic: no atomics anywhere in the step


def test_readme_tiny_sgd_golden():
    """README.md:74-83: 10 SGD steps on loss_sum / N at 0.01; per-step losses against the fixture."""
    gold = torch.load(os.path.join(GOLD, "readme_tiny.pt"))
    cfg = fb.GPTConfig(**TINY)
    lay = fb.parameter_layout(cfg)
    for name in ("ref_init", "all_nonzero"):
        c = gold[name]
        params = fb.Params(c["theta0"].clone().cuda())
        tok, tgt, pos = gold["tokens"], gold["targets"], gold["positions"]
        st = fb.gradient_state(params, cfg, lay, tok, tgt, pos)
        nt = int((tgt != -1).sum())
        for step in range(10):
            loss = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos, reduction="sum")
            if step == 0:
                assert cosine(params.delta.cpu(), c["delta_step1"]) >= 0.999999
            assert loss / nt == pytest.approx(float(c["losses"][step]), rel=1e-5)
            params.theta -= 0.01 * params.delta / nt
            st.refresh_weights(params.theta)
        assert float((params.theta.cpu() - c["theta10"]).abs().max()) < 1e-5


@pytest.mark.parametrize("doc_mask,reduction", [(False, "sum"), (True, "mean")])
def test_mid_fp32_windows_gqa(doc_mask, reduction):
    r = run_both(MID, 3, "float32", short_window=32, doc_mask=doc_mask, reduction=reduction)
    assert abs(r["l1"] - r["l0"]) <= 1e-5 * abs(r["l0"])
    assert cosine(r["g0"], r["g1"]) >= 0.999999
    assert r["bitwise"]


def test_index_handling_is_bit_exact():
    """Padded vocabulary rows and never-seen token rows get exactly zero gradient; an ignored
    target contributes nothing; out-of-range ids raise the status word instead of faulting."""
    r = run_both(MID, 3, "float32", short_window=32)
    lay, g1 = r["lay"], r["g1"]
    tok, tgt, pos = r["inputs"]
    V, Vp, d = MID["vocab_size"], lay.padded_vocab_size, MID["n_embed"]
    glm = g1[lay.lm_head.offset:lay.lm_head.offset + lay.lm_head.size].view(d, Vp)
    assert float(glm[:, V:].abs().max()) == 0.0
    gw = g1[lay.embedding.offset:lay.embedding.offset + lay.embedding.size].view(Vp, d)
    seen = set((tok - 1).flatten().tolist())
    unseen = [i for i in range(Vp) if i not in seen]
    assert float(gw[unseen].abs().max()) == 0.0
    assert all(float(gw[i].abs().max()) > 0 for i in list(seen)[:10])
    # n_valid
    cfg = fb.GPTConfig(**MID)
    st, params = r["st"], r["params"]
    loss, nv = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos, sync=False)
    assert int(nv.item()) == int((tgt != -1).sum())
    bad = tok.clone()
    bad[0, 0] = V + 5
    fb.loss_and_gradient_(params, st, lay, bad, tgt, pos)
    assert st.status_word() & 1


def test_accumulate_matches_two_micro_steps():
    """scripts/train.jl:117-131: the first micro-step overwrites delta, later ones add."""
    cfg = fb.GPTConfig(**MID)
    lay = fb.parameter_layout(cfg)
    th = torch.zeros(lay.nparams)
    fo.initialize(th, fo.GPTConfig(**MID), fo.parameter_layout(fo.GPTConfig(**MID)), 3, all_nonzero=True)
    params = fb.Params(th.cuda())
    a, b = inputs(MID, 2, 1), inputs(MID, 2, 2)
    st = fb.gradient_state(params, cfg, lay, *a)
    fb.loss_and_gradient_(params, st, lay, *a)
    ga = params.delta.clone()
    fb.loss_and_gradient_(params, st, lay, *b)
    gb = params.delta.clone()
    fb.loss_and_gradient_(params, st, lay, *a)
    fb.loss_and_gradient_(params, st, lay, *b, accumulate=True)
    assert float((params.delta - (ga + gb)).abs().max()) <= 1e-5 * float((ga + gb).abs().max())


def test_side_streams_give_the_bits_of_one_stream(monkeypatch):
    """A handle created with FEMTO_SIDE_STREAM=0 keeps every launch of the training step on the caller's stream; the
    default runs the weight-gradient GEMMs, the zero fill of delta and the AdamW tables on a second internal stream.
    Same kernels, same reduction orders: loss, delta, Theta and the moments must agree bit for bit over several
    steps (a missing dependency between the two streams shows up here as a difference)."""
    BIG = dict(sequence_len=512, max_document_tokens=512, vocab_size=2048, n_layer=6, n_head=4, n_kv_head=2, n_embed=512,
               window_pattern="SSL")
    cfg, ocfg = fb.GPTConfig(**BIG), fo.GPTConfig(**BIG)
    lay = fb.parameter_layout(cfg)
    th = torch.zeros(lay.nparams)
    fo.initialize(th, ocfg, fo.parameter_layout(ocfg), 11, all_nonzero=True)
    batches = [inputs(BIG, 4, seed) for seed in (1, 2, 3)]
    results = []
    for side in ("0", "1"):
        monkeypatch.setenv("FEMTO_SIDE_STREAM", side)
        params = fb.Params(th.clone().cuda())
        st = fb.gradient_state(params, cfg, lay, *batches[0], compute_type="bfloat16", short_window=128, doc_mask=True)
        opt = fb.MuonAdamW(params, lay, st, compute_type="bfloat16")
        losses, deltas = [], []
        for rep in range(2):          # two passes over the batches: the second one starts from updated weights
            for i, b in enumerate(batches):
                losses.append(fb.loss_and_gradient_(params, st, lay, *b, reduction="mean"))
                # a second micro-step that accumulates, then the update
                losses.append(fb.loss_and_gradient_(params, st, lay, *batches[(i + 1) % 3], reduction="mean", accumulate=True))
                deltas.append(params.delta.clone())
                opt.step(eta=0.5)
        torch.cuda.synchronize()
        assert st.status_word() == 0
        results.append((losses, deltas, params.theta.clone(),
                        [x.clone() for x in (opt.adam_m, opt.adam_v, opt.muon_m, opt.muon_v)]))
    (l0, d0, t0, s0), (l1, d1, t1, s1) = results
    assert l0 == l1
    for a, b in zip(d0, d1):
        assert torch.equal(a, b)
    assert torch.equal(t0, t1)
    for a, b in zip(s0, s1):
        assert torch.equal(a, b)


def test_bf16_small_simt_paths():
    r = run_both(MID, 3, "bfloat16", short_window=32)
    assert abs(r["l1"] - r["l0"]) <= 1e-2 * abs(r["l0"])
    assert cosine(r["g0"], r["g1"]) >= 0.999
    assert r["bitwise"]


@pytest.mark.parametrize("doc_mask", [False, True])
def test_bf16_tensor_core_paths(doc_mask):
    """bf16 build on shapes that take the tcgen05 GEMM, attention and lm_head-tail kernels:
    per-step loss within 1e-2 relative, delta cosine >= 0.999 (tolerances of the north-star)."""
    r = run_both(TC, 4, "bfloat16", short_window=128, doc_mask=doc_mask)
    assert abs(r["l1"] - r["l0"]) <= 1e-2 * abs(r["l0"])
    assert cosine(r["g0"], r["g1"]) >= 0.999
    lay = r["lay"]
    for name in ("wq", "wk", "wv", "wo", "fc", "proj"):
        for i, blk in enumerate(lay.blocks):
            s = blk[name]
            assert cosine(r["g0"][s.offset:s.offset + s.size], r["g1"][s.offset:s.offset + s.size]) >= 0.995, (i, name)
    for s in (lay.embedding, lay.lm_head):
        assert cosine(r["g0"][s.offset:s.offset + s.size], r["g1"][s.offset:s.offset + s.size]) >= 0.999
    assert r["bitwise"]


def test_forward_only_model_call_matches():
    cfg = fb.GPTConfig(**MID)
    lay = fb.parameter_layout(cfg)
    th = torch.zeros(lay.nparams)
    ocfg = fo.GPTConfig(**MID)
    fo.initialize(th, ocfg, fo.parameter_layout(ocfg), 3, all_nonzero=True)
    tok, tgt, pos = inputs(MID, 2)
    ref = float(fo.Model(ocfg, fo.StepOptions(reduction="mean")).forward(th.double(), tok, tgt, pos))
    model = fb.GPT(fb.Params(th.cuda()), cfg, lay)
    assert model(tok, tgt, positions=pos) == pytest.approx(ref, rel=1e-5)   # reduction=:mean is the call's default


def test_model_call_without_targets_returns_softcapped_logits():
    """`logits = model(tokens; positions)` (src/gpt.jl:129-170): fp32 [B][T][vocab_size], first V rows only."""
    cfg = fb.GPTConfig(**MID)
    lay = fb.parameter_layout(cfg)
    th = torch.zeros(lay.nparams)
    ocfg = fo.GPTConfig(**MID)
    fo.initialize(th, ocfg, fo.parameter_layout(ocfg), 5, all_nonzero=True)
    tok, tgt, pos = inputs(MID, 2)
    cache = {}
    fo.Model(ocfg, fo.StepOptions(reduction="sum")).forward(th.double(), tok, tgt, pos, cache=cache)
    z_ref = cache["z"].float()
    model = fb.GPT(fb.Params(th.cuda()), cfg, lay)
    z = model(tok, positions=pos).cpu()
    assert z.shape == (tok.shape[0], tok.shape[1], cfg.vocab_size)
    assert (z - z_ref.reshape(z.shape)).abs().max() <= 2e-4   # fp32 build: tolerance of the tanh/GEMM rounding
    assert z.abs().max() <= 15.0


def test_model_call_reduction_none_returns_token_losses():
    """reduction=:none (src/gpt.jl:191-193), the form the evaluation loop consumes (src/loss_eval.jl:8-46)."""
    cfg = fb.GPTConfig(**MID)
    lay = fb.parameter_layout(cfg)
    th = torch.zeros(lay.nparams)
    ocfg = fo.GPTConfig(**MID)
    fo.initialize(th, ocfg, fo.parameter_layout(ocfg), 7, all_nonzero=True)
    tok, tgt, pos = inputs(MID, 2)
    ref = fo.Model(ocfg, fo.StepOptions(reduction="none")).forward(th.double(), tok, tgt, pos)
    model = fb.GPT(fb.Params(th.cuda()), cfg, lay)
    got = model(tok, tgt, positions=pos, reduction="none").cpu()
    assert got.shape == tok.shape
    assert torch.equal(got == 0, (tgt == -1) | (ref.float() == 0))          # ignored slots are exactly zero
    assert torch.allclose(got.double(), ref.reshape(got.shape), rtol=1e-5, atol=1e-5)
    assert float(got.sum()) == pytest.approx(model(tok, tgt, positions=pos, reduction="sum"), rel=1e-6)


SHARD = dict(sequence_len=32, max_document_tokens=64, vocab_size=8192, n_layer=5, n_head=2, n_kv_head=1, n_embed=128,
             window_pattern="SL")


@pytest.mark.parametrize("cfgkw,ctype,world,tol", [(SHARD, "float32", 2, 1e-6), (SHARD, "float32", 3, 1e-6),
                                                   (TC, "bfloat16", 2, 2e-3)])
def test_owner_sharded_update_matches_full_update(cfgkw, ctype, world, tol):
    """Data-parallel owner-sharded MuonAdamW, emulated on one GPU: every rank updates only its share of Theta from the
    same delta; merging the shares by their owner must give the full update (src/optim.jl:430-440), the shares must
    be disjoint, and what no rank owns alone must come out the same on every rank."""
    cfg = fb.GPTConfig(**cfgkw)
    lay = fb.parameter_layout(cfg)
    theta0 = torch.empty(lay.nparams, dtype=torch.float32, device="cuda")
    fb.initialize_(theta0, lay, seed=5, all_nonzero=True)
    st = fb.GradientState(cfg, max_batch=1, compute_type=ctype)
    g = torch.Generator(device="cuda").manual_seed(9)
    deltas = [torch.randn(lay.nparams, generator=g, device="cuda") * 0.3 for _ in range(2)]

    full = fb.Params(theta0.clone())
    opt_full = fb.MuonAdamW(full, lay, st, compute_type=ctype, weight_decay=0.1)
    ranks = [fb.Params(theta0.clone()) for _ in range(world)]
    opts = [fb.MuonAdamW(p, lay, st, compute_type=ctype, weight_decay=0.1) for p in ranks]
    for r, o in enumerate(opts):
        o.shard(r, world)
    ranges = opts[0].shard_ranges()
    assert ranges == opts[world - 1].shard_ranges()
    assert sorted(ranges) == fb.shard_plan(lay, world)  # the library's partition is the documented one
    owned = torch.zeros(lay.nparams, dtype=torch.int32)
    for off, n, owner in ranges:
        assert 0 <= owner < world and n > 0
        owned[off:off + n] += 1
    assert int(owned.max()) == 1                       # disjoint
    muon_elems = sum(sp.size for grp in opt_full.muon for sp in grp.specs if sp.size >= 1024)   # gates: every rank
    big_tables = sum(gv.spec.size for gv in opt_full.adamw if gv.spec.size >= 1 << 20 and gv.spec.size % (4 * world) == 0)
    assert int(owned.sum()) == muon_elems + big_tables  # every Muon matrix and every divisible large table has one owner
    assert {o for _, _, o in ranges} == set(range(world))

    for i, d in enumerate(deltas):
        kw = dict(eta=0.5 + 0.25 * i, mu=0.9, lam=0.05, Nt=64.0)
        full.delta.copy_(d)
        opt_full.step(**kw)
        for p, o in zip(ranks, opts):
            p.delta.copy_(d)
            o.step(**kw)
        merged = ranks[0].theta.clone()
        shared = owned.cuda() == 0
        for p in ranks[1:]:
            assert torch.equal(p.theta[shared], merged[shared])      # replicated groups agree bit for bit
        for off, n, owner in ranges:
            merged[off:off + n] = ranks[owner].theta[off:off + n]
        err = float((merged - full.theta).abs().max())
        assert err <= tol, (i, err)
        for p in ranks:
            p.theta.copy_(merged)
    assert all(o.get_t() == opt_full.get_t() for o in opts)
    # the moments: each part of each state buffer is current on the rank that state_ranges names (what
    # gather_state collects before a checkpoint), and the covers tile the buffers
    for which, name in enumerate(["adam_m", "adam_v", "muon_m", "muon_v"]):
        cover = opts[0].state_ranges(which)
        want = getattr(opt_full, name)
        at = 0
        merged = torch.empty_like(want)
        for off, n, owner in cover:
            assert off == at and n > 0 and 0 <= owner < world
            merged[off:off + n] = getattr(opts[owner], name)[off:off + n]
            at += n
        assert at == want.numel()
        if which >= 2:                                 # every rank owns some block's matrices
            assert {o for _, _, o in cover} >= set(range(world))
        err = float((merged - want).abs().max())
        assert err <= tol * max(1.0, float(want.abs().max())), (name, err)
    opts[0].shard(0, 1)                                # back to the full update
    assert opts[0].shard_ranges() == []


def test_checkpoint_round_trip_resumes_bit_for_bit(tmp_path):
    """src/checkpoints.jl:9-39: the per-group optimiser state (AdamW m, v, t; Muon momentum and NorMuon second moment)
    and Theta go to a file, a FRESH optimiser restores them, and the next update equals the uninterrupted run's bit
    for bit.  The saved groups have the reference's order and shapes."""
    cfg = fb.GPTConfig(**SHARD)
    lay = fb.parameter_layout(cfg)
    theta0 = torch.empty(lay.nparams, dtype=torch.float32, device="cuda")
    fb.initialize_(theta0, lay, seed=5, all_nonzero=True)
    st = fb.GradientState(cfg, max_batch=1)
    g = torch.Generator(device="cuda").manual_seed(3)
    deltas = [torch.randn(lay.nparams, generator=g, device="cuda") * 0.3 for _ in range(3)]
    kw = dict(eta=0.7, mu=0.9, lam=0.05, Nt=64.0)

    a = fb.Params(theta0.clone())
    opt_a = fb.MuonAdamW(a, lay, st, weight_decay=0.1)
    for d in deltas[:2]:
        a.delta.copy_(d)
        opt_a.step(**kw)
    file = fb.save_checkpoint(str(tmp_path), 2, a, opt_a, dict(config=SHARD))
    assert file.endswith("checkpoint_000002.pt") and not os.path.exists(file + ".part")
    a.delta.copy_(deltas[2])
    opt_a.step(**kw)

    ck = fb.load_checkpoint(str(tmp_path), 2)
    assert ck["step"] == 2 and ck["metadata"]["config"] == SHARD
    saved = ck["optimizer"]
    # the reference's group structure (src/optim.jl:333-425): lm_head, wte, per block [ve table], lam_b, lam_x0, then
    # smear gate, lam_s, lam_y; Muon groups by shape in order of first appearance
    n_ve = sum(1 for b in lay.blocks if b["ve_table"] is not None)
    assert len(saved["adamw"]) == 2 + n_ve + 2 * cfg.n_layer + 3
    assert saved["adamw"][0]["m"].numel() == lay.lm_head.size and saved["adamw"][1]["m"].numel() == lay.embedding.size
    assert all(s["t"] == 2 for s in saved["adamw"])
    d, kv = cfg.n_embed, cfg.n_embed // cfg.n_head * cfg.n_kv_head
    shapes = [tuple(s["m"].shape) for s in saved["muon"]]         # row-major [k][cols][rows] of a Julia (rows, cols, k)
    assert shapes[0] == (2 * cfg.n_layer, d, d) and shapes[1] == (2 * cfg.n_layer, d, kv)
    assert shapes[2] == (cfg.n_layer, d, 4 * d) and shapes[3] == (cfg.n_layer, 4 * d, d)
    assert tuple(saved["muon"][2]["v"].shape) == (cfg.n_layer, 4 * d)      # fc is (4d, d): rows >= cols -> (rows,1,k)

    b = fb.Params(ck["parameters"].cuda())
    opt_b = fb.MuonAdamW(b, lay, st, weight_decay=0.1)             # fresh moments, t = 0
    fb.restore_optimizer_(opt_b, saved)
    assert opt_b.get_t() == opt_a.get_t()[:0] + [2] * len(opt_b.adamw)
    b.delta.copy_(deltas[2])
    opt_b.step(**kw)
    assert torch.equal(a.theta, b.theta)
    for x, y in ((opt_a.adam_m, opt_b.adam_m), (opt_a.adam_v, opt_b.adam_v), (opt_a.muon_m, opt_b.muon_m),
                 (opt_a.muon_v, opt_b.muon_v)):
        assert torch.equal(x, y)


GEN = dict(sequence_len=64, max_document_tokens=128, vocab_size=100, n_layer=3, n_head=4, n_kv_head=2, n_embed=64,
           window_pattern="SL")
GEN_TC = dict(sequence_len=256, max_document_tokens=512, vocab_size=1000, n_layer=4, n_head=4, n_kv_head=2, n_embed=512,
              window_pattern="SL")


@pytest.mark.parametrize("cfgkw,ctype,doc_mask,tol", [(GEN, "float32", False, 1e-4), (GEN, "float32", True, 1e-4),
                                                      (GEN_TC, "bfloat16", True, 3e-2)])
def test_kv_cache_decode_matches_full_context_recompute(cfgkw, ctype, doc_mask, tol):
    """src/generation.jl:40-52 recomputes the whole context for every token; with the key/value cache the prompt runs
    once and each new token is one row.  The logits of every decoded position must equal the oracle's logits of the
    full forward pass at that position (soft-capped, first vocab_size rows), for two columns with different
    tokens, a short window, positions that restart inside the prompt (a second document) and the document mask."""
    cfg, ocfg = fb.GPTConfig(**cfgkw), fo.GPTConfig(**cfgkw)
    lay, olay = fb.parameter_layout(cfg), fo.parameter_layout(ocfg)
    th = torch.zeros(lay.nparams)
    fo.initialize(th, ocfg, olay, 13, all_nonzero=True)
    T, V, B = cfgkw["sequence_len"], cfgkw["vocab_size"], 2
    g = torch.Generator().manual_seed(6)
    tok = torch.randint(1, V + 1, (B, T), generator=g, dtype=torch.int32)
    pos = torch.arange(T, dtype=torch.int32)[None, :].repeat(B, 1)
    pos[1, 9:] -= 9                                         # column 1: a new document starts at t = 9
    sw = T // 4
    eps = fo.EPS_BF16 if ctype == "bfloat16" else fo.EPS_F32
    cache_o = {}
    fo.Model(ocfg, fo.StepOptions(eps=eps, short_window=sw, doc_mask=doc_mask)).forward(
        th.double() if ctype == "float32" else th, tok, tok, pos, cache=cache_o)
    z_ref = cache_o["z"].float().reshape(B, T, V)           # logits of every position of the full sequence
    tol = tol * float(z_ref.abs().max()) + 1e-6             # relative to the largest logit
    model = fb.GPT(fb.Params(th.cuda()), cfg, lay, compute_type=ctype, short_window=sw, doc_mask=doc_mask)
    st = model.state(B)
    kc = fb.KVCache(st, B, T)
    Tp = 20 if T == 64 else 131                             # the prompt; not a multiple of any tile size
    z = fb.prefill(model, kc, tok[:, :Tp], pos[:, :Tp]).cpu()
    assert len(kc) == Tp
    assert (z - z_ref[:, Tp - 1]).abs().max() <= tol
    for t in range(Tp, min(T, Tp + 40)):
        z = fb.decode_step(model, kc, tok[:, t], pos[:, t]).cpu()
        assert (z - z_ref[:, t]).abs().max() <= tol, t
    assert len(kc) == min(T, Tp + 40)
    assert st.status_word() == 0
    # positions=None continues each column's document
    kc2 = fb.KVCache(st, B, T)
    fb.prefill(model, kc2, tok[:, :Tp], pos[:, :Tp])
    z2 = fb.decode_step(model, kc2, tok[:, Tp]).cpu()
    kc3 = fb.KVCache(st, B, T)
    fb.prefill(model, kc3, tok[:, :Tp], pos[:, :Tp])
    assert torch.equal(z2, fb.decode_step(model, kc3, tok[:, Tp], pos[:, Tp]).cpu())
    for c in (kc, kc2, kc3):
        c.close()


def test_generate_with_cache_equals_generate_by_recompute():
    """`generate` (src/generation.jl:26-56): greedy decoding (temperature 0) through the cache gives the tokens of
    the reference's recompute-everything loop; with sampling the same generator state gives the same tokens."""
    cfg = fb.GPTConfig(**GEN)
    lay = fb.parameter_layout(cfg)
    th = torch.zeros(lay.nparams)
    fo.initialize(th, fo.GPTConfig(**GEN), fo.parameter_layout(fo.GPTConfig(**GEN)), 2, all_nonzero=True)
    model = fb.GPT(fb.Params(th.cuda()), cfg, lay)
    prompt = [5, 17, 3, 42]
    a = fb.generate(model, prompt, max_new_tokens=12, temperature=0.0)
    b = fb.generate(model, prompt, max_new_tokens=12, temperature=0.0, use_cache=False)
    assert a == b and len(a) == 16 and a[:4] == prompt and all(1 <= t <= 100 for t in a)
    ga, gb = torch.Generator().manual_seed(1), torch.Generator().manual_seed(1)
    c = fb.generate(model, prompt, max_new_tokens=12, temperature=0.8, top_k=10, generator=ga)
    d = fb.generate(model, prompt, max_new_tokens=12, temperature=0.8, top_k=10, generator=gb, use_cache=False)
    assert c == d
    # the context window slides once the sequence is longer than sequence_len (src/generation.jl:41-43)
    e = fb.generate(model, list(range(1, 61)), max_new_tokens=8, temperature=0.0)
    f = fb.generate(model, list(range(1, 61)), max_new_tokens=8, temperature=0.0, use_cache=False)
    assert e == f and len(e) == 68


@pytest.mark.parametrize("cfgkw,ctype", [(MID, "float32"), (TC, "bfloat16")])
def test_update_kernels_refresh_the_compute_type_weights(cfgkw, ctype):
    """The AdamW and Muon update kernels write the model's compute-type copy of every weight in the same pass as
    Theta.  That copy must be exactly what a fresh cast of Theta gives: the loss right after an update equals, bit
    for bit, the loss after an explicit femto_refresh_weights."""
    cfg = fb.GPTConfig(**cfgkw)
    lay = fb.parameter_layout(cfg)
    th = torch.zeros(lay.nparams)
    fo.initialize(th, fo.GPTConfig(**cfgkw), fo.parameter_layout(fo.GPTConfig(**cfgkw)), 3, all_nonzero=True)
    tok, tgt, pos = inputs(cfgkw, 2, 5)
    params = fb.Params(th.cuda())
    st = fb.gradient_state(params, cfg, lay, tok, tgt, pos, compute_type=ctype)
    opt = fb.MuonAdamW(params, lay, st, compute_type=ctype, weight_decay=0.1)
    for step in range(2):
        fb.loss_and_gradient_(params, st, lay, tok, tgt, pos)
        opt.step(eta=1.0, Nt=float(tok.numel()))
        after_update = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos)
        delta_a = params.delta.clone()
        st.refresh_weights(params.theta)
        after_refresh = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos)
        assert after_update == after_refresh, step
        assert torch.equal(delta_a, params.delta)
