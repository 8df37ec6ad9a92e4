"""Properties of the training step at the benchmark's full size (d20, 32 x 2048 tokens, bf16, document
mask, short window 1024), where the CPU oracle is far too slow to run: they hold for any input, so they
check the large-shape code paths (64-bit offsets, all GEMM tile / split-K configurations, full-length
attention, 65 536-row tables) that the small parity cases cannot reach."""
import numpy as np
import pytest
import torch

import femtochat_b200 as fb

pytestmark = pytest.mark.gpu

D20 = dict(sequence_len=2048, max_document_tokens=8192, vocab_size=65536, n_layer=20, n_head=10, n_kv_head=5,
           n_embed=1280, window_pattern="SSSL")


@pytest.fixture(scope="module")
def d20():
    if torch.cuda.get_device_properties(0).total_memory < 100e9:
        pytest.skip("needs about 70 GB of device memory")
    cfg = fb.GPTConfig(**D20)
    lay = fb.parameter_layout(cfg)
    theta = torch.empty(lay.nparams, device="cuda")
    fb.initialize_(theta, lay, seed=123, all_nonzero=True)
    params = fb.Params(theta)
    B = 32
    st = fb.GradientState(cfg, max_batch=B, compute_type="bfloat16", short_window=1024, doc_mask=True)
    st.refresh_weights(theta)
    pk = fb.PackedBatches(cfg.vocab_size, cfg.sequence_len, B)
    tok, tgt, pos = (torch.from_numpy(x).cuda() for x in pk.next())
    tgt = tgt.clone()
    tgt[3, 100:164] = -1          # some ignored targets
    yield dict(cfg=cfg, lay=lay, params=params, st=st, batch=(tok, tgt, pos), B=B)
    st.close()


def test_step_is_bitwise_repeatable_and_accumulation_is_exact(d20):
    p, st, lay = d20["params"], d20["st"], d20["lay"]
    tok, tgt, pos = d20["batch"]
    l1 = fb.loss_and_gradient_(p, st, lay, tok, tgt, pos, reduction="sum")
    g1 = p.delta.clone()
    l2 = fb.loss_and_gradient_(p, st, lay, tok, tgt, pos, reduction="sum")
    assert st.status_word() == 0
    assert l1 == l2 and torch.equal(g1, p.delta)                 # fixed summation order everywhere
    # a second micro-step on the same batch adds the same gradient.  Tensors whose gradient is produced by one
    # accumulation (the block matrices) double exactly; lm_head is accumulated chunk by chunk, so there the
    # association order of the fp32 sums differs and only rounding-level agreement holds.
    fb.loss_and_gradient_(p, st, lay, tok, tgt, pos, reduction="sum", accumulate=True)
    for blk in (lay.blocks[0], lay.blocks[len(lay.blocks) // 2], lay.blocks[-1]):
        for name in ("wq", "wk", "wv", "wo", "fc", "proj"):
            r = blk[name].range
            assert torch.equal(p.delta[r.start:r.stop], 2 * g1[r.start:r.stop]), name
    assert torch.allclose(p.delta, 2 * g1, rtol=1e-5, atol=1e-6 * float(g1.abs().max()))
    assert np.isfinite(l1) and 9.0 < l1 / int((tgt != -1).sum()) < 12.5   # near log(65536) = 11.09 at initialisation
    assert bool(torch.isfinite(g1).all())


def test_rows_of_unseen_tokens_have_exactly_zero_gradient(d20):
    p, st, lay = d20["params"], d20["st"], d20["lay"]
    tok, tgt, pos = d20["batch"]
    fb.loss_and_gradient_(p, st, lay, tok, tgt, pos, reduction="sum")
    seen = torch.zeros(d20["cfg"].vocab_size, dtype=torch.bool, device="cuda")
    seen[(tok - 1).long().flatten()] = True
    V = d20["cfg"].vocab_size
    unseen = ~seen
    assert int(unseen.sum()) > 0
    tables = [fb.paramview(p.delta, lay.embedding)] + [fb.paramview(p.delta, b["ve_table"]) for b in lay.blocks if b["ve_table"]]
    assert len(tables) == 11                                      # wte and the ten value-embedding tables
    for t in tables:                                              # row-major [padded vocabulary][channels]
        assert t.shape[0] >= V
        assert float(t[:V][unseen].abs().max()) == 0.0
        assert float(t[:V][seen].abs().sum()) > 0.0


def test_sum_of_token_losses_is_the_summed_loss_and_ignored_slots_are_zero(d20):
    p, lay, cfg = d20["params"], d20["lay"], d20["cfg"]
    tok, tgt, pos = d20["batch"]
    model = fb.GPT(p, cfg, lay, compute_type="bfloat16", short_window=1024, doc_mask=True)
    model._state = d20["st"]                                      # reuse the 50 GB arena
    per_token = model(tok, tgt, positions=pos, reduction="none")
    total = model(tok, tgt, positions=pos, reduction="sum")
    mean = model(tok, tgt, positions=pos, reduction="mean")
    nvalid = int((tgt != -1).sum())
    assert per_token.shape == tok.shape
    assert float(per_token[tgt == -1].abs().max()) == 0.0
    assert float(per_token.double().sum()) == pytest.approx(total, rel=1e-5)
    assert mean == pytest.approx(total / nvalid, rel=1e-5)
    assert bool((per_token[tgt != -1] > 0).all())                 # logsumexp(z) > z[target]
