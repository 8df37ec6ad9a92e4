"""Generates tests/golden/*.pt from the CPU oracle (oracle/femto_oracle.py) on fixed seeded inputs.

The reference publishes no outputs for this path and cannot be run without a Julia toolchain, so
these are outputs of the restatement, not of the reference: they pin the oracle against accidental
edits and give the GPU tests fixed targets.  Run from the repository root:
    python tests/golden/make_golden.py
"""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import femto_oracle as fo  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

README_CFG = dict(sequence_len=4, max_document_tokens=64, vocab_size=16, n_layer=2, n_head=2, n_kv_head=1, n_embed=32,
                  window_pattern="L")


def readme_case():
    """README.md:57-63 inputs; 10 SGD steps at 0.01 on loss_sum / N (README.md:74-83)."""
    cfg = fo.GPTConfig(**README_CFG)
    lay = fo.parameter_layout(cfg)
    tokens = torch.tensor([[1, 2, 3, 4], [2, 3, 4, 5]], dtype=torch.int32)
    targets = torch.tensor([[2, 3, 4, 5], [3, 4, 5, 6]], dtype=torch.int32)
    positions = torch.tensor([[0, 1, 2, 3], [8, 9, 10, 11]], dtype=torch.int32)
    out = {}
    for name, nz in (("ref_init", False), ("all_nonzero", True)):
        th = torch.zeros(lay.nparams, dtype=torch.float32)
        fo.initialize(th, cfg, lay, 123, all_nonzero=nz)
        theta0 = th.clone()
        M = fo.Model(cfg, fo.StepOptions(eps=fo.EPS_F32, reduction="sum"))
        losses = []
        th64 = th.double()
        delta1 = None
        for step in range(10):
            loss, delta, _ = M.loss_and_gradient(th64, tokens, targets, positions)
            if step == 0:
                delta1 = delta.clone()
            nt = int((targets != -1).sum())
            th64 -= 0.01 * delta.double() / nt
            losses.append(loss / nt)
        out[name] = dict(theta0=theta0, delta_step1=delta1, losses=torch.tensor(losses, dtype=torch.float64),
                         theta10=th64.float())
    out["tokens"], out["targets"], out["positions"] = tokens, targets, positions
    torch.save(out, os.path.join(HERE, "readme_tiny.pt"))


def optimizer_case():
    """Three MuonAdamW steps on a small GQA model with seeded gradients."""
    cfg = fo.GPTConfig(sequence_len=32, max_document_tokens=64, vocab_size=96, n_layer=2, n_head=4, n_kv_head=2,
                       n_embed=64, window_pattern="SL")
    lay = fo.parameter_layout(cfg)
    th = torch.zeros(lay.nparams, dtype=torch.float32)
    fo.initialize(th, cfg, lay, 7, all_nonzero=True)
    theta0 = th.clone()
    g = torch.Generator().manual_seed(11)
    deltas = [torch.randn(lay.nparams, generator=g) * 3.0 for _ in range(3)]
    opt = fo.MuonAdamW(lay, weight_decay=0.1)
    thetas = []
    for i, d in enumerate(deltas):
        opt.step(th, d, eta=0.5 + 0.25 * i, mu=0.9, lam=0.05, Nt=64.0)
        thetas.append(th.clone())
    torch.save(dict(theta0=theta0, deltas=deltas, thetas=thetas), os.path.join(HERE, "optimizer_small.pt"))


if __name__ == "__main__":
    readme_case()
    optimizer_case()
    print("wrote", os.listdir(HERE))
