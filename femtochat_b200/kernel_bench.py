"""Isolated kernel sweep: attention forward/reverse, fused lm_head tail,
Newton-Schulz chains and the GEMM forms of the step, timed with CUDA events on seeded Gaussian inputs.

    python -m femtochat_b200.kernel_bench [--kernel all|attn|xent|ns|gemm|stream] [--small] [--iters N]

`--small` shrinks the problem (for profiler captures); the default shapes are the benchmark's:
attention B=8, T=2048, 10 query / 5 kv heads, head_dim 128, geometric(512) documents;
cross-entropy 65536 tokens x 1280 against a 65536-vocabulary head; Newton-Schulz on 1280x1280 and
1280x5120 stacks."""
from __future__ import annotations

import argparse
import ctypes as C

import numpy as np
import torch

from . import _lib


def _time(fn, iters):
    for _ in range(3):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def doc_starts(B, T, mean=512, seed=2):
    rng = np.random.default_rng(seed)
    ds = np.zeros((B, T), dtype=np.int32)
    for b in range(B):
        t = 0
        while t < T:
            n = int(max(2, rng.geometric(1.0 / mean)))
            ds[b, t:t + n] = t
            t += n
    return torch.from_numpy(ds).cuda()


def unmasked_pairs(T, left, ds=None):
    q = np.arange(T)
    lo = np.maximum(0, q - left)
    if ds is not None:
        lo = np.maximum(lo[None, :], ds.cpu().numpy())
        return int((q[None, :] - lo + 1).sum())
    return int((q - lo + 1).sum())


def bench_attention(small, iters):
    L = _lib.lib()
    B, T, H, Hkv, hd = (2, 2048, 10, 5, 128) if small else (8, 2048, 10, 5, 128)
    g = torch.Generator(device="cuda").manual_seed(1)
    mk = lambda *s: torch.randn(*s, generator=g, device="cuda").bfloat16()
    Q, K, V, dO = mk(B, T, H, hd), mk(B, T, Hkv, hd), mk(B, T, Hkv, hd), mk(B, T, H, hd)
    O, lse = torch.zeros_like(Q), torch.zeros(B, H, T, device="cuda")
    dQ, dK, dV = torch.zeros_like(Q), torch.zeros_like(K), torch.zeros_like(V)
    ds = doc_starts(B, T)
    for name, left, docs in (("causal", T, None), ("causal+documents", T, ds), ("window 1024", 1024, None),
                             ("window 512", 512, None)):
        fwd = lambda: _lib.check(L.femto_attention_fwd(_lib.BF16, _lib.ptr(O), None, None, _lib.ptr(lse), _lib.ptr(Q),
                                                       _lib.ptr(K), _lib.ptr(V), B, T, H, Hkv, hd, left, _lib.ptr(docs), None))
        bwd = lambda: _lib.check(L.femto_attention_bwd_static(_lib.BF16, _lib.ptr(dQ), _lib.ptr(dK), _lib.ptr(dV), _lib.ptr(dO),
                                                              _lib.ptr(Q), _lib.ptr(K), _lib.ptr(V), _lib.ptr(O), _lib.ptr(lse),
                                                              B, T, H, Hkv, hd, left, _lib.ptr(docs), None))
        pairs = unmasked_pairs(T, left, docs) if docs is not None else unmasked_pairs(T, left) * B
        fl = 4.0 * hd * pairs * H
        tf, tb = _time(fwd, iters), _time(bwd, iters)
        print(f"attention {name:18s} fwd {tf:7.3f} ms {fl / tf / 1e9:7.0f} TFLOP/s | bwd {tb:7.3f} ms {2.5 * fl / tb / 1e9:7.0f} TFLOP/s "
              f"(exact unmasked pairs; bwd credited 2.5x fwd)")


def bench_xent(small, iters):
    L = _lib.lib()
    N, D, V = (8192, 1280, 65536) if small else (65536, 1280, 65536)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(N, D, generator=g, device="cuda")
    x = (x / x.pow(2).mean(-1, keepdim=True).sqrt()).bfloat16()
    W = (torch.randn(D, V, generator=g, device="cuda") * 0.02).bfloat16()
    tgt = torch.randint(0, V, (N,), generator=g, device="cuda", dtype=torch.int32)
    tgt[::100] = -1
    dx, dw = torch.zeros_like(x), torch.zeros(D, V, device="cuda")
    loss, nv = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda", dtype=torch.int32)
    fn = lambda: _lib.check(L.femto_xent_fused(_lib.BF16, _lib.ptr(x), _lib.ptr(W), V, _lib.ptr(tgt), N, D, V, 1.0, _lib.ptr(dx),
                                               _lib.ptr(dw), _lib.ptr(loss), _lib.ptr(nv), None))
    t = _time(fn, max(1, iters // 2))
    print(f"fused lm_head tail N={N} d={D} V={V}: {t:8.3f} ms  {6.0 * N * D * V / t / 1e9:7.0f} TFLOP/s credited (6NdV)  "
          f"loss/token {float(loss) / int(nv):.4f}")


def bench_ns(small, iters):
    L = _lib.lib()
    from .optim import POLAR_EXPRESS_COEFFS, QUINTIC_COEFFS
    for rows, cols, k in ((1280, 1280, 8 if small else 40), (1280, 5120, 4 if small else 20)):
        g = torch.Generator(device="cuda").manual_seed(3)
        X0 = torch.randn(k, rows, cols, generator=g, device="cuda")
        X0 = (X0 / (1.01 * X0.pow(2).sum(dim=(1, 2), keepdim=True).sqrt() + 1e-6)).bfloat16()
        for nm, co in (("quintic", QUINTIC_COEFFS), ("polar-express", POLAR_EXPRESS_COEFFS)):
            cf = (C.c_float * 15)(*[c for abc in co for c in abc])
            X = X0.clone()
            fn = lambda: _lib.check(L.femto_newton_schulz(_lib.BF16, _lib.ptr(X), k, rows, cols, cf, 5, None))
            t = _time(fn, max(1, iters // 2))
            r, c = min(rows, cols), max(rows, cols)
            fl = 5.0 * (4.0 * r * r * c + 2.0 * r ** 3) * k
            print(f"newton-schulz {nm:13s} {k} x [{rows}x{cols}]: {t:8.3f} ms  {fl / t / 1e9:7.0f} TFLOP/s")


def bench_gemm(small, iters):
    L = _lib.lib()
    N = 16384 if small else 65536
    # fp32 weight gradient with accumulation, the form the step uses (split-K partials + ordered reduce)
    for mode in (0, 1):
        L.femto_gemm_pair_mode(mode)
        A = torch.randn(N, 1280, device="cuda").bfloat16()
        B = torch.randn(N, 5120, device="cuda").bfloat16()
        Cf = torch.zeros(1280, 5120, device="cuda")
        fn = lambda: _lib.check(L.femto_gemm_bf16(_lib.ptr(A), 0, 1280, _lib.ptr(B), 0, 5120, _lib.ptr(Cf), 5120, 1280, 5120, N,
                                                  1, 0, 0, 0, 1, 1, None))
        t = _time(fn, iters)
        print(f"gemm dW += X^T dY (fc, fp32) 1280x5120x{N} {'CTA pairs' if mode else 'single CTAs'}: {t:7.3f} ms "
              f"{2.0 * 1280 * 5120 * N / t / 1e9:7.0f} TFLOP/s")
    for mode in (0, 1):
      L.femto_gemm_pair_mode(mode)
      print("tile mode:", "CTA pairs, 256 x 256 tiles (cta_group::2)" if mode else "single CTAs, 128 x 256 tiles")
      for nm, M, Nn, K, ak, bk in (("Y = X W      (fc)", N, 5120, 1280, 1, 0), ("Y = X W    (proj)", N, 1280, 5120, 1, 0),
                                 ("dX = dY W^T  (fc)", N, 1280, 5120, 1, 1), ("dW = X^T dY  (fc)", 1280, 5120, N, 0, 0)):
        A = torch.randn(M, K, device="cuda").bfloat16()
        B = torch.randn(K, Nn, device="cuda").bfloat16()
        As = A if ak else A.t().contiguous()
        Bs = B.t().contiguous() if bk else B
        Cc = torch.empty(M, Nn, device="cuda", dtype=torch.bfloat16)
        fn = lambda: _lib.check(L.femto_gemm_bf16(_lib.ptr(As), ak, K if ak else M, _lib.ptr(Bs), bk, K if bk else Nn,
                                                  _lib.ptr(Cc), Nn, M, Nn, K, 1, 0, 0, 0, 0, 0, None))
        t = _time(fn, iters)
        print(f"gemm {nm} {M}x{Nn}x{K}: {t:7.3f} ms {2.0 * M * Nn * K / t / 1e9:7.0f} TFLOP/s")
    L.femto_gemm_pair_mode(1)


def bench_stream(small, iters):
    """HBM-bound kernels that have their own entry point: AdamW (28 B per parameter) and the deterministic
    embedding-gradient scatter (2 B per input element read + fp32 read-modify-write of the touched rows)."""
    L = _lib.lib()
    n = (1 << 22) if small else 83886080          # one embedding table of the d20 model
    th, de = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    fn = lambda: _lib.check(L.femto_adamw(_lib.ptr(th), _lib.ptr(de), _lib.ptr(m), _lib.ptr(v), n, 1e-3, 0.9, 0.95, 1e-10,
                                          0.0, 3, 65536.0, None))
    t = _time(fn, iters)
    print(f"adamw n={n}: {t:7.3f} ms {28.0 * n / t / 1e6:7.0f} GB/s (28 B/param)")
    N, D, rows = (8192, 1280, 65536) if small else (65536, 1280, 65536)
    rng = np.random.default_rng(4)
    ranks = np.arange(1, rows + 1, dtype=np.float64) ** -1.1     # Zipf(1.1): a few rows receive thousands of adds
    tok = torch.from_numpy(rng.choice(rows, size=N, p=ranks / ranks.sum()).astype(np.int32)).cuda()
    dy = torch.randn(N, D, device="cuda").bfloat16()
    table = torch.zeros(rows, D, device="cuda")
    fn = lambda: _lib.check(L.femto_embedding_gradient(_lib.BF16, _lib.ptr(table), _lib.ptr(dy), _lib.ptr(tok), N, D, rows, None))
    t = _time(fn, iters)
    touched = int(torch.unique(tok).numel())
    byts = 2.0 * N * D + 8.0 * touched * D
    print(f"embedding scatter N={N} D={D} rows touched {touched}: {t:7.3f} ms {byts / t / 1e6:7.0f} GB/s "
          f"(input read + fp32 read-modify-write of touched rows; the stand-alone call also builds the sort / run-length "
          f"plan every time, which the training step does once per batch for its eleven tables)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all", choices=["all", "attn", "xent", "ns", "gemm", "stream"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    if a.kernel in ("all", "gemm"):
        bench_gemm(a.small, a.iters)
    if a.kernel in ("all", "attn"):
        bench_attention(a.small, a.iters)
    if a.kernel in ("all", "xent"):
        bench_xent(a.small, a.iters)
    if a.kernel in ("all", "ns"):
        bench_ns(a.small, a.iters)
    if a.kernel in ("all", "stream"):
        bench_stream(a.small, a.iters)


if __name__ == "__main__":
    main()
