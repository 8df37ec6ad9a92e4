"""Data-parallel parity on real GPUs: N ranks through the library == 1 rank on the concatenated batch.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        -m femtochat_b200.dp_check

The reference is single-GPU (scripts/train.jl:13); its micro-step accumulation (scripts/train.jl:117-131) and its
update (src/optim.jl:430-440) define what the N-rank job must reproduce.  Every rank runs the library on its own
columns of one global batch; rank 0 also runs a second, single-rank handle on all columns.  Compared after each of
three updates: the loss sum and the token count, the summed gradient (on its owner where the sharded sum sends a
range to one rank only), Theta, and (after femto_optimizer_gather_state) the four moment buffers.  Cases: owner-
sharded and replicated update, two micro-steps with the sum taken after the last one only, and the bucketed sum that
overlaps the reverse pass; the sharded update with both forms of its exchange (fp32 Theta every step, or only the
compute-type weights with Theta completed on demand).  After every update the loss of a forward pass over each
rank's columns, summed over ranks, is compared with the single-rank model's: the weights a rank computes with must be
complete and current.  Plain NCCL collectives only.  Prints ONE JSON line on rank 0; exit code 0 iff every
check passed.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

import torch
import torch.distributed as dist

import femtochat_b200 as fb
from femtochat_b200 import _lib

CASES = {
    # fp32 build: the gradients differ by summation order only (tol_delta); Theta and the moments pass through five
    # Newton-Schulz iterations, which amplify those last-bit differences (tol)
    "fp32": dict(cfg=dict(sequence_len=32, max_document_tokens=64, vocab_size=8192, n_layer=5, n_head=2, n_kv_head=1,
                          n_embed=128, window_pattern="SL"), ctype="float32", tol_delta=1e-5, tol=2e-4),
    # bf16 build on the tensor-core kernels: each rank's partial gradient is rounded on its own
    "bf16": dict(cfg=dict(sequence_len=256, max_document_tokens=512, vocab_size=4096, n_layer=4, n_head=4, n_kv_head=2,
                          n_embed=512, window_pattern="SL"), ctype="bfloat16", tol_delta=1e-3, tol=2e-2),
}


def share_nccl_id(rank):
    idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        buf = C.create_string_buffer(128)
        _lib.check(_lib.lib().femto_nccl_unique_id(buf))
        idt.copy_(torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8))
    dist.broadcast(idt, 0)
    return bytes(idt.cpu().numpy().tobytes())


def rel_err(a, b):
    return float((a.double() - b.double()).abs().max() / (b.double().abs().max() + 1e-30))


def run_case(name, spec, rank, world, sharded, micro_steps, overlap, exchange=0):
    cfg = fb.GPTConfig(**spec["cfg"])
    lay = fb.parameter_layout(cfg)
    T, Bl = cfg.sequence_len, 2
    B = Bl * world
    nccl_id = share_nccl_id(rank)
    theta0 = torch.empty(lay.nparams, dtype=torch.float32, device="cuda")
    fb.initialize_(theta0, lay, seed=5, all_nonzero=True)          # same seed on every rank -> same Theta
    g = torch.Generator().manual_seed(1234)
    steps = 3
    batches = []
    for _ in range(steps * micro_steps):
        tok = torch.randint(1, cfg.vocab_size + 1, (B, T), generator=g, dtype=torch.int32)
        tgt = torch.randint(1, cfg.vocab_size + 1, (B, T), generator=g, dtype=torch.int32)
        tgt[1, 3] = -1
        tgt[B - 1, T - 2:] = -1
        pos = ((torch.arange(T)[None, :].repeat(B, 1) + 3 * torch.arange(B)[:, None]) % (T // 2 + 1)).int()
        batches.append((tok.cuda(), tgt.cuda(), pos.cuda()))

    params = fb.Params(theta0.clone())
    st = fb.GradientState(cfg, max_batch=Bl, compute_type=spec["ctype"], short_window=16, doc_mask=True, rank=rank,
                          world=world, nccl_id=nccl_id)
    st.refresh_weights(params.theta)
    opt = fb.MuonAdamW(params, lay, st, compute_type=spec["ctype"], weight_decay=0.1)
    if sharded:
        opt.shard(rank, world)
        opt.set_exchange(exchange)
    ranges = opt.shard_ranges() if sharded else []

    ref = None
    if rank == 0:
        rp = fb.Params(theta0.clone())
        rst = fb.GradientState(cfg, max_batch=B, compute_type=spec["ctype"], short_window=16, doc_mask=True)
        rst.refresh_weights(rp.theta)
        ropt = fb.MuonAdamW(rp, lay, rst, compute_type=spec["ctype"], weight_decay=0.1)
        ref = (rp, rst, ropt)

    worst = dict(loss=0.0, delta=0.0, theta=0.0, moments=0.0, loss_after_update=0.0)
    nt_exact = True
    replicated = True
    loss_acc = torch.zeros(1, device="cuda")
    nv_acc = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in range(steps):
        loss_acc.zero_()
        nv_acc.zero_()
        for ms in range(micro_steps):
            tok, tgt, pos = batches[step * micro_steps + ms]
            sl = slice(rank * Bl, (rank + 1) * Bl)
            last = ms == micro_steps - 1
            _lib.check(_lib.lib().femto_set_overlap(st.h, 1 if (overlap and last) else 0))
            l, nv = fb.loss_and_gradient_(params, st, lay, tok[sl].contiguous(), tgt[sl].contiguous(),
                                          pos[sl].contiguous(), reduction="sum", accumulate=ms > 0, sync=False)
            loss_acc += l
            nv_acc += nv
        opt.grad_sync(loss_acc, nv_acc)                           # only after the last micro-step
        torch.cuda.synchronize()
        nt = int(nv_acc.item())
        delta_local = params.delta.clone()
        kw = dict(eta=0.5 + 0.25 * step, mu=0.9, lam=0.05, Nt=float(nt))
        opt.step(**kw)
        # The weights every rank now computes with (exchanged by the step) must be complete and current: the loss of a
        # forward pass over this rank's columns, summed over ranks, against the single-rank model after ITS update.
        ftok, ftgt, fpos = batches[step * micro_steps]
        tok, tgt, pos = ftok, ftgt, fpos
        sl = slice(rank * Bl, (rank + 1) * Bl)
        fwd = torch.zeros(1, device="cuda")
        _lib.check(_lib.lib().femto_forward_loss(st.h, _lib.ptr(params.theta), _lib.ptr(tok[sl].contiguous()),
                                                 _lib.ptr(tgt[sl].contiguous()), _lib.ptr(pos[sl].contiguous()), Bl, 0,
                                                 _lib.ptr(fwd), _lib.ptr(st._nvalid), _lib.stream_ptr()))
        dist.all_reduce(fwd)
        if sharded and exchange == 1:
            opt.gather_theta()     # the fp32 Theta is completed on demand in this mode
        opt.gather_state()
        torch.cuda.synchronize()
        # Theta identical on every rank (bitwise) after the exchange, before anything else touches it
        cs = torch.stack([params.theta.double().sum(), params.theta.double().abs().sum()])
        hi, lo = cs.clone(), cs.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        replicated = replicated and bool((hi == lo).all().item())

        # the owners' parts of delta travel to rank 0 for the comparison
        owner_parts = []
        for off, n, owner in ranges:
            buf = delta_local[off:off + n].clone()
            dist.broadcast(buf, owner)
            owner_parts.append((off, n, buf))
        if rank == 0:
            rp, rst, ropt = ref
            rl, rnv = 0.0, 0
            for ms in range(micro_steps):
                tok, tgt, pos = batches[step * micro_steps + ms]
                l, nv = fb.loss_and_gradient_(rp, rst, lay, tok, tgt, pos, reduction="sum", accumulate=ms > 0, sync=False)
                rl += float(l.item())
                rnv += int(nv.item())
            nt_exact = nt_exact and (rnv == nt)
            worst["loss"] = max(worst["loss"], abs(float(loss_acc.item()) - rl) / abs(rl))
            merged = delta_local.clone()
            for off, n, buf in owner_parts:
                merged[off:off + n] = buf
            worst["delta"] = max(worst["delta"], rel_err(merged, rp.delta))
            ropt.step(**{**kw, "Nt": float(rnv)})
            rf = torch.zeros(1, device="cuda")
            _lib.check(_lib.lib().femto_forward_loss(rst.h, _lib.ptr(rp.theta), _lib.ptr(ftok), _lib.ptr(ftgt), _lib.ptr(fpos), B, 0,
                                                     _lib.ptr(rf), _lib.ptr(rst._nvalid), _lib.stream_ptr()))
            torch.cuda.synchronize()
            worst["loss_after_update"] = max(worst["loss_after_update"], abs(float(fwd.item()) - float(rf.item())) / abs(float(rf.item())))
            worst["theta"] = max(worst["theta"], rel_err(params.theta, rp.theta))
            for a, b in ((opt.adam_m, ropt.adam_m), (opt.adam_v, ropt.adam_v), (opt.muon_m, ropt.muon_m),
                         (opt.muon_v, ropt.muon_v)):
                worst["moments"] = max(worst["moments"], rel_err(a, b))
            # keep both trajectories together so that later steps compare one update, not accumulated drift
            params.theta.copy_(rp.theta)
        dist.broadcast(params.theta, 0)
        st.refresh_weights(params.theta)
    status = st.status_word()
    tol = spec["tol"]
    ok = (nt_exact and replicated and status == 0 and worst["loss"] <= 1e-5 + tol * 1e-2 and worst["delta"] <= spec["tol_delta"] and
          worst["theta"] <= tol and worst["moments"] <= tol and worst["loss_after_update"] <= tol and
          int(_lib.lib().femto_comm_check(st.h)) == 0)
    opt.close()
    st.close()
    if ref is not None:
        ref[2].close()
        ref[1].close()
    return dict(case=name, sharded=sharded, micro_steps=micro_steps, overlap=overlap,
                exchange=("compute-type weights" if (sharded and exchange == 1) else "fp32 Theta"), ok=bool(ok), nt_exact=nt_exact,
                theta_bitwise_replicated=replicated, status=status, **{k: float(v) for k, v in worst.items()})


def main():
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    results = []
    for name, spec in CASES.items():
        for sharded, micro, overlap, exchange in ((True, 1, False, 0), (True, 1, False, 1), (False, 1, False, 0),
                                                  (True, 2, False, 1), (False, 1, True, 0)):
            results.append(run_case(name, spec, rank, world, sharded, micro, overlap, exchange))
    ok = torch.tensor([1 if all(r["ok"] for r in results) else 0], device="cuda")
    dist.broadcast(ok, 0)
    if rank == 0:
        print(json.dumps(dict(check="data-parallel parity: N ranks == 1 rank on the concatenated batch", n_gpus=world,
                              ok=bool(ok.item()), cases=results)), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
