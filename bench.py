"""Benchmark of the GPT training step (forward, reverse, gradient sync, Muon/AdamW update).

    python bench.py --gpus N --steps K --warmup W            # this library, one rank per GPU
    python bench.py --impl reference --gpus N --steps K ...   # CPU restatement of the reference

Prints ONE JSON line: training tokens/s at d20 (1280-wide, 20 layers, T=2048, B=32 per GPU),
device-timed with CUDA events, max over ranks.  Inputs are synthetic (Zipf(1.1) tokens, BOS,
geometric(512) documents) and weights random-init: the climbmix dataset and a trained tokenizer
are not available offline.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # the headline model: d20, GQA 10/5, "SSSL" with a 1024-token short window, B=32 per GPU
    "d20": dict(cfg=dict(sequence_len=2048, max_document_tokens=8192, vocab_size=65536, n_layer=20, n_head=10,
                         n_kv_head=5, n_embed=1280, window_pattern="SSSL"), batch=32, short_window=1024),
    # d12, full windows, one GPU
    "d12": dict(cfg=dict(sequence_len=2048, max_document_tokens=8192, vocab_size=65536, n_layer=12, n_head=6,
                         n_kv_head=6, n_embed=768, window_pattern="L"), batch=32, short_window=0),
    # d26: B=16 per GPU x 2 gradient-accumulation micro-steps per update
    "d26": dict(cfg=dict(sequence_len=2048, max_document_tokens=8192, vocab_size=65536, n_layer=26, n_head=13,
                         n_kv_head=13, n_embed=1664, window_pattern="SSSL"), batch=16, short_window=1024, micro_steps=2),
    "small": dict(cfg=dict(sequence_len=256, max_document_tokens=512, vocab_size=4096, n_layer=4, n_head=4,
                           n_kv_head=2, n_embed=512, window_pattern="SL"), batch=8, short_window=128),
}


# DRAM traffic of the dominant kernel from one ncu capture of the full-size step (dram__bytes_read.sum +
# dram__bytes_write.sum over the 312 gemm_tc_kernel launches of a step; profiles/gemm_tc_kernel_d20_step_dram.md),
# and the algorithmic bytes of the same launches (operands and results once, fp32 weight gradients read-modify-write).
NCU_GEMM_TRAFFIC = {("d20", 32, 1): dict(bytes_per_launch=922.5e6, algorithmic_bytes_per_launch=729.3e6, launches=312)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d.get("hbm_gbs"), bf16_tflops=d.get("bf16_tflops"),
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        sm = sorted(float(r[1]) for r in self.rows if len(r) > 2 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in self.rows if len(r) > 2 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# --------------------------------------------------------------------------------------------------
# CPU baseline: the oracle (restatement of the reference's CPU path) on a bounded sample
# --------------------------------------------------------------------------------------------------
def cpu_step_sample(name: str, sample_T: int, muon_layers: int = 1, warm: bool = True):
    """One bounded sample of a training step on the host cores: forward+reverse on one column of
    `sample_T` tokens, AdamW over every AdamW group, Muon over the matrices of `muon_layers`
    blocks (scaled to all blocks).  Returns tokens/s of a full step of B*T tokens per GPU."""
    import torch
    from oracle import femto_oracle as fo
    # all host cores, whatever the launcher exported (torchrun sets OMP_NUM_THREADS=1 for its workers)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    spec = CONFIGS[name]
    full = spec["cfg"]
    cfg = fo.GPTConfig(**{**full, "sequence_len": sample_T})
    lay = fo.parameter_layout(cfg)
    th = torch.zeros(lay.nparams, dtype=torch.float32)
    fo.initialize(th, cfg, lay, 123, all_nonzero=True)
    import femtochat_b200 as fb
    pk = fb.PackedBatches(full["vocab_size"], sample_T, 1, max_document_tokens=full["max_document_tokens"])
    tok, tgt, pos = (torch.from_numpy(x) for x in pk.next())
    M = fo.Model(cfg, fo.StepOptions(eps=fo.EPS_BF16, short_window=spec["short_window"], doc_mask=True))
    if warm:   # one untimed pass on a two-layer, 128-token copy of the model (thread pool and allocator start-up)
        wcfg = fo.GPTConfig(**{**full, "sequence_len": 128, "n_layer": 2})
        wlay = fo.parameter_layout(wcfg)
        wth = torch.zeros(wlay.nparams, dtype=torch.float32)
        fo.initialize(wth, wcfg, wlay, 1, all_nonzero=True)
        wpk = fb.PackedBatches(full["vocab_size"], 128, 1, max_document_tokens=full["max_document_tokens"])
        wtok, wtgt, wpos = (torch.from_numpy(x) for x in wpk.next())
        fo.Model(wcfg, fo.StepOptions(eps=fo.EPS_BF16, short_window=spec["short_window"], doc_mask=True)).loss_and_gradient(
            wth, wtok, wtgt, wpos)
    t0 = time.time()
    loss, delta, _ = M.loss_and_gradient(th, tok, tgt, pos)
    t_fb = time.time() - t0
    opt = fo.MuonAdamW(lay)
    t0 = time.time()
    for st in opt.adamw:
        sl = slice(st.spec.offset, st.spec.offset + st.spec.size)
        g = delta[sl]
        st.m.mul_(st.b1).add_((1 - st.b1) * g)
        st.v.mul_(st.b2).add_((1 - st.b2) * g * g)
        th[sl] = th[sl] * (1 - st.alpha * st.lam) - st.alpha * st.m / (torch.sqrt(st.v) + st.eps)
    t_adam = time.time() - t0
    blk = lay.blocks[0]
    t0 = time.time()
    for key in ("wq", "wk", "wv", "wo", "fc", "proj"):
        s = blk[key]
        G = fo.julia_stack(delta, [s])
        fo.polar_express(G)
    t_muon = (time.time() - t0) * cfg.n_layer / muon_layers
    tokens_full = spec["batch"] * full["sequence_len"]
    t_full = t_fb * tokens_full / sample_T + t_adam + t_muon
    return dict(tokens_per_s=tokens_full / t_full, t_fb=t_fb, t_adam=t_adam, t_muon=t_muon, loss=float(loss) / sample_T,
                cores=torch.get_num_threads(), measured_s=t_fb + t_adam + t_muon / cfg.n_layer * muon_layers,
                step_s_extrapolated=t_full,
                sample=(f"oracle fp32 on host: forward+reverse on 1 column of {sample_T} tokens ({t_fb:.1f}s, scaled to "
                        f"{tokens_full} tokens), AdamW on all groups ({t_adam:.1f}s), Polar Express on 1 of "
                        f"{cfg.n_layer} blocks ({t_muon / cfg.n_layer:.1f}s, scaled)"))


def run_reference(args):
    """`--impl reference`: the reference's own Julia CPU step cannot run (no Julia toolchain: unavailable
    on this box); the timed arm is the CPU restatement in oracle/ (kind "port") on every host core.  A full step
    (65 536 tokens at d20) takes minutes on a CPU, so ONE bounded sample is timed after one small warm-up pass:
    forward + reverse on one column of 1024 tokens, AdamW over all groups, Polar Express on one block, and the
    step time is extrapolated from it (the line says so and gives the seconds that were actually measured).
    --steps / --warmup are echoed, not multiplied into more samples.  Under torchrun only rank 0 works."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec = CONFIGS[args.config]
    c = cpu_step_sample(args.config, 1024)
    v = c["tokens_per_s"]
    tokens_full = spec["batch"] * spec["cfg"]["sequence_len"]
    line = dict(metric="training tokens/sec", value=v, unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1e3 * c["step_s_extrapolated"], higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic", impl="reference", extrapolated=True,
                measured_seconds=c["measured_s"],
                config=dict(workload=f"{args.config} GPT training step, B={spec['batch']} x T={spec['cfg']['sequence_len']} per GPU",
                            note="reference Julia CPU path unavailable on this box (no Julia); CPU restatement timed on one "
                                 "bounded sample, ms_per_step extrapolated to the full batch"),
                cpu_baseline=dict(value=v, unit="tokens/s", cores=c["cores"], kind="port", sample=c["sample"]),
                e2e=dict(value=v, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    import femtochat_b200 as fb
    from femtochat_b200 import _lib
    import ctypes as C

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    nccl_id = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf = C.create_string_buffer(128)
            _lib.check(_lib.lib().femto_nccl_unique_id(buf))
            idt.copy_(torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        nccl_id = bytes(idt.cpu().numpy().tobytes())

    spec = CONFIGS[args.config]
    B = args.batch or spec["batch"]
    micro = args.micro_steps or spec.get("micro_steps", 1)   # gradient-accumulation micro-steps per update
    cfg = fb.GPTConfig(**spec["cfg"])
    T = cfg.sequence_len
    lay = fb.parameter_layout(cfg)
    theta = torch.empty(lay.nparams, dtype=torch.float32, device="cuda")
    fb.initialize_(theta, lay, seed=123, all_nonzero=True)
    params = fb.Params(theta)
    st = fb.GradientState(cfg, max_batch=B, compute_type="bfloat16", short_window=spec["short_window"], doc_mask=True,
                          rank=rank, world=world, nccl_id=nccl_id)
    st.refresh_weights(params.theta)
    use_overlap = world > 1 and args.overlap   # reduce delta while the LAST micro-step's reverse pass runs
    opt = fb.MuonAdamW(params, lay, st, compute_type="bfloat16", weight_decay=0.01)
    if world > 1 and args.shard_optimizer:
        opt.shard(rank, world)   # each rank updates its share of Theta, then the shares are exchanged
        if args.exchange_weights:
            opt.set_exchange(1)  # ... as compute-type weights only; the fp32 Theta is completed on demand (below)
    total = args.steps + args.warmup
    pk = fb.PackedBatches(cfg.vocab_size, T, B, max_document_tokens=cfg.max_document_tokens, rank=rank)
    host = []
    for _ in range(total * micro):
        host.append(tuple(torch.from_numpy(x).pin_memory() for x in pk.next()))
    dev = [tuple(x.cuda() for x in h) for h in host]
    L = _lib.lib()
    sp = _lib.stream_ptr

    def sync_and_update(loss_dev, nv_dev, step):
        if world > 1:
            opt.grad_sync(loss_dev, nv_dev)   # femto_grad_sync, or its reduce-to-owner form under the sharded update
        sch = fb.training_schedule(step, 1000)
        opt.step(eta=sch["eta"], mu=sch["mu"], lam=sch["lam"] * 0.01, Nt=float(B * T * world * micro))

    # One update = `micro` micro-steps (scripts/train.jl:117-131: the first overwrites delta, the others add),
    # then ONE gradient sum and ONE optimiser step.
    def step_resident(i):
        for ms in range(micro):
            tok, tgt, pos = dev[i * micro + ms]
            if use_overlap:
                _lib.check(L.femto_set_overlap(st.h, 1 if ms == micro - 1 else 0))
            loss_dev, nv_dev = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos, reduction="sum", accumulate=ms > 0,
                                                     sync=False)
        sync_and_update(loss_dev, nv_dev, i)
        return loss_dev

    def step_e2e(i):
        for ms in range(micro):
            tok, tgt, pos = host[i * micro + ms]
            if use_overlap:
                _lib.check(L.femto_set_overlap(st.h, 1 if ms == micro - 1 else 0))
            loss, nv = fb.loss_and_gradient_host_(params, st, tok, tgt, pos, reduction="sum", accumulate=ms > 0)
        sync_and_update(st._loss, st._nvalid, i)
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    flops_tok = fb.estimate_flops(cfg, lay, short_window=spec["short_window"])

    # ---- resident-input timing: the headline `value` ----
    for i in range(args.warmup):
        step_resident(i)
    barrier()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    l0 = st.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    losses = []
    for i in range(args.warmup, total):
        losses.append(step_resident(i))
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = st.launch_count() - l0
    final_loss = float(losses[-1].item()) / (B * T * world)   # last micro-step's loss sum, all-reduced by femto_grad_sync
    clk = clocks.stop() if rank == 0 else None

    # ---- end to end: host buffers through the public call, H2D and D2H inside the timed region ----
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for i in range(args.warmup, total):
        step_e2e(i)
    e3.record()
    barrier()
    ms_e2e = e2.elapsed_time(e3)

    # ---- one profiled step: summed time and flops of the dominant kernel (tcgen05 GEMM) ----
    L.femto_profile_gemm(1)
    step_resident(total - 1)
    torch.cuda.synchronize()
    gms, gfl, gl = C.c_double(0), C.c_double(0), C.c_int32(0)
    L.femto_profile_gemm_report(C.byref(gms), C.byref(gfl), C.byref(gl))
    L.femto_profile_gemm(0)

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    status = st.status_word()
    # Theta must still be the same on every rank (the sharded update exchanges each rank's share)
    replicated = True
    if world > 1:
        if args.shard_optimizer and args.exchange_weights:
            opt.gather_theta()
        cs = torch.stack([params.theta.sum(dtype=torch.float64), params.theta.abs().sum(dtype=torch.float64)])
        hi, lo = cs.clone(), cs.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        replicated = bool((hi == lo).all().item())
    if rank == 0:
        tokens = B * T * world * micro * args.steps
        value = tokens / (ms / 1e3)
        peaks = measured_peaks()
        peak_tf = peaks["bf16_tflops_sustained"]
        ach = gfl.value / (gms.value / 1e3) / 1e12 if gms.value > 0 else 0.0
        line = dict(
            metric="training tokens/sec", value=value, unit="tokens/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
            ms_per_step=ms / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
            data="synthetic",
            config=dict(workload=f"{args.config} GPT training step (forward, reverse, grad sync, Muon+AdamW), "
                                 f"B={B} x T={T} per GPU{f' x {micro} micro-steps' if micro > 1 else ''}, short window {spec['short_window'] or 'reference rule'}, "
                                 f"document mask on",
                        parallelism=f"dp{world}",
                        optimizer=("owner-sharded" if world > 1 and args.shard_optimizer else "replicated"),
                        exchange=("compute-type weights per step, fp32 Theta on demand"
                                  if world > 1 and args.shard_optimizer and args.exchange_weights else "fp32 Theta per step"),
                        theta_replicated=replicated, l2="inputs and activations per step far exceed the 126 MB L2",
                        mfu_nominal_2p25e15=value * flops_tok / (world * 2.25e15), flops_per_token=flops_tok,
                        loss_per_token=final_loss, device_status=status),
            e2e=dict(value=tokens / (ms_e2e / 1e3), unit="tokens/s", h2d_bytes_per_step=3 * 4 * B * T * micro,
                     d2h_bytes_per_step=8 * micro),
            gpu_launches=int(launches),
            clocks=clk,
            roofline=dict(bound="tensor", achieved=ach, peak=peak_tf, unit="TFLOP/s", frac=ach / peak_tf if peak_tf else None,
                          traffic=(NCU_GEMM_TRAFFIC.get((args.config, B, micro)) or {}).get("bytes_per_launch"),
                          traffic_algorithmic=(NCU_GEMM_TRAFFIC.get((args.config, B, micro)) or {}).get("algorithmic_bytes_per_launch"),
                          traffic_source="ncu, one capture of the full-size step: profiles/gemm_tc_kernel_d20_step_dram.md",
                          kernel="gemm_tc_kernel", launches_per_step=gl.value,
                          kernel_ms_per_step=gms.value, peak_source=f"{peaks['source']} (sustained cuBLAS bf16)"),
        )
        if args.cpu_baseline and world == 1:   # the host baseline belongs to the one-GPU line only
            try:
                c = cpu_step_sample(args.config, 1024)
                line["cpu_baseline"] = dict(value=c["tokens_per_s"], unit="tokens/s", cores=c["cores"], kind="port",
                                            sample=c["sample"])
            except Exception as e:  # the GPU number stands even if the host baseline cannot run
                line["cpu_baseline"] = dict(value=None, unit="tokens/s", cores=None, kind="port", sample=f"failed: {e}")
        print(json.dumps(line), flush=True)
    if args.phases and world > 1:
        # Per-phase device times of the data-parallel step, with a barrier between the phases so that one rank's
        # wait for another is not booked to a collective: reverse pass | gradient sum | update (+ exchange), for
        # the owner-sharded and the replicated update on the same ranks.  Printed on stderr (stdout keeps its one line).
        tok, tgt, pos = dev[total - 1]
        for mode in ("owner-sharded", "replicated"):
            opt.shard(*((rank, world) if mode == "owner-sharded" else (0, 1)))
            acc = [0.0, 0.0, 0.0]
            for it in range(5):
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
                barrier()
                ev[0].record()
                loss_dev, nv_dev = fb.loss_and_gradient_(params, st, lay, tok, tgt, pos, reduction="sum", sync=False)
                ev[1].record()
                barrier()
                ev[2].record()
                opt.grad_sync(loss_dev, nv_dev)
                ev[3].record()
                barrier()
                ev[4].record()
                opt.step(eta=0.01, mu=0.95, lam=0.0, Nt=float(B * T * world))
                ev[5].record()
                torch.cuda.synchronize()
                if it >= 2:
                    for k in range(3):
                        acc[k] += ev[2 * k].elapsed_time(ev[2 * k + 1]) / 3
            t = torch.tensor(acc, dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if rank == 0:
                print(json.dumps(dict(phases=mode, n_gpus=world, forward_reverse_ms=float(t[0]),
                                      gradient_sum_ms=float(t[1]), update_ms=float(t[2]))), file=sys.stderr, flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="d20", choices=sorted(CONFIGS))
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--micro-steps", type=int, default=0,
                    help="gradient-accumulation micro-steps per update (default: the configuration's own, 2 for d26)")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--overlap", dest="overlap", action="store_true",
                    help="sum delta over ranks bucket by bucket during the reverse pass instead of after it "
                         "(measured equal or slightly slower on 2 and 8 B200: NCCL's CTAs only run between the "
                         "persistent GEMM launches)")
    ap.add_argument("--no-overlap", dest="overlap", action="store_false", help="the default")
    ap.add_argument("--replicated-optimizer", dest="shard_optimizer", action="store_false",
                    help="N > 1: every rank repeats the whole Muon/AdamW update instead of updating its share of "
                         "Theta and exchanging the shares (the default)")
    ap.add_argument("--exchange-theta", dest="exchange_weights", action="store_false",
                    help="N > 1, sharded update: exchange the fp32 Theta after every update instead of only the "
                         "compute-type weights (the default; Theta is then completed once, before it is read)")
    ap.add_argument("--phases", action="store_true",
                    help="N > 1: after the bench line, time reverse pass / gradient sum / update separately for the "
                         "owner-sharded and the replicated update (stderr)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        if int(os.environ.get("WORLD_SIZE", "1")) != args.gpus and args.gpus > 1:
            # launched without torchrun: re-launch one rank per GPU
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", "29511"] + sys.argv
            sys.exit(subprocess.call(cmd))
        run_ours(args)


if __name__ == "__main__":
    main()
