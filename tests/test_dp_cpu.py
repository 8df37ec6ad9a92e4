"""Data-parallel semantics on CPU ranks (gloo, world_size 2): the batch is sharded by columns, delta,
loss sum and n_valid are summed over ranks, and every rank applies the same update with the global
token count.  Checked with the CPU oracle standing in for the per-rank step: the 2-rank result must
equal the 1-rank result on the concatenated batch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import femto_oracle as fo

CFG = dict(sequence_len=32, max_document_tokens=64, vocab_size=96, n_layer=2, n_head=4, n_kv_head=2, n_embed=64,
           window_pattern="SL")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _batch(B, seed):
    g = torch.Generator().manual_seed(seed)
    T, V = CFG["sequence_len"], CFG["vocab_size"]
    tok = torch.randint(1, V + 1, (B, T), generator=g, dtype=torch.int32)
    tgt = torch.randint(1, V + 1, (B, T), generator=g, dtype=torch.int32)
    tgt[0, 3] = -1
    pos = (torch.arange(T)[None, :].repeat(B, 1) % 17).int()
    return tok, tgt, pos


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    cfg = fo.GPTConfig(**CFG)
    lay = fo.parameter_layout(cfg)
    th = torch.zeros(lay.nparams, dtype=torch.float64)
    fo.initialize(th, cfg, lay, 7, all_nonzero=True)
    tok, tgt, pos = _batch(4, 1)
    per = 4 // world
    sl = slice(rank * per, (rank + 1) * per)                 # shard the batch columns
    M = fo.Model(cfg, fo.StepOptions(short_window=8))
    loss, delta, c = M.loss_and_gradient(th, tok[sl], tgt[sl], pos[sl])
    red = torch.tensor([loss, float(c["nvalid"])], dtype=torch.float64)
    delta = delta.double()
    dist.all_reduce(delta)                                   # what femto_grad_sync does with NCCL
    dist.all_reduce(red)
    opt = fo.MuonAdamW(lay, weight_decay=0.1)
    th32 = th.float()
    opt.step(th32, delta.float(), eta=0.7, mu=0.9, lam=0.05, Nt=float(red[1]))
    if rank == 0:
        torch.save(dict(delta=delta, loss=float(red[0]), nvalid=int(red[1]), theta=th32), out)
    # every rank must hold the same parameters after the update
    chk = th32.double().clone()
    dist.all_reduce(chk)
    assert float((chk / world - th32.double()).abs().max()) == 0.0
    dist.destroy_process_group()


def test_two_rank_step_equals_one_rank_on_the_concatenated_batch(tmp_path):
    out = str(tmp_path / "dp.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    cfg = fo.GPTConfig(**CFG)
    lay = fo.parameter_layout(cfg)
    th = torch.zeros(lay.nparams, dtype=torch.float64)
    fo.initialize(th, cfg, lay, 7, all_nonzero=True)
    tok, tgt, pos = _batch(4, 1)
    M = fo.Model(cfg, fo.StepOptions(short_window=8))
    loss, delta, c = M.loss_and_gradient(th, tok, tgt, pos)
    assert got["nvalid"] == c["nvalid"]                       # exact
    assert got["loss"] == pytest.approx(loss, rel=1e-12)
    assert float((got["delta"] - delta.double()).abs().max()) <= 1e-6 * float(delta.abs().max())
    opt = fo.MuonAdamW(lay, weight_decay=0.1)
    th32 = th.float()
    opt.step(th32, delta, eta=0.7, mu=0.9, lam=0.05, Nt=float(c["nvalid"]))
    assert float((got["theta"] - th32).abs().max()) <= 1e-5


def test_rank_streams_of_the_synthetic_loader_are_disjoint_and_reproducible():
    import femtochat_b200 as fb
    a0 = fb.PackedBatches(4096, 64, 2, rank=0).next()[0]
    a1 = fb.PackedBatches(4096, 64, 2, rank=1).next()[0]
    b0 = fb.PackedBatches(4096, 64, 2, rank=0).next()[0]
    assert (a0 == b0).all() and (a0 != a1).any()


SHARD_CFG = dict(sequence_len=16, max_document_tokens=64, vocab_size=256, n_layer=3, n_head=2, n_kv_head=1, n_embed=32,
                 window_pattern="SL")


def _shard_worker(rank, world, port, out):
    """The owner-sharded protocol with the oracle's optimiser standing in for the per-rank update: delta is summed
    onto the owner of each range only (all-reduced elsewhere), every rank updates, clears what it does not own (the
    replicated remainder counts as rank 0's) and one all-reduce rebuilds Theta."""
    import femtochat_b200 as fb
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    cfg = fo.GPTConfig(**SHARD_CFG)
    lay = fo.parameter_layout(cfg)
    plan = fb.shard_plan(lay, world, min_table=4096)
    th = torch.zeros(lay.nparams, dtype=torch.float64)
    fo.initialize(th, cfg, lay, 7, all_nonzero=True)
    th32 = th.float()
    g = torch.Generator().manual_seed(100 + rank)
    local = torch.randn(lay.nparams, generator=g)            # this rank's gradient
    owned = torch.zeros(lay.nparams, dtype=torch.bool)
    delta = local.clone()
    covered = torch.zeros(lay.nparams, dtype=torch.bool)
    for off, n, owner in plan:                                # reduce to the owner
        part = local[off:off + n].clone()
        dist.reduce(part, dst=owner)
        if owner == rank:
            delta[off:off + n] = part
            owned[off:off + n] = True
        covered[off:off + n] = True
    rest = local[~covered].clone()
    dist.all_reduce(rest)                                     # the replicated remainder
    delta[~covered] = rest
    if rank == 0:
        owned |= ~covered
    opt = fo.MuonAdamW(lay, weight_decay=0.1)
    opt.step(th32, delta, eta=0.7, mu=0.9, lam=0.05, Nt=64.0)
    th32[~owned] = 0.0                                        # clear the foreign ranges
    dist.all_reduce(th32)                                     # x + 0 + ... + 0 is exact
    full = local.clone()
    dist.all_reduce(full)
    if rank == 0:
        torch.save(dict(theta=th32, delta=full, plan=plan), out)
    chk = th32.double().clone()
    dist.all_reduce(chk)
    assert float((chk / world - th32.double()).abs().max()) == 0.0
    dist.destroy_process_group()


def test_owner_sharded_protocol_equals_the_replicated_update(tmp_path):
    out = str(tmp_path / "shard.pt")
    mp.spawn(_shard_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    cfg = fo.GPTConfig(**SHARD_CFG)
    lay = fo.parameter_layout(cfg)
    plan = got["plan"]
    assert {o for _, _, o in plan} == {0, 1}
    assert any(n == lay.lm_head.size // 2 for _, n, _ in plan)       # a sliced table
    th = torch.zeros(lay.nparams, dtype=torch.float64)
    fo.initialize(th, cfg, lay, 7, all_nonzero=True)
    th32 = th.float()
    opt = fo.MuonAdamW(lay, weight_decay=0.1)
    opt.step(th32, got["delta"], eta=0.7, mu=0.9, lam=0.05, Nt=64.0)
    assert torch.equal(got["theta"], th32)                            # bit for bit the replicated update


@pytest.mark.parametrize("world", [2, 3, 8])
def test_shard_plan_is_a_partition_of_the_large_tensors(world):
    import femtochat_b200 as fb
    cfg = fo.GPTConfig(sequence_len=64, max_document_tokens=64, vocab_size=8192, n_layer=6, n_head=2, n_kv_head=1,
                       n_embed=128, window_pattern="SL")
    lay = fo.parameter_layout(cfg)
    plan = fb.shard_plan(lay, world)
    assert fb.shard_plan(lay, 1) == []
    seen = torch.zeros(lay.nparams, dtype=torch.int32)
    for off, n, owner in plan:
        assert 0 <= owner < world
        seen[off:off + n] += 1
    assert int(seen.max()) == 1
    # matrices below 1024 elements (the value-embedding gates) stay replicated
    mats = sum(b[k].size for b in lay.blocks for k in ("wq", "wk", "wv", "wo", "fc", "proj", "ve_gate")
               if b[k] is not None and b[k].size >= 1024)
    tables = sum(sp.size for sp in (lay.lm_head, lay.embedding) if sp.size % (4 * world) == 0)   # 2^20 each; ve tables 2^19
    assert int(seen.sum()) == mats + tables
    # whole matrices, and the blocks of a rank are consecutive
    owner_of_block = []
    for i, b in enumerate(lay.blocks):
        owners = {o for off, n, o in plan if off <= b["wq"].offset < off + n}
        assert len(owners) == 1
        owner_of_block.append(owners.pop())
        for k in ("wq", "wk", "wv", "wo", "fc", "proj"):
            assert any(off <= b[k].offset and b[k].offset + b[k].size <= off + n and o == owner_of_block[-1] for off, n, o in plan)
    assert owner_of_block == sorted(owner_of_block) == [i * world // 6 for i in range(6)]
