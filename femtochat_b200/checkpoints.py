"""Host mirror of src/checkpoints.jl: the optimiser's persistent state in the reference's per-group layout, and
write-then-rename checkpoint files.

`optimizer_state(ω)` returns what the reference serialises (src/checkpoints.jl:9-12):

    adamw = [(m, v, t), ...]   one entry per AdamW group in the order of src/optim.jl:333-403
    muon  = [(m, v), ...]      one entry per Muon shape group (src/optim.jl:405-425); m is the Julia (rows, cols, k)
                               array, i.e. the row-major [k][cols][rows] tensor, v is (rows,1,k) or (1,cols,k)

as CPU tensors, so a checkpoint written here restores into a reference optimiser with the same groups and the other
way round.  Under the owner-sharded data-parallel update the moments of a range are current only on its owner:
`optimizer_state` first completes them on every rank (femto_optimizer_gather_state), as a checkpoint is written by
rank 0 alone (src/checkpoints.jl:27-28)."""
from __future__ import annotations

import os

from .optim import MuonAdamW


def optimizer_state(opt: MuonAdamW, gather: bool = True):
    """src/checkpoints.jl:9-12."""
    import torch
    if gather:
        opt.gather_state()
        torch.cuda.synchronize()
    ts = opt.get_t()
    return dict(
        adamw=[dict(m=g.m.detach().cpu().clone(), v=g.v.detach().cpu().clone(), t=int(ts[i])) for i, g in enumerate(opt.adamw)],
        muon=[dict(m=g.m.detach().cpu().clone(), v=g.v.detach().cpu().clone()) for g in opt.muon],
    )


def restore_optimizer_(opt: MuonAdamW, saved) -> None:
    """src/checkpoints.jl:14-25: copies the saved moments into the optimiser's own buffers and restores the AdamW
    step counters."""
    if len(saved["adamw"]) != len(opt.adamw) or len(saved["muon"]) != len(opt.muon):
        raise ValueError("checkpoint has different optimiser groups")
    for g, s in zip(opt.adamw, saved["adamw"]):
        if g.m.numel() != s["m"].numel():
            raise ValueError("AdamW group size differs from the checkpoint")
        g.m.copy_(s["m"].reshape(g.m.shape))
        g.v.copy_(s["v"].reshape(g.v.shape))
    for g, s in zip(opt.muon, saved["muon"]):
        if g.m.numel() != s["m"].numel() or g.v.numel() != s["v"].numel():
            raise ValueError("Muon group shape differs from the checkpoint")
        g.m.copy_(s["m"].reshape(g.m.shape))
        g.v.copy_(s["v"].reshape(g.v.shape))
    opt.set_t([int(s["t"]) for s in saved["adamw"]])


def save_checkpoint(path: str, step: int, params, optimizer: MuonAdamW, metadata, rank: int = 0):
    """src/checkpoints.jl:27-36: rank 0 writes `checkpoint_%06d` under `path`, first to a `.part` file that is then
    renamed, so an interrupted write leaves the previous checkpoint intact.  Every rank must call it (the sharded
    optimiser state is gathered with a collective); only rank 0 touches the file system."""
    import torch
    state = optimizer_state(optimizer)
    if rank != 0:
        return None
    os.makedirs(path, exist_ok=True)
    file = os.path.join(path, "checkpoint_%06d.pt" % step)
    torch.save(dict(version=1, step=step, parameters=params.theta.detach().cpu(), optimizer=state, metadata=metadata),
               file + ".part")
    os.replace(file + ".part", file)
    return file


def load_checkpoint(path: str, step: int = None):
    """src/checkpoints.jl:38-39."""
    import torch
    file = path if step is None else os.path.join(path, "checkpoint_%06d.pt" % step)
    return torch.load(file, weights_only=False)
