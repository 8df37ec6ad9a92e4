"""Host-side scalars of src/scaling.jl: parameter counts, the FLOP model behind MFU, schedules."""
from __future__ import annotations

import math

from .parameters import GPTConfig, Layout, parameter_layout, window_sizes

PEAK_FLOPS_B200 = 2.25e15      # src/common.jl:39
PEAK_BANDWIDTH_B200 = 8.0e12   # src/common.jl:88


def num_scaling_params(layout: Layout):
    """src/scaling.jl:7-28."""
    n = lambda s: 0 if s is None else s.size
    ve = sum(n(b["ve_table"]) for b in layout.blocks)
    mats = sum(n(b[k]) for b in layout.blocks for k in ("wq", "wk", "wv", "wo", "ve_gate", "fc", "proj"))
    scalars = layout.smear_gate.size + layout.lam_s.size + layout.lam_y.size + 2 * len(layout.blocks)
    wte, lm = layout.embedding.size, layout.lm_head.size
    return dict(wte=wte, value_embeds=ve, lm_head=lm, transformer_matrices=mats, scalars=scalars,
                total=wte + ve + lm + mats + scalars)


def num_matmul_params(layout: Layout) -> int:
    """src/scaling.jl:30-33."""
    c = num_scaling_params(layout)
    return c["transformer_matrices"] + c["lm_head"] + layout.smear_gate.size


def estimate_flops(config: GPTConfig, layout: Layout = None, short_window: int = 0) -> int:
    """src/scaling.jl:33-43."""
    layout = layout or parameter_layout(config)
    t = config.sequence_len
    att = sum(12 * config.n_embed * (t if w < 0 else min(w, t)) for w, _ in window_sizes(config, short_window))
    return 6 * num_matmul_params(layout) + att


def training_scaling(config: GPTConfig, total_batch_size=None, target_param_data_ratio=12, weight_decay=0.28):
    """src/scaling.jl:46-56."""
    counts = num_scaling_params(parameter_layout(config))
    ref = num_scaling_params(parameter_layout(GPTConfig(vocab_size=config.vocab_size)))
    D = math.floor(target_param_data_ratio * (counts["transformer_matrices"] + counts["lm_head"]))
    Dr = target_param_data_ratio * (ref["transformer_matrices"] + ref["lm_head"])
    Br = 2 ** 19
    B = 2 ** round(math.log2(Br * (D / Dr) ** 0.383)) if total_batch_size is None else total_batch_size
    eta = math.sqrt(B / Br)
    lam = weight_decay * eta * Dr / D
    return dict(total_batch_size=B, target_tokens=D, eta=eta, lam=lam)


def training_schedule(step: int, steps: int, warmup_steps=40, warmdown_ratio=0.65, final_lr_frac=0.05):
    """src/scaling.jl:59-78; `step` counts completed updates from zero."""
    warmdown = round(warmdown_ratio * steps)
    start = steps - warmdown
    if step < warmup_steps:
        eta = (step + 1) / warmup_steps
    elif step <= start:
        eta = 1.0
    else:
        p = (steps - step) / warmdown
        eta = p + (1 - p) * final_lr_frac
    if step < 400:
        mu = 0.85 + (0.97 - 0.85) * step / 400
    elif step >= start and warmdown > 0:
        mu = 0.97 + (0.90 - 0.97) * (step - start) / warmdown
    else:
        mu = 0.97
    return dict(eta=eta, mu=mu, lam=(1 + math.cos(math.pi * step / steps)) / 2)
