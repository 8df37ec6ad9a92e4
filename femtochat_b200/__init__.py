"""femtochat_b200: host mirror of femtochat's GPT training-step API over libfemto_sm100a.so."""
from .parameters import GPTConfig, Layout, Params, ParamSpec, has_ve, parameter_layout, paramview, window_sizes
from .gpt import GPT, GradientState, gradient_state, initialize_, loss_and_gradient_, loss_and_gradient_host_
from .optim import MuonAdamW, POLAR_EXPRESS_COEFFS, QUINTIC_COEFFS, shard_plan
from .scaling import (estimate_flops, num_matmul_params, num_scaling_params, training_scaling, training_schedule,
                      PEAK_FLOPS_B200, PEAK_BANDWIDTH_B200)
from .data import PackedBatches, DevicePackedBatches, Feeder, bos_token_id
from .checkpoints import optimizer_state, restore_optimizer_, save_checkpoint, load_checkpoint
from .generation import KVCache, prefill, decode_step, generate, sample_token
