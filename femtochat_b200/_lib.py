"""ctypes binding of libfemto_sm100a.so (the C ABI declared in include/femto.h).

The same signatures are what the Julia shim (julia/FemtoChatCUDAExt.jl) binds with ccall.
There is no fallback: if the library is missing or no CUDA device is present, calls fail.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfemto_sm100a.so")

F32, BF16 = 0, 1
REDUCTION = {"sum": 0, "mean": 1}


class FemtoConfig(C.Structure):
    _fields_ = [
        ("sequence_len", C.c_int32), ("max_document_tokens", C.c_int32), ("vocab_size", C.c_int32),
        ("n_layer", C.c_int32), ("n_head", C.c_int32), ("n_kv_head", C.c_int32), ("n_embed", C.c_int32),
        ("window_pattern", C.c_char * 32), ("short_window", C.c_int32), ("compute_dtype", C.c_int32),
        ("doc_mask", C.c_int32), ("index_base", C.c_int32), ("max_batch", C.c_int32),
        ("pad_vocab_size_to", C.c_int32),
    ]


class TensorDesc(C.Structure):
    _fields_ = [("kind", C.c_int32), ("layer", C.c_int32), ("offset", C.c_int64), ("rows", C.c_int64),
                ("cols", C.c_int64)]


class Segment(C.Structure):
    _fields_ = [("src", C.c_int64), ("col", C.c_int32), ("row", C.c_int32), ("n", C.c_int32), ("pos0", C.c_int32),
                ("next", C.c_int32), ("reserved", C.c_int32)]


class OptimizerConfig(C.Structure):
    _fields_ = [
        ("unembedding_lr", C.c_float), ("embedding_lr", C.c_float), ("matrix_lr", C.c_float),
        ("weight_decay", C.c_float), ("scalar_lr", C.c_float), ("smear_lr", C.c_float),
        ("ns_steps", C.c_int32), ("ns_coeffs", C.c_float * 15), ("compute_dtype", C.c_int32),
    ]


class FemtoError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"libfemto error {code}: {msg}")
        self.code = code


_lib = None

P, I32, I64, F = C.c_void_p, C.c_int32, C.c_int64, C.c_float

# name -> (restype, argtypes); every name must be exported by the library (checked in tests)
SIGNATURES = {
    "femto_version": (I32, []),
    "femto_last_error": (C.c_char_p, [P]),
    "femto_nparams": (I64, [C.POINTER(FemtoConfig)]),
    "femto_layout": (I32, [C.POINTER(FemtoConfig), C.POINTER(TensorDesc), I32]),
    "femto_window_sizes": (I32, [C.POINTER(FemtoConfig), C.POINTER(I32), C.POINTER(I32)]),
    "femto_nccl_unique_id": (I32, [P]),
    "femto_create": (I32, [C.POINTER(FemtoConfig), I32, I32, P, C.POINTER(P)]),
    "femto_destroy": (I32, [P]),
    "femto_refresh_weights": (I32, [P, P, P]),
    "femto_loss_and_gradient": (I32, [P, P, P, P, P, P, I32, I32, I32, P, P, P]),
    "femto_forward_loss": (I32, [P, P, P, P, P, I32, I32, P, P, P]),
    "femto_forward_logits": (I32, [P, P, P, P, I32, P, P]),
    "femto_forward_token_losses": (I32, [P, P, P, P, P, I32, P, P, P]),
    "femto_loss_and_gradient_host": (I32, [P, P, P, P, P, P, I32, I32, I32, C.POINTER(F), C.POINTER(I32), P]),
    "femto_kv_cache_create": (I32, [P, I32, I32, C.POINTER(P)]),
    "femto_kv_cache_destroy": (I32, [P]),
    "femto_kv_cache_length": (I32, [P]),
    "femto_prefill": (I32, [P, P, P, P, P, I32, I32, P, P]),
    "femto_decode_step": (I32, [P, P, P, P, P, I32, P, P]),
    "femto_pack_batch": (I32, [P, I64, P, I32, I32, I32, I32, I32, P, P, P, P, P]),
    "femto_feeder_create": (I32, [I32, I32, I32, C.POINTER(P)]),
    "femto_feeder_destroy": (I32, [P]),
    "femto_feeder_submit": (I32, [P, P, P, P]),
    "femto_feeder_next": (I32, [P, P, C.POINTER(P), C.POINTER(P), C.POINTER(P)]),
    "femto_feeder_release": (I32, [P, P]),
    "femto_grad_sync": (I32, [P, P, P, P, P]),
    "femto_comm_check": (I32, [P]),
    "femto_comm_abort": (I32, [P]),
    "femto_selftest_bounded_wait": (I32, [I32, C.POINTER(I32), C.POINTER(I32)]),
    "femto_set_overlap": (I32, [P, I32]),
    "femto_optimizer_state_sizes": (I32, [P, C.POINTER(I64)]),
    "femto_optimizer_create": (I32, [P, C.POINTER(OptimizerConfig), P, P, P, P, C.POINTER(P)]),
    "femto_optimizer_destroy": (I32, [P]),
    "femto_optimizer_step": (I32, [P, P, P, F, I32, F, I32, F, F, P]),
    "femto_optimizer_set_shard": (I32, [P, I32, I32]),
    "femto_optimizer_set_exchange": (I32, [P, I32]),
    "femto_optimizer_gather_theta": (I32, [P, P, P]),
    "femto_optimizer_grad_sync": (I32, [P, P, P, P, P]),
    "femto_optimizer_state_ranges": (I32, [P, I32, C.POINTER(I64), I32]),
    "femto_optimizer_gather_state": (I32, [P, P]),
    "femto_optimizer_shard_ranges": (I32, [P, C.POINTER(I64), I32]),
    "femto_optimizer_get_t": (I32, [P, C.POINTER(I32), I32]),
    "femto_optimizer_set_t": (I32, [P, C.POINTER(I32), I32]),
    "femto_attention_fwd": (I32, [I32, P, P, P, P, P, P, P, I32, I32, I32, I32, I32, I32, P, P]),
    "femto_attention_bwd": (I32, [I32, P, P, P, P, P, P, P, P, P, P, P, I32, I32, I32, I32, I32, I32, P, I32, P]),
    "femto_attention_bwd_static": (I32, [I32, P, P, P, P, P, P, P, P, P, I32, I32, I32, I32, I32, I32, P, P]),
    "femto_gemm_bf16": (I32, [P, I32, I64, P, I32, I64, P, I64, I32, I32, I32, I32, I64, I64, I64, I32, I32, P]),
    "femto_gemm_pair_mode": (I32, [I32]),
    "femto_embedding_gradient": (I32, [I32, P, P, P, I32, I32, I32, P]),
    "femto_xent_fused": (I32, [I32, P, P, I64, P, I32, I32, I32, F, P, P, P, P, P]),
    "femto_newton_schulz": (I32, [I32, P, I32, I32, I32, C.POINTER(F), I32, P]),
    "femto_cross_entropy": (I32, [P, I64, P, I32, I32, I32, P, P, P]),
    "femto_cross_entropy_gradient": (I32, [P, I64, P, I64, P, I32, I32, I32, F, P, P]),
    "femto_adamw": (I32, [P, P, P, P, I64, F, F, F, F, F, I32, F, P]),
    "femto_rmsnorm_fwd": (I32, [I32, P, P, P, I32, I32, F, P]),
    "femto_rmsnorm_bwd": (I32, [I32, P, P, P, P, I32, I32, P]),
    "femto_embed_gather": (I32, [I32, P, P, P, I32, I32, I32, P]),
    "femto_muon_direction": (I32, [I32, P, P, P, P, I32, I32, I32, F, F, F, C.POINTER(F), I32, P]),
    "femto_status_word": (I32, [P, C.POINTER(I32)]),
    "femto_sync": (I32, [P, P]),
    "femto_launch_count": (I64, [P]),
    "femto_profile_gemm": (I32, [I32]),
    "femto_profile_gemm_report": (I32, [C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(I32)]),
}


def lib():
    """Loads the shared library (no compute happens on load)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FemtoError(-1, f"{LIB_PATH} is not built; run `python -m femtochat_b200.build`")
        L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(code: int) -> int:
    if code != 0:
        msg = lib().femto_last_error(None)
        raise FemtoError(code, msg.decode("utf-8", "replace") if msg else "")
    return code


def ptr(t):
    """Device (or pinned host) pointer of a torch tensor, None -> NULL."""
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)
