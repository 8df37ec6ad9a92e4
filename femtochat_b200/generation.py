"""Host mirror of src/generation.jl: top-k sampling around the model's logits, with the key/value cache the
reference leaves as a TODO (src/gpt.jl:81).  `generate` keeps the reference's signature and semantics: the prompt
is a list of 1-based token ids, each step samples from the logits of the last position, and at most
`sequence_len` tokens of context are used (src/generation.jl:40-46)."""
from __future__ import annotations

import ctypes as C

from . import _lib
from .gpt import GPT, _dev_i32


class KVCache:
    """Per-block keys and values of `max_batch` columns of up to `max_len` tokens (femto_kv_cache_*)."""

    def __init__(self, state, max_batch: int, max_len: int):
        c = C.c_void_p()
        _lib.check(_lib.lib().femto_kv_cache_create(state.h, max_batch, max_len, C.byref(c)))
        self.c, self.state, self.max_batch, self.max_len = c, state, max_batch, max_len

    def __len__(self):
        return int(_lib.lib().femto_kv_cache_length(self.c))

    def close(self):
        if self.c:
            _lib.lib().femto_kv_cache_destroy(self.c)
            self.c = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def prefill(model: GPT, cache: KVCache, tokens, positions=None):
    """Runs the prompt [B][Tp] and returns the soft-capped logits of each column's last position, fp32 [B][V]."""
    import torch
    tok, pos = _dev_i32(tokens), _dev_i32(positions)
    B, Tp = tok.shape
    st = cache.state
    st.refresh_weights(model.params.theta)
    out = torch.empty(B, model.config.vocab_size, device="cuda", dtype=torch.float32)
    _lib.check(_lib.lib().femto_prefill(st.h, cache.c, _lib.ptr(model.params.theta), _lib.ptr(tok), _lib.ptr(pos), B, Tp,
                                        _lib.ptr(out), _lib.stream_ptr()))
    return out


def decode_step(model: GPT, cache: KVCache, tokens, positions=None):
    """One new token per column ([B] ids): logits of the next position, fp32 [B][V]."""
    import torch
    tok, pos = _dev_i32(tokens), _dev_i32(positions)
    B = tok.shape[0]
    out = torch.empty(B, model.config.vocab_size, device="cuda", dtype=torch.float32)
    _lib.check(_lib.lib().femto_decode_step(cache.state.h, cache.c, _lib.ptr(model.params.theta), _lib.ptr(tok), _lib.ptr(pos), B,
                                            _lib.ptr(out), _lib.stream_ptr()))
    return out


def sample_token(generator, logits, temperature: float, top_k: int) -> int:
    """src/generation.jl:7-24 on a 1-D logits tensor; returns a 1-based token id."""
    import torch
    if temperature == 0:
        return int(torch.argmax(logits)) + 1
    k = min(top_k, logits.numel())
    scores, candidates = torch.topk(logits, k)          # descending, like partialsortperm(...; rev=true)
    scores = scores.double().cpu() / temperature
    weights = torch.exp(scores - scores.max())
    threshold = float(torch.rand((), generator=generator, dtype=torch.float64)) * float(weights.sum())
    cumulative = 0.0
    for token, weight in zip(candidates.tolist(), weights.tolist()):
        cumulative += weight
        if cumulative >= threshold:
            return token + 1
    return candidates[-1].item() + 1


def generate(model: GPT, prompt, max_new_tokens: int = 20, temperature: float = 0.8, top_k: int = 40, generator=None,
             use_cache: bool = True):
    """`generate(model, prompt; max_new_tokens, temperature, top_k, rng)` (src/generation.jl:26-56).  With
    use_cache=False every step recomputes the whole context through the model call, as the reference does; with
    the cache the prompt is run once and each new token costs one row.  Both give the same logits while the
    context fits in `sequence_len`; once it no longer does, the reference drops the oldest tokens, which changes
    every cached activation, so the cache is rebuilt from the slid context at that point."""
    import torch
    if len(prompt) == 0:
        raise ValueError("prompt must contain at least one token")
    if max_new_tokens < 0 or temperature < 0 or top_k <= 0:
        raise ValueError("max_new_tokens and temperature must be nonnegative, top_k positive")
    tokens = [int(t) for t in prompt]
    L = model.config.sequence_len
    cache = None
    for _ in range(max_new_tokens):
        first = max(0, len(tokens) - L)
        if use_cache and cache is not None and first == 0 and len(cache) == len(tokens) - 1:
            logits = decode_step(model, cache, torch.tensor([tokens[-1]], dtype=torch.int32))[0]
        else:
            ctx = torch.tensor([tokens[first:]], dtype=torch.int32)
            pos = torch.arange(first, len(tokens), dtype=torch.int32)[None, :]
            if use_cache:
                if cache is None:
                    cache = KVCache(model.state(1), 1, L)
                logits = prefill(model, cache, ctx, pos)[0]
            else:
                # the reference's way: the whole context through the forward pass, of which only the last row of
                # logits is kept (`[:, end, 1]`); the cache this run fills is thrown away
                scratch = KVCache(model.state(1), 1, L)
                logits = prefill(model, scratch, ctx, pos)[0]
                scratch.close()
        tokens.append(sample_token(generator, logits, temperature, top_k))
    if cache is not None:
        cache.close()
    return tokens
