# Replacement for femtochat's ext/FemtoChatCUDAExt.jl: every method the reference's CUDA extension and
# its gradient drivers provide for CuArray-backed `Params` becomes one `ccall` into libfemto_sm100a.so.
# No Enzyme, Reactant, Triton or CPU fallback is involved on this path.  (Not executed in this
# repository's tests: the build machines have no Julia toolchain; the same C ABI is exercised from
# Python ctypes, see femtochat_b200/_lib.py.)
module FemtoChatCUDAExt

using CUDA
using FemtoChat
using FemtoChat.Parameters: Params, GPTConfig
import FemtoChat: loss_and_gradient!, gradient_state
import FemtoChat.Kernels: attention!, Δattention!, embedding_gradient!

const libfemto = get(ENV, "LIBFEMTO_SM100A", "libfemto_sm100a.so")

# Mirrors `femto_config` of include/femto.h field for field.
struct FemtoConfig
    sequence_len::Int32; max_document_tokens::Int32; vocab_size::Int32; n_layer::Int32
    n_head::Int32; n_kv_head::Int32; n_embed::Int32
    window_pattern::NTuple{32,UInt8}
    short_window::Int32; compute_dtype::Int32; doc_mask::Int32; index_base::Int32
    max_batch::Int32; pad_vocab_size_to::Int32
end

function FemtoConfig(c::GPTConfig; compute_type=Float32, short_window=0, doc_mask=false, max_batch=1)
    pat = ntuple(i -> i <= ncodeunits(c.window_pattern) ? codeunit(c.window_pattern, i) : 0x00, 32)
    FemtoConfig(c.sequence_len, c.max_document_tokens, c.vocab_size, c.n_layer, c.n_head, c.n_kv_head,
                c.n_embed, pat, short_window, compute_type == Float32 ? 0 : 1, doc_mask ? 1 : 0, 1, max_batch, 64)
end

check(code) = code == 0 ? nothing :
    error("libfemto error $code: " * unsafe_string(ccall((:femto_last_error, libfemto), Cstring, (Ptr{Cvoid},), C_NULL)))

mutable struct FemtoGradientState
    handle::Ptr{Cvoid}
    loss::CuArray{Float32,1}
    nvalid::CuArray{Int32,1}
end

# gradient_state(params, config, layout, tokens, targets; positions)   (src/FemtoChat.jl:30)
function gradient_state(params::Params{Float32,<:CuArray}, config::GPTConfig, layout, tokens, targets;
                        positions=nothing, compute_type=Float32, short_window=0, doc_mask=false)
    cfg = Ref(FemtoConfig(config; compute_type, short_window, doc_mask, max_batch=size(tokens, 2)))
    h = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:femto_create, libfemto), Int32, (Ref{FemtoConfig}, Int32, Int32, Ptr{Cvoid}, Ref{Ptr{Cvoid}}),
                cfg, 0, 1, C_NULL, h))
    state = FemtoGradientState(h[], CUDA.zeros(Float32, 1), CUDA.zeros(Int32, 1))
    finalizer(s -> ccall((:femto_destroy, libfemto), Int32, (Ptr{Cvoid},), s.handle), state)
    check(ccall((:femto_refresh_weights, libfemto), Int32, (Ptr{Cvoid}, CuPtr{Float32}, Ptr{Cvoid}),
                state.handle, params.Θ, stream().handle))
    state
end

# loss_and_gradient!(params, state, layout, tokens, targets; positions)   (src/FemtoChat.jl:29)
# tokens/targets/positions are (T, B) Int32 CuArrays == the library's [B][T] row-major arrays.
function loss_and_gradient!(params::Params, state::FemtoGradientState, layout, tokens, targets;
                            positions=nothing, reduction=:sum, accumulate=false)
    pos = isnothing(positions) ? CU_NULL : pointer(positions)
    check(ccall((:femto_loss_and_gradient, libfemto), Int32,
                (Ptr{Cvoid}, CuPtr{Float32}, CuPtr{Float32}, CuPtr{Int32}, CuPtr{Int32}, CuPtr{Int32}, Int32, Int32,
                 Int32, CuPtr{Float32}, CuPtr{Int32}, Ptr{Cvoid}),
                state.handle, params.Θ, params.δ, tokens, targets, pos, size(tokens, 2),
                reduction == :mean ? 1 : 0, accumulate ? 1 : 0, state.loss, state.nvalid, stream().handle))
    Array(state.loss)[1]
end

# logits = model(tokens; positions)   (src/gpt.jl:129-170): (V, T, B) Float32, soft-capped, first vocab_size rows
function forward_logits(params::Params, state::FemtoGradientState, config, tokens; positions=nothing)
    pos = isnothing(positions) ? CU_NULL : pointer(positions)
    logits = CUDA.zeros(Float32, config.vocab_size, size(tokens, 1), size(tokens, 2))
    check(ccall((:femto_forward_logits, libfemto), Int32,
                (Ptr{Cvoid}, CuPtr{Float32}, CuPtr{Int32}, CuPtr{Int32}, Int32, CuPtr{Float32}, Ptr{Cvoid}),
                state.handle, params.Θ, tokens, pos, size(tokens, 2), logits, stream().handle))
    logits
end

# cross_entropy(logits, targets, ignore, reduction) on a (V, T, B) Float32 CuArray   (src/gpt.jl:175-193)
function cross_entropy(logits::CuArray{Float32,3}, targets::CuArray, ignore, reduction)
    V, Tn, B = size(logits)
    tg0 = Int32.(ifelse.(targets .== ignore, Int32(-1), targets .- Int32(1)))
    red = reduction == :sum ? 0 : reduction == :mean ? 1 : 2
    out = CUDA.zeros(Float32, red == 2 ? Tn * B : 1)
    check(ccall((:femto_cross_entropy, libfemto), Int32,
                (CuPtr{Float32}, Int64, CuPtr{Int32}, Int32, Int32, Int32, CuPtr{Float32}, CuPtr{Int32}, Ptr{Cvoid}),
                logits, V, tg0, Tn * B, V, red, out, CU_NULL, stream().handle))
    red == 2 ? reshape(out, Tn, B) : Array(out)[1]
end

# cross_entropy_gradient!(δ, logits, targets, dy, ignore, reduction)   (src/kernels.jl:16-28)
function cross_entropy_gradient!(δ::CuArray{Float32}, logits::CuArray{Float32,3}, targets::CuArray, dy, ignore, reduction)
    V, Tn, B = size(logits)
    tg0 = Int32.(ifelse.(targets .== ignore, Int32(-1), targets .- Int32(1)))
    red = reduction == :sum ? 0 : reduction == :mean ? 1 : 2
    rows = red == 2 ? pointer(CuArray{Float32}(vec(dy))) : CU_NULL
    check(ccall((:femto_cross_entropy_gradient, libfemto), Int32,
                (CuPtr{Float32}, Int64, CuPtr{Float32}, Int64, CuPtr{Int32}, Int32, Int32, Int32, Float32, CuPtr{Float32}, Ptr{Cvoid}),
                δ, V, logits, V, tg0, Tn * B, V, red, red == 2 ? 0f0 : Float32(dy), rows, stream().handle))
    nothing
end

# attention!(𝒜, O, ℓ, m, Q, K, V, window)   (ext/FemtoChatCUDAExt.jl:1242 of the reference)
function attention!(_, O::CuArray{T,4}, ℓ, m, Q, K, V, window) where {T}
    D, H, Tn, B = size(Q)
    check(ccall((:femto_attention_fwd, libfemto), Int32,
                (Int32, CuPtr{T}, CuPtr{Float32}, CuPtr{Float32}, CuPtr{Float32}, CuPtr{T}, CuPtr{T}, CuPtr{T}, Int32,
                 Int32, Int32, Int32, Int32, Int32, CuPtr{Int32}, Ptr{Cvoid}),
                T == Float32 ? 0 : 1, O, ℓ, m, CU_NULL, Q, K, V, B, Tn, H, size(K, 2), D, first(window), CU_NULL,
                stream().handle))
    O
end

# embedding_gradient!(δ, dy, tokens)   (src/kernels.jl:8-14); tokens are 1-based in Julia.
function embedding_gradient!(δ::CuArray{Float32,2}, dy::CuArray{T}, tokens::CuArray) where {T}
    tok0 = Int32.(tokens) .- Int32(1)
    check(ccall((:femto_embedding_gradient, libfemto), Int32,
                (Int32, CuPtr{Float32}, CuPtr{T}, CuPtr{Int32}, Int32, Int32, Int32, Ptr{Cvoid}),
                T == Float32 ? 0 : 1, δ, dy, tok0, length(tokens), size(δ, 1), size(δ, 2), stream().handle))
    nothing
end

end
