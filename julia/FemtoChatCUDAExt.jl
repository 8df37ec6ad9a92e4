# Replacement for femtochat's ext/FemtoChatCUDAExt.jl: every method the reference's CUDA extension and
# its gradient drivers provide for CuArray-backed `Params` becomes one `ccall` into libfemto_sm100a.so.
# No Enzyme, Reactant, Triton or CPU fallback is involved on this path.  (Not executed in this
# repository's tests: the build machines have no Julia toolchain; the same C ABI is exercised from
# Python ctypes, see femtochat_b200/_lib.py, and tests/test_host.py checks every ccall signature in
# this file against include/femto.h.)
module FemtoChatCUDAExt

using CUDA
using FemtoChat
using FemtoChat.Parameters: Params, GPTConfig
using FemtoChat.Optimizer: AdamW, Muon, ParameterUpdate, MuonGroup
import FemtoChat: loss_and_gradient!, gradient_state
import FemtoChat.Kernels: attention!, Δattention!, embedding_gradient!
import FemtoChat.Optimizer: MuonAdamW, batched_mul!, gather!, scatter!

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

# Mirrors `femto_optimizer_config`.
struct FemtoOptimizerConfig
    unembedding_lr::Float32; embedding_lr::Float32; matrix_lr::Float32
    weight_decay::Float32; scalar_lr::Float32; smear_lr::Float32
    ns_steps::Int32
    ns_coeffs::NTuple{15,Float32}
    compute_dtype::Int32
end

# The reference's five Polar-Express triples (src/optim.jl:90-96).
const POLAR_EXPRESS = (8.156554524902461f0, -22.48329292557795f0, 15.878769915207462f0,
                       4.042929935166739f0, -2.808917465908714f0, 0.5000178451051316f0,
                       3.8916678022926607f0, -2.772484153217685f0, 0.5060648178503393f0,
                       3.285753657755655f0, -2.3681294933425376f0, 0.46449024233003106f0,
                       2.3465413258596377f0, -1.7097828382687081f0, 0.42323551169305323f0)

check(code) = code == 0 ? nothing :
    error("libfemto error $code: " * unsafe_string(ccall((:femto_last_error, libfemto), Cstring, (Ptr{Cvoid},), C_NULL)))

dtype_code(::Type{Float32}) = Int32(0)
dtype_code(::Type) = Int32(1)          # BFloat16

mutable struct FemtoGradientState
    handle::Ptr{Cvoid}
    loss::CuArray{Float32,1}
    nvalid::CuArray{Int32,1}
    optimizer_owns_weights::Bool       # a bound MuonAdamW refreshes the compute-type weights after every update
end

# The optimiser is built from (params, layout) alone (src/optim.jl:318), so it finds the library handle of the
# parameters through this table, filled by gradient_state.
const STATES = IdDict{Any,FemtoGradientState}()

# gradient_state(params, config, layout, tokens, targets; positions)   (src/FemtoChat.jl:30)
function gradient_state(params::Params{Float32,<:CuArray}, config::GPTConfig, layout, tokens, targets;
                        positions=nothing, compute_type=Float32, short_window=0, doc_mask=false)
    cfg = Ref(FemtoConfig(config; compute_type, short_window, doc_mask, max_batch=size(tokens, 2)))
    h = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:femto_create, libfemto), Int32, (Ref{FemtoConfig}, Int32, Int32, Ptr{Cvoid}, Ref{Ptr{Cvoid}}),
                cfg, 0, 1, C_NULL, h))
    state = FemtoGradientState(h[], CUDA.zeros(Float32, 1), CUDA.zeros(Int32, 1), false)
    finalizer(s -> ccall((:femto_destroy, libfemto), Int32, (Ptr{Cvoid},), s.handle), state)
    refresh_weights!(state, params)
    STATES[params.Θ] = state
    state
end

# The library keeps a compute-type copy of the weights.  Whoever writes Θ outside the library (manual SGD as in
# README.md:74-83, a checkpoint load) must call this before the next loss_and_gradient!.
refresh_weights!(state::FemtoGradientState, params::Params) =
    check(ccall((:femto_refresh_weights, libfemto), Int32, (Ptr{Cvoid}, CuPtr{Float32}, Ptr{Cvoid}),
                state.handle, params.Θ, stream().handle))

# loss_and_gradient!(params, state, layout, tokens, targets; positions)   (src/FemtoChat.jl:29)
# tokens/targets/positions are (T, B) Int32 CuArrays == the library's [B][T] row-major arrays.  The reference's
# drivers differentiate the model call's default reduction, the mean (ext/FemtoChatEnzymeExt.jl:15,38-44;
# src/gpt.jl:196); the training script asks for the sum (scripts/train.jl:118) and adds the micro-steps up
# (`accumulate`, scripts/train.jl:121-128).  Unless a MuonAdamW built by this extension owns the weights, Θ may have
# been changed by the caller since the last call, so the compute-type copy is rebuilt first.
function loss_and_gradient!(params::Params, state::FemtoGradientState, layout, tokens, targets;
                            positions=nothing, reduction=:mean, accumulate=false)
    state.optimizer_owns_weights || refresh_weights!(state, params)
    pos = isnothing(positions) ? CU_NULL : pointer(positions)
    check(ccall((:femto_loss_and_gradient, libfemto), Int32,
                (Ptr{Cvoid}, CuPtr{Float32}, CuPtr{Float32}, CuPtr{Int32}, CuPtr{Int32}, CuPtr{Int32}, Int32, Int32,
                 Int32, CuPtr{Float32}, CuPtr{Int32}, Ptr{Cvoid}),
                state.handle, params.Θ, params.δ, tokens, targets, pos, size(tokens, 2),
                reduction == :mean ? 1 : 0, accumulate ? 1 : 0, state.loss, state.nvalid, stream().handle))
    Array(state.loss)[1]
end

# 🤖(...)(tokens, targets; positions, reduction)   (src/gpt.jl:196-199), forward only
function forward_loss(params::Params, state::FemtoGradientState, tokens, targets; positions=nothing, reduction=:mean)
    state.optimizer_owns_weights || refresh_weights!(state, params)
    pos = isnothing(positions) ? CU_NULL : pointer(positions)
    if reduction == :none
        losses = CUDA.zeros(Float32, size(tokens, 1), size(tokens, 2))
        check(ccall((:femto_forward_token_losses, libfemto), Int32,
                    (Ptr{Cvoid}, CuPtr{Float32}, CuPtr{Int32}, CuPtr{Int32}, CuPtr{Int32}, Int32, CuPtr{Float32},
                     CuPtr{Int32}, Ptr{Cvoid}),
                    state.handle, params.Θ, tokens, targets, pos, size(tokens, 2), losses, state.nvalid, stream().handle))
        return losses
    end
    check(ccall((:femto_forward_loss, libfemto), Int32,
                (Ptr{Cvoid}, CuPtr{Float32}, CuPtr{Int32}, CuPtr{Int32}, CuPtr{Int32}, Int32, Int32, CuPtr{Float32},
                 CuPtr{Int32}, Ptr{Cvoid}),
                state.handle, params.Θ, tokens, targets, pos, size(tokens, 2), reduction == :mean ? 1 : 0, state.loss,
                state.nvalid, stream().handle))
    Array(state.loss)[1]
end

# logits = model(tokens; positions)   (src/gpt.jl:129-170): (V, T, B) Float32, soft-capped, first vocab_size rows
function forward_logits(params::Params, state::FemtoGradientState, config, tokens; positions=nothing)
    state.optimizer_owns_weights || refresh_weights!(state, params)
    pos = isnothing(positions) ? CU_NULL : pointer(positions)
    logits = CUDA.zeros(Float32, config.vocab_size, size(tokens, 1), size(tokens, 2))
    check(ccall((:femto_forward_logits, libfemto), Int32,
                (Ptr{Cvoid}, CuPtr{Float32}, CuPtr{Int32}, CuPtr{Int32}, Int32, CuPtr{Float32}, Ptr{Cvoid}),
                state.handle, params.Θ, tokens, pos, size(tokens, 2), logits, stream().handle))
    logits
end

# ── MuonAdamW (src/optim.jl:318-440) ────────────────────────────────────────────────────────────
# The update runs in the library; the persistent state stays in Julia-owned CuArrays.  The groups are the
# reference's own `ParameterUpdate(AdamW …)` / `MuonGroup(ParameterUpdate(Muon …))` objects whose 𝓂ₜ / 𝓋ₜ are views
# into four flat buffers laid out in the reference's group order, so `optimizer_state(ω)` and
# `restore_optimizer!(ω, saved)` (src/checkpoints.jl:9-24) work on this optimiser unchanged.
mutable struct FemtoMuonAdamW{A,M}
    adamw::A
    muon::M
    handle::Ptr{Cvoid}
    params::Params
    state::FemtoGradientState
    buffers::NTuple{4,CuArray{Float32,1}}     # adam 𝓂ₜ, adam 𝓋ₜ, muon 𝓂ₜ, muon 𝓋ₜ
end

function MuonAdamW(params::Params{Float32,<:CuArray}, layout; unembedding_lr=0.004f0, embedding_lr=0.2f0,
                   matrix_lr=0.02f0, weight_decay=0f0, scalar_lr=0.5f0, smear_lr=0.2f0, compute_type=Float32, t=0,
                   state::FemtoGradientState=get(STATES, params.Θ) do
                       error("call gradient_state(params, config, layout, tokens, targets) before MuonAdamW(params, layout)")
                   end)
    sizes = zeros(Int64, 4)
    check(ccall((:femto_optimizer_state_sizes, libfemto), Int32, (Ptr{Cvoid}, Ptr{Int64}), state.handle, sizes))
    buffers = ntuple(i -> CUDA.zeros(Float32, sizes[i]), 4)
    cfg = Ref(FemtoOptimizerConfig(unembedding_lr, embedding_lr, matrix_lr, weight_decay, scalar_lr, smear_lr, 5,
                                   POLAR_EXPRESS, dtype_code(compute_type)))
    o = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:femto_optimizer_create, libfemto), Int32,
                (Ptr{Cvoid}, Ref{FemtoOptimizerConfig}, CuPtr{Float32}, CuPtr{Float32}, CuPtr{Float32}, CuPtr{Float32},
                 Ref{Ptr{Cvoid}}),
                state.handle, cfg, buffers[1], buffers[2], buffers[3], buffers[4], o))
    # Group views in the reference's order: AdamW groups as src/optim.jl:333-403, Muon groups by shape in order of
    # first appearance (:405-425).  Hyper-parameters on these structs are informative; the library holds its own.
    (; embedding, blocks) = layout.transformer
    D = embedding.shape[1]
    scale = √(768f0 / D)
    specs = Any[(layout.lm_head, unembedding_lr * scale, 0.8f0, 0.96f0, 0.01f0),
                (embedding, embedding_lr * scale, 0.8f0, 0.995f0, 0.001f0)]
    for block in blocks
        isnothing(block.🍰.𝔼) || push!(specs, (block.🍰.𝔼, 0.5f0 * embedding_lr * scale, 0.8f0, 0.995f0, 0.01f0))
        push!(specs, (block.λᵦ, 0.01f0 * scalar_lr, 0.8f0, 0.95f0, 0.05f0))
        push!(specs, (block.λx₀, Float32(scalar_lr), 0.96f0, 0.95f0, 0f0))
    end
    for spec in (layout.smear_gate, layout.λₛ, layout.λᵧ)
        push!(specs, (spec, Float32(smear_lr), 0.8f0, 0.95f0, 0f0))
    end
    adamw, at = Any[], 0
    for (spec, α, β₁, β₂, λ) in specs
        n = length(spec.range)
        ω = AdamW(α, β₁, β₂, view(buffers[1], at+1:at+n), view(buffers[2], at+1:at+n), t, 1f-10, λ)
        push!(adamw, ParameterUpdate(ω, view(params.Θ, spec.range), view(params.δ, spec.range), first(spec.range) - 1))
        at += n
    end
    muon_specs = Any[]
    for block in blocks
        (; 👀, 🧠) = block
        append!(muon_specs, (👀.𝕎, 👀.𝕂, 👀.𝕍, 👀.ℙ, 🧠.𝔽, 🧠.ℙ))
        isnothing(👀.𝕧𝕖) || push!(muon_specs, 👀.𝕧𝕖)
    end
    muon, mo, vo = Any[], 0, 0
    for shape in unique(spec.shape for spec in muon_specs)
        group = filter(spec -> spec.shape == shape, muon_specs)
        (m, n), k = shape, length(group)
        𝓂ₜ = reshape(view(buffers[3], mo+1:mo+m*n*k), m, n, k)
        vshape = m ≥ n ? (m, 1, k) : (1, n, k)
        𝓋ₜ = reshape(view(buffers[4], vo+1:vo+prod(vshape)), vshape)
        ω = Muon(Float32(matrix_lr), 0.95f0, 0.9f0, Float32(weight_decay), 5, 𝓂ₜ, 𝓋ₜ, nothing)
        offsets = CuArray([first(spec.range) - 1 for spec in group])
        push!(muon, MuonGroup(ParameterUpdate(ω, nothing, nothing), params, offsets))
        mo += m * n * k
        vo += prod(vshape)
    end
    optimizer = FemtoMuonAdamW(Tuple(adamw), Tuple(muon), o[], params, state, buffers)
    state.optimizer_owns_weights = true
    finalizer(ω -> ccall((:femto_optimizer_destroy, libfemto), Int32, (Ptr{Cvoid},), ω.handle), optimizer)
    optimizer
end

# ω(; η, μ, λ, Nₜ)   (src/optim.jl:430-440).  The AdamW step counters live on the Julia structs (restore_optimizer!
# writes them, src/checkpoints.jl:18), so they are handed to the library before the update and advanced after it.
function (ω::FemtoMuonAdamW)(; η=1f0, μ=nothing, λ=nothing, Nₜ=1f0)
    ts = Int32[u.ω.t for u in ω.adamw]
    check(ccall((:femto_optimizer_set_t, libfemto), Int32, (Ptr{Cvoid}, Ptr{Int32}, Int32), ω.handle, ts, length(ts)))
    check(ccall((:femto_optimizer_step, libfemto), Int32,
                (Ptr{Cvoid}, CuPtr{Float32}, CuPtr{Float32}, Float32, Int32, Float32, Int32, Float32, Float32, Ptr{Cvoid}),
                ω.handle, ω.params.Θ, ω.params.δ, η, isnothing(μ) ? 0 : 1, isnothing(μ) ? 0f0 : μ,
                isnothing(λ) ? 0 : 1, isnothing(λ) ? 0f0 : λ, Nₜ, stream().handle))
    for u in ω.adamw
        u.ω.t += 1
    end
    nothing
end

# ── kernel-level seams ───────────────────────────────────────────────────────────────────────
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
                dtype_code(T), O, ℓ, m, CU_NULL, Q, K, V, B, Tn, H, size(K, 2), D, first(window), CU_NULL,
                stream().handle))
    O
end

# Δattention!(𝒜, dQ, dK, dV, dO, Q, K, V, O, ℓ, m, window; accumulate=true)   (ext/FemtoChatCUDAExt.jl:1771-1776):
# the saved statistics are the row sum ℓ and the row max m; the gradients are added to unless accumulate=false.
function Δattention!(_, dQ::CuArray{T,4}, dK::CuArray{T,4}, dV::CuArray{T,4}, dO::CuArray{T,4}, Q::CuArray{T,4},
                     K::CuArray{T,4}, V::CuArray{T,4}, O::CuArray{T,4}, ℓ::CuArray{Float32,4}, m::CuArray{Float32,4},
                     window::Tuple{Int,Int}; accumulate::Bool=true, kwargs...) where {T}
    D, H, Tn, B = size(Q)
    check(ccall((:femto_attention_bwd, libfemto), Int32,
                (Int32, CuPtr{T}, CuPtr{T}, CuPtr{T}, CuPtr{T}, CuPtr{T}, CuPtr{T}, CuPtr{T}, CuPtr{T}, CuPtr{Float32},
                 CuPtr{Float32}, CuPtr{Float32}, Int32, Int32, Int32, Int32, Int32, Int32, CuPtr{Int32}, Int32, Ptr{Cvoid}),
                dtype_code(T), dQ, dK, dV, dO, Q, K, V, O, CU_NULL, ℓ, m, B, Tn, H, size(K, 2), D, first(window), CU_NULL,
                accumulate ? 1 : 0, stream().handle))
    nothing
end

# embedding_gradient!(δ, dy, tokens)   (src/kernels.jl:8-14); tokens are 1-based in Julia.
function embedding_gradient!(δ::CuArray{Float32,2}, dy::CuArray{T}, tokens::CuArray) where {T}
    tok0 = Int32.(tokens) .- Int32(1)
    check(ccall((:femto_embedding_gradient, libfemto), Int32,
                (Int32, CuPtr{Float32}, CuPtr{T}, CuPtr{Int32}, Int32, Int32, Int32, Ptr{Cvoid}),
                dtype_code(T), δ, dy, tok0, length(tokens), size(δ, 1), size(δ, 2), stream().handle))
    nothing
end

# Embedding call 𝔼[:, tokens]   (src/gpt.jl:34; the reference's GPU kernel ext/FemtoChatCUDAExt.jl:63-75)
function embedding_gather!(y::CuArray{T}, 𝔼::CuArray{T,2}, tokens::CuArray) where {T}
    tok0 = Int32.(tokens) .- Int32(1)
    check(ccall((:femto_embed_gather, libfemto), Int32,
                (Int32, CuPtr{T}, CuPtr{T}, CuPtr{Int32}, Int32, Int32, Int32, Ptr{Cvoid}),
                dtype_code(T), y, 𝔼, tok0, length(tokens), size(𝔼, 1), size(𝔼, 2), stream().handle))
    y
end

# norm (src/gpt.jl:16-20) over dim 1 and its reverse (ext/FemtoChatMooncakeExt.jl:248-255)
function norm!(y::CuArray{T}, r::CuArray{Float32}, x::CuArray{T}) where {T}
    D = size(x, 1)
    check(ccall((:femto_rmsnorm_fwd, libfemto), Int32,
                (Int32, CuPtr{T}, CuPtr{T}, CuPtr{Float32}, Int32, Int32, Float32, Ptr{Cvoid}),
                dtype_code(T), x, y, r, length(x) ÷ D, D, Float32(eps(T)), stream().handle))
    y
end
function Δnorm!(dx::CuArray{T}, dy::CuArray{T}, y::CuArray{T}, r::CuArray{Float32}) where {T}
    D = size(y, 1)
    check(ccall((:femto_rmsnorm_bwd, libfemto), Int32,
                (Int32, CuPtr{T}, CuPtr{T}, CuPtr{Float32}, CuPtr{T}, Int32, Int32, Ptr{Cvoid}),
                dtype_code(T), dy, y, r, dx, length(y) ÷ D, D, stream().handle))
    dx
end

# batched_mul!(C, A, B, transpose_A, transpose_B)   (ext/FemtoChatCUDAExt.jl:121-125; src/optim.jl:123).
# Column-major C = op(A) op(B) is the row-major product Cᵀ = op(B)ᵀ op(A)ᵀ: Julia's B becomes the library's
# left operand and A its right one; a Julia (p, q, k) array is the row-major stack [k][q][p].
function batched_mul!(C::CuArray{T,3}, A::CuArray{T,3}, B::CuArray{T,3}, transpose_A=false, transpose_B=false) where {T<:Core.BFloat16}
    m, n, k = size(C)
    p = transpose_A ? size(A, 1) : size(A, 2)
    check(ccall((:femto_gemm_bf16, libfemto), Int32,
                (CuPtr{T}, Int32, Int64, CuPtr{T}, Int32, Int64, CuPtr{T}, Int64, Int32, Int32, Int32, Int32, Int64, Int64,
                 Int64, Int32, Int32, Ptr{Cvoid}),
                B, transpose_B ? 0 : 1, size(B, 1), A, transpose_A ? 1 : 0, size(A, 1), C, m, n, m, p, k,
                size(B, 1) * size(B, 2), size(A, 1) * size(A, 2), m * n, 0, 0, stream().handle))
    C
end

# polar_express! (src/optim.jl:131-149) on a stack, and the whole muon_direction! (src/optim.jl:198-236)
function polar_express!(X::CuArray{T,3}, coefficients=POLAR_EXPRESS) where {T}
    m, n, k = size(X)
    c = Float32[coefficients...]
    check(ccall((:femto_newton_schulz, libfemto), Int32,
                (Int32, CuPtr{T}, Int32, Int32, Int32, Ptr{Float32}, Int32, Ptr{Cvoid}),
                dtype_code(T), X, k, n, m, c, length(c) ÷ 3, stream().handle))
    X
end
function muon_direction!(X::CuArray{Float32,3}, G::CuArray{Float32,3}, 𝓂ₜ::CuArray{Float32,3}, 𝓋ₜ::CuArray{Float32,3};
                         μ=0.95f0, β₂=0.9f0, Nₜ=1f0, compute_type=Float32)
    m, n, k = size(G)
    c = Float32[POLAR_EXPRESS...]
    check(ccall((:femto_muon_direction, libfemto), Int32,
                (Int32, CuPtr{Float32}, CuPtr{Float32}, CuPtr{Float32}, CuPtr{Float32}, Int32, Int32, Int32, Float32,
                 Float32, Float32, Ptr{Float32}, Int32, Ptr{Cvoid}),
                dtype_code(compute_type), X, G, 𝓂ₜ, 𝓋ₜ, k, n, m, μ, β₂, Nₜ, c, 5, stream().handle))
    X
end

# gather! / scatter! (ext/FemtoChatCUDAExt.jl:141-149): flat Θ/δ ↔ stacked (m, n, k).  The library's optimiser reads
# the matrices where they lie, so these exist only for callers of the reference's own MuonGroup; they are plain
# device-to-device copies, one per matrix.
function gather!(stack::CuArray, vector::CuArray, offsets::CuArray)
    width = size(stack, 1) * size(stack, 2)
    for (k, off) in enumerate(Array(offsets))
        copyto!(stack, (k - 1) * width + 1, vector, off + 1, width)
    end
    stack
end
function scatter!(vector::CuArray, stack::CuArray, offsets::CuArray)
    width = size(stack, 1) * size(stack, 2)
    for (k, off) in enumerate(Array(offsets))
        copyto!(vector, off + 1, stack, (k - 1) * width + 1, width)
    end
    vector
end

# AdamW on one flat range (src/optim.jl:75-87)
function adamw!(θ::CuArray{Float32}, δ::CuArray{Float32}, ω::AdamW; α=ω.α, Nₜ=1f0)
    ω.t += 1
    check(ccall((:femto_adamw, libfemto), Int32,
                (CuPtr{Float32}, CuPtr{Float32}, CuPtr{Float32}, CuPtr{Float32}, Int64, Float32, Float32, Float32, Float32,
                 Float32, Int32, Float32, Ptr{Cvoid}),
                θ, δ, ω.𝓂ₜ, ω.𝓋ₜ, length(θ), α, ω.β₁, ω.β₂, ω.ϵ, ω.λ, ω.t, Nₜ, stream().handle))
    nothing
end

# ReactantCUDACall.check() (ext/reactant/cuda_call.jl:94-97): surface a deferred device-side error
function check_device(state::FemtoGradientState)
    word = Ref{Int32}(0)
    check(ccall((:femto_status_word, libfemto), Int32, (Ptr{Cvoid}, Ref{Int32}), state.handle, word))
    word[] == 0 || error("libfemto device status word $(word[]) (1 = token id out of range, 2 = a bounded wait ran out)")
    nothing
end

end
