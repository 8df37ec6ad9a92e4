/* libfemto_sm100a — C ABI of the B200-native femtochat GPT training step.
 *
 * Every entry point returns int32: 0 = ok, negative = argument/shape/alignment/state error
 * detected on the host before any launch, positive = CUDA / NCCL error code or a device status
 * word.  Nothing throws, exits or aborts (the reference never lets an exception cross a C frame
 * either: ext/reactant/cuda_call.jl:37-50, deps/reactant/xla_ffi.cpp:21-23).  The text of the last
 * error is available through femto_last_error().
 *
 * Pointers are DEVICE pointers unless the name starts with h_.  The library borrows caller buffers
 * for the duration of a call; it owns only its workspace arena (allocated once in femto_create) and
 * its NCCL communicator.  Launch-type calls are asynchronous on the given stream.
 *
 * Layout rule: the reference's column-major Julia arrays are byte-identical to the row-major arrays
 * named here: Julia (d,T,B) == [B][T][d]; a Julia weight (out,in) == [in][out]; (1,T,H,B) == [B][H][T].
 * Token and target ids are 1-based and the ignore target is -1 (src/gpt.jl:34,172), positions are
 * 0-based (src/gpt.jl:45), unless index_base says otherwise.
 */
#ifndef FEMTO_H
#define FEMTO_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define FEMTO_OK 0
#define FEMTO_ERR_ARG (-1)
#define FEMTO_ERR_SHAPE (-2)
#define FEMTO_ERR_ALIGN (-3)
#define FEMTO_ERR_STATE (-4)
#define FEMTO_ERR_UNSUPPORTED (-5)
#define FEMTO_ERR_NOMEM (-6)
#define FEMTO_ERR_DEVICE_STATUS 100000 /* + device status word */

#define FEMTO_F32 0
#define FEMTO_BF16 1

#define FEMTO_REDUCTION_SUM 0  /* reduction=:sum, the training script's call (scripts/train.jl:118) */
#define FEMTO_REDUCTION_MEAN 1 /* reduction=:mean, the default of the model call (src/gpt.jl:196) */
#define FEMTO_REDUCTION_NONE 2 /* reduction=:none, per-token losses (stand-alone cross-entropy entry points only) */

/* Mirrors GPTConfig (src/parameters.jl:71-80) plus the build options the reference passes as
 * keyword arguments (compute_type, src/parameters.jl:451) and the four switches on which the
 * benchmark configurations differ from the reference's defaults. */
typedef struct femto_config {
  int32_t sequence_len;
  int32_t max_document_tokens;
  int32_t vocab_size;
  int32_t n_layer;
  int32_t n_head;
  int32_t n_kv_head;
  int32_t n_embed;
  char window_pattern[32]; /* NUL-terminated, 'S' / 'L' */
  int32_t short_window;    /* 0 = reference rule min(L, cld(L,512)*128) (src/parameters.jl:204) */
  int32_t compute_dtype;   /* FEMTO_F32 | FEMTO_BF16: activations and matrix multiplies */
  int32_t doc_mask;        /* 0 = reference (attention crosses documents); 1 = keys >= document start */
  int32_t index_base;      /* 1 = reference (1-based tokens/targets); 0 = zero-based wire format */
  int32_t max_batch;       /* largest B (columns of sequence_len tokens) a call may pass */
  int32_t pad_vocab_size_to; /* 64 in the reference (src/parameters.jl:221) */
} femto_config;

typedef struct femto_handle femto_handle;

/* One row of the flat layout (src/parameters.jl:219-337).  `rows`,`cols` are the Julia shape. */
typedef struct femto_tensor_desc {
  int32_t kind;  /* 0 wte, 1 wq, 2 wk, 3 wv, 4 wo, 5 ve_gate, 6 fc, 7 proj, 8 ve_table, 9 lam_b, 10 lam_x0,
                    11 lm_head, 12 smear_gate, 13 lam_s, 14 lam_y */
  int32_t layer; /* 0-based block index, -1 for global tensors */
  int64_t offset; /* 0-based element offset into Theta / delta */
  int64_t rows, cols;
} femto_tensor_desc;

/* ---- lifetime ------------------------------------------------------------------------------- */
/* Replaces gradient_state (ext/FemtoChatEnzymeExt.jl:27-36): builds the per-shape state once.
 * rank/world describe the data-parallel job; h_nccl_id is the 128-byte ncclUniqueId shared by all
 * ranks (NULL when world == 1). */
int32_t femto_create(const femto_config* h_cfg, int32_t rank, int32_t world, const void* h_nccl_id,
                     femto_handle** h_out);
int32_t femto_destroy(femto_handle* h);
const char* femto_last_error(femto_handle* h); /* h may be NULL: last error of a failed femto_create */
int32_t femto_version(void);
/* Fills the 128-byte ncclUniqueId on the calling rank (rank 0 shares it with the others). */
int32_t femto_nccl_unique_id(void* h_id128);

/* ---- layout (parameter_layout, src/parameters.jl:219-337) ------------------------------------ */
int64_t femto_nparams(const femto_config* h_cfg);
/* Writes up to `capacity` descriptors in flat order; returns the number of tensors (or <0). */
int32_t femto_layout(const femto_config* h_cfg, femto_tensor_desc* h_out, int32_t capacity);
/* window_sizes (src/parameters.jl:200-210): left window per layer; has_ve (:197-198) as 0/1. */
int32_t femto_window_sizes(const femto_config* h_cfg, int32_t* h_left, int32_t* h_has_ve);

/* ---- model ---------------------------------------------------------------------------------- */
/* Rebuilds the compute-type copy of the weights from Theta (fp32).  The reference casts the fp32
 * master weights on every Linear call (src/gpt.jl:27); here the cast happens once per update.
 * Call after any external write to Theta; femto_optimizer_step does it itself. */
int32_t femto_refresh_weights(femto_handle* h, const float* theta, void* stream);

/* loss_and_gradient! (ext/FemtoChatEnzymeExt.jl:38-44) with the training script's accumulation
 * (scripts/train.jl:117-131): delta = (accumulate ? delta : 0) + d loss / d Theta.
 * tokens/targets/positions are int32 [B][T] device arrays (positions may be NULL = 0..T-1).
 * loss_out (float) and n_valid_out (int32) are device scalars written on the stream. */
int32_t femto_loss_and_gradient(femto_handle* h, const float* theta, float* delta, const int32_t* tokens,
                                const int32_t* targets, const int32_t* positions, int32_t B,
                                int32_t reduction, int32_t accumulate, float* loss_out,
                                int32_t* n_valid_out, void* stream);
/* The model call without the reverse pass (src/gpt.jl:196-199). */
int32_t femto_forward_loss(femto_handle* h, const float* theta, const int32_t* tokens,
                           const int32_t* targets, const int32_t* positions, int32_t B, int32_t reduction,
                           float* loss_out, int32_t* n_valid_out, void* stream);
/* The model call without targets (src/gpt.jl:129-170, `logits = omega(tokens; positions)`): writes the
 * soft-capped logits z = 15 tanh(x W / 15) of the first vocab_size rows as fp32 [B][T][vocab_size]
 * (the reference's (V,T,B) array).  Meant for small evaluation shapes: the output is B*T*V floats. */
int32_t femto_forward_logits(femto_handle* h, const float* theta, const int32_t* tokens,
                             const int32_t* positions, int32_t B, float* logits_out, void* stream);
/* The model call with reduction=:none (src/gpt.jl:191-193), what the reference's evaluation loop uses
 * (src/loss_eval.jl:8-46): fp32 losses [B][T], zero where the target is ignored. */
int32_t femto_forward_token_losses(femto_handle* h, const float* theta, const int32_t* tokens,
                                   const int32_t* targets, const int32_t* positions, int32_t B,
                                   float* losses_out, int32_t* n_valid_out, void* stream);
/* Host-buffer convenience used by the end-to-end path: copies the three int32 [B][T] host arrays to
 * the device, runs femto_loss_and_gradient, reads loss and n_valid back and synchronises. */
int32_t femto_loss_and_gradient_host(femto_handle* h, const float* theta, float* delta,
                                     const int32_t* h_tokens, const int32_t* h_targets,
                                     const int32_t* h_positions, int32_t B, int32_t reduction,
                                     int32_t accumulate, float* h_loss, int32_t* h_n_valid, void* stream);

/* ---- generation with a key/value cache (src/generation.jl:26-56) ----------------------------- */
/* The reference's `generate` runs the whole context through the model for every new token (the cache is a TODO
 * at src/gpt.jl:81).  Here femto_prefill runs the prompt once and keeps every block's keys and values;
 * femto_decode_step then costs one row per column.  Logits are what `model(input; positions)[:, end, b]`
 * returns: fp32 [B][vocab_size], soft-capped.  Sampling (temperature, top-k, src/generation.jl:7-24) stays on
 * the host.  Valid while prompt + generated tokens <= max_len; the reference's sliding of the context window
 * beyond sequence_len is a fresh femto_prefill of the slid context. */
typedef struct femto_kv_cache femto_kv_cache;
int32_t femto_kv_cache_create(femto_handle* h, int32_t max_batch, int32_t max_len, femto_kv_cache** h_out);
int32_t femto_kv_cache_destroy(femto_kv_cache* c);
int32_t femto_kv_cache_length(femto_kv_cache* c); /* tokens cached per column */
/* tokens / positions: int32 [B][Tp] device arrays (positions NULL = 0..Tp-1); resets the cache to this prompt. */
int32_t femto_prefill(femto_handle* h, femto_kv_cache* c, const float* theta, const int32_t* tokens,
                      const int32_t* positions, int32_t B, int32_t Tp, float* logits_out, void* stream);
/* tokens: int32 [B], one new token per column; positions: int32 [B] or NULL (= each column's last position + 1). */
int32_t femto_decode_step(femto_handle* h, femto_kv_cache* c, const float* theta, const int32_t* tokens,
                          const int32_t* positions, int32_t B, float* logits_out, void* stream);

/* ---- batch producer (src/dataloader.jl:241-274; scripts/train.jl:144-145) ---------------------- */
/* One run of a document inside a batch column: rows row..row+n-1 of column col take the tokens
 * stream[src..src+n-1]; positions count up from pos0; the target of the last row is `next` (0-based id of the
 * document's next token when it continues in the following batch, BOS when it ends here, -1 for none). */
typedef struct femto_segment {
  int64_t src;
  int32_t col, row, n, pos0, next, reserved;
} femto_segment;
/* model_batch! (src/dataloader.jl:241-274) on the device: builds the three int32 [B][T] arrays of a packed batch
 * from a token stream that already lies in device memory as 0-based 16-bit ids (documents back to back, each
 * starting with BOS) and a list of segments (device array; the O(#documents) assignment of documents to columns
 * stays on the host).  Rows no segment covers are padding: token BOS, target -1, position 0 (:243-245).  Ids are
 * written with `index_base` added (1 = the reference's 1-based ids).  A segment that leaves the batch or the
 * stream is skipped and raises bit 1 of *status (device word, may be NULL).  Asynchronous. */
int32_t femto_pack_batch(const uint16_t* stream0, int64_t n_stream, const femto_segment* segments,
                         int32_t n_segments, int32_t B, int32_t T, int32_t bos0, int32_t index_base,
                         int32_t* tokens, int32_t* targets, int32_t* positions, uint32_t* status, void* stream);
/* Pinned, multi-buffered feeder for hosts that build batches on the CPU (the reference's producer task and
 * Channel(2), scripts/train.jl:88-100,144-145): femto_feeder_submit copies the three host arrays into a pinned
 * slot and queues the host-to-device copy on the feeder's own stream; femto_feeder_next makes `compute_stream` wait
 * for the oldest submitted batch and returns its device arrays (positions NULL if none were submitted);
 * femto_feeder_release, called once the work that reads them has been queued, lets the slot be refilled (the next
 * femto_feeder_next does it implicitly).  With depth >= 2 the copy of batch i+1 overlaps the step on batch i.
 * No counterpart as a function in the reference, where the copy is a blocking to_rarray inside the loop. */
typedef struct femto_feeder femto_feeder;
int32_t femto_feeder_create(int32_t B, int32_t T, int32_t depth, femto_feeder** h_out);
int32_t femto_feeder_destroy(femto_feeder* f);
int32_t femto_feeder_submit(femto_feeder* f, const int32_t* h_tokens, const int32_t* h_targets,
                            const int32_t* h_positions);
int32_t femto_feeder_next(femto_feeder* f, void* compute_stream, const int32_t** d_tokens,
                          const int32_t** d_targets, const int32_t** d_positions);
int32_t femto_feeder_release(femto_feeder* f, void* compute_stream);

/* ---- data parallel (new; the reference is single-GPU, scripts/train.jl:13) ------------------- */
/* Sums delta, loss and n_valid over ranks (in place).  No-op when world == 1. */
int32_t femto_grad_sync(femto_handle* h, float* delta, float* loss_inout, int32_t* n_valid_inout,
                        void* stream);

/* Health of the handle's communicator between steps: 0 while every collective enqueued so far succeeded or is still
 * running, otherwise 200000 + the NCCL result (a peer died, a link fault).  Collectives report errors only when
 * they are enqueued, so a training loop polls this (with its own wall-clock limit) and, on an error or a timeout,
 * calls femto_comm_abort, which tears the communicator down without waiting; data-parallel calls then return
 * FEMTO_ERR_STATE instead of blocking.  The reference has no counterpart (single process, single GPU). */
int32_t femto_comm_check(femto_handle* h);
int32_t femto_comm_abort(femto_handle* h);

/* When enabled (world > 1), femto_loss_and_gradient sums each finished range of delta over ranks on a
 * communication stream while the rest of the reverse pass runs; femto_grad_sync then only waits for
 * those reductions.  Enable it for the LAST micro-step of an update only: earlier micro-steps must
 * leave delta local (scripts/train.jl:117-131 accumulates before the single update). */
int32_t femto_set_overlap(femto_handle* h, int32_t enable);

/* ---- optimiser: MuonAdamW (src/optim.jl:318-440) ---------------------------------------------- */
typedef struct femto_optimizer_config {
  float unembedding_lr, embedding_lr, matrix_lr, weight_decay, scalar_lr, smear_lr; /* :321-326 */
  int32_t ns_steps;       /* 5 (:421) */
  float ns_coeffs[15];    /* 5 x (a,b,c): the reference's rho_t table (:90-96) unless overridden */
  int32_t compute_dtype;  /* dtype of the Polar-Express chain (:327): FEMTO_F32 | FEMTO_BF16 */
} femto_optimizer_config;
typedef struct femto_optimizer femto_optimizer;

/* Sizes (in floats) of the four caller-owned state buffers, in the reference's group order:
 * adam moments m,v over all AdamW groups (:333-403), Muon momentum over all Muon groups (:412-425)
 * and the NorMuon second moments. h_out[0..3] = adam_m, adam_v (equal), muon_m, muon_v. */
int32_t femto_optimizer_state_sizes(femto_handle* h, int64_t* h_out4);
int32_t femto_optimizer_create(femto_handle* h, const femto_optimizer_config* h_cfg, float* adam_m,
                               float* adam_v, float* muon_m, float* muon_v, femto_optimizer** h_out);
int32_t femto_optimizer_destroy(femto_optimizer* o);
/* One update `ω(; η, μ, λ, Nₜ)` (:430-440): has_mu/has_lambda == 0 keeps the groups' own values.
 * Reads delta, updates Theta and the moments, then refreshes the compute-type weights. */
int32_t femto_optimizer_step(femto_optimizer* o, float* theta, const float* delta, float eta, int32_t has_mu,
                             float mu, int32_t has_lambda, float lambda, float n_tokens, void* stream);
/* Owner-sharded update for data parallelism (no counterpart in the reference, which is single-GPU:
 * scripts/train.jl:13).  After femto_grad_sync every rank holds the same delta, so rank `rank` of `world`
 * updates only slice `rank` of every large AdamW table (:333-390) and the Muon matrices (:405-425) of the
 * blocks [rank L / world, (rank+1) L / world) (the tiny value-embedding gates excepted: every rank updates
 * those); femto_optimizer_step then exchanges the new values over the
 * handle's communicator (each rank clears what it does not own, then one all-reduce of Theta), so Theta stays
 * replicated.
 * Small AdamW groups (scalars, gates) stay replicated.  The moments of ranges a rank does not own are not
 * advanced on that rank.  world == 1 restores the full update.  On a handle without a communicator the
 * exchange is skipped and the caller merges the ranges itself (femto_optimizer_shard_ranges). */
int32_t femto_optimizer_set_shard(femto_optimizer* o, int32_t rank, int32_t world);
/* What the sharded femto_optimizer_step exchanges.  mode 0 (default): the fp32 Theta, complete on every rank after
 * every update.  mode 1: only the model's compute-type weights (one all-reduce over half the bytes in a bf16 model,
 * and no second pass that re-casts Theta); the fp32 values of ranges owned by other ranks are then stale until
 * femto_optimizer_gather_theta, which a host calls before it reads Theta (a checkpoint, src/checkpoints.jl:27-36).
 * Training itself never reads them: a rank's optimiser touches only the ranges it owns, and the forward and reverse
 * passes read the compute-type weights (the fp32 scalars and gates are updated by every rank). */
int32_t femto_optimizer_set_exchange(femto_optimizer* o, int32_t mode);
int32_t femto_optimizer_gather_theta(femto_optimizer* o, float* theta, void* stream);
/* femto_grad_sync for a sharded optimiser: a range of delta that one rank alone consumes is summed only onto
 * that rank (in-place reduce-scatter per table, reduce to the owner per block), which moves half the bytes of
 * the all-reduce; on the other ranks such a range keeps the local gradient.  Everything else, the loss and
 * n_valid are all-reduced.  Without sharding it equals femto_grad_sync. */
int32_t femto_optimizer_grad_sync(femto_optimizer* o, float* delta, float* loss_inout, int32_t* n_valid_inout,
                                  void* stream);
/* (offset, count, owner rank) triplets, in floats, of every range of Theta that one rank alone updates under
 * the current sharding; returns their number (h_out receives at most `capacity` of them). */
int32_t femto_optimizer_shard_ranges(femto_optimizer* o, int64_t* h_out, int32_t capacity);
/* Which rank holds the current moments of which part of a state buffer under the sharding (which: 0 adam_m,
 * 1 adam_v, 2 muon_m, 3 muon_v): sorted (offset, count, owner) triplets in floats covering the whole buffer;
 * replicated groups are listed with owner 0.  Returns their number. */
int32_t femto_optimizer_state_ranges(femto_optimizer* o, int32_t which, int64_t* h_out, int32_t capacity);
/* Make the four state buffers complete on every rank, so that `optimizer_state` (src/checkpoints.jl:9-12) can be
 * taken from any one of them and the sharding (or the number of ranks) may change afterwards: each rank clears
 * the parts held elsewhere, then one all-reduce per buffer.  No-op without sharding.  Asynchronous on `stream`. */
int32_t femto_optimizer_gather_state(femto_optimizer* o, void* stream);
/* Step counters t of the AdamW groups (:17,35), for checkpoints (src/checkpoints.jl:9-12). */
int32_t femto_optimizer_get_t(femto_optimizer* o, int32_t* h_t, int32_t capacity);
int32_t femto_optimizer_set_t(femto_optimizer* o, const int32_t* h_t, int32_t count);

/* ---- kernel-level seams (ext/FemtoChatCUDAExt.jl:3-5,161-163) --------------------------------- */
/* attention!(A,O,l,m,Q,K,V,window) (ext/FemtoChatCUDAExt.jl:1242).  Q,O: [B][T][H][hd]; K,V:
 * [B][T][Hkv][hd]; l,m: fp32 [B][H][T] (row sum and row max in natural-log units; either may be
 * NULL); lse: fp32 [B][H][T] = m + log l (may be NULL).  doc_start: int32 [B][T] or NULL. */
int32_t femto_attention_fwd(int32_t dtype, void* O, float* l, float* m, float* lse, const void* Q,
                            const void* K, const void* V, int32_t B, int32_t T, int32_t H, int32_t Hkv,
                            int32_t hd, int32_t window_left, const int32_t* doc_start, void* stream);
/* Δattention!(A,dQ,dK,dV,dO,Q,K,V,O,l,m,window; accumulate=true) (ext/FemtoChatCUDAExt.jl:1771-1776).  The saved
 * row statistics are given either as lse = m + log l, or as the reference's pair (l, m) with lse NULL.
 * accumulate != 0 adds to dQ / dK / dV (the reference's default), 0 overwrites them.  Synchronises before returning
 * (its scratch is a grow-only buffer that the library keeps per device); a bounded wait that ran out inside a kernel
 * comes back as FEMTO_ERR_DEVICE_STATUS + the status word. */
int32_t femto_attention_bwd(int32_t dtype, void* dQ, void* dK, void* dV, const void* dO, const void* Q,
                            const void* K, const void* V, const void* O, const float* lse, const float* l,
                            const float* m, int32_t B, int32_t T, int32_t H, int32_t Hkv, int32_t hd,
                            int32_t window_left, const int32_t* doc_start, int32_t accumulate, void* stream);
/* Same computation as femto_attention_bwd for callers that cannot allocate device memory (a host
 * runtime that owns the whole device pool, or a phase in which cudaMalloc is forbidden or would
 * stall the device).  No counterpart in the reference.  The scratch (two floats per (batch, head,
 * query)) lives in an 8 MiB array compiled into the library, so the call is limited to
 * B*H*T <= 1 048 576 and fails with FEMTO_ERR_SHAPE beyond that; it never calls cudaMalloc/cudaFree.
 * The first call on a device looks up the array's device address (make that call before any stream
 * capture).  All calls on a device share the array: calls that overlap on the GPU (different
 * streams) race; calls on one stream are safe.  Asynchronous on `stream`; always overwrites dQ / dK / dV and takes
 * lse only.  Its device status word (also part of the library image) is included in femto_status_word(NULL, ..).
 * The cached device addresses are looked up without locking (two first calls from different host threads both do
 * the lookup) and are not refreshed after cudaDeviceReset. */
int32_t femto_attention_bwd_static(int32_t dtype, void* dQ, void* dK, void* dV, const void* dO, const void* Q,
                                   const void* K, const void* V, const void* O, const float* lse, int32_t B,
                                   int32_t T, int32_t H, int32_t Hkv, int32_t hd, int32_t window_left,
                                   const int32_t* doc_start, void* stream);
/* C[M][N] = A[M][K] * B[K][N] in bf16 with fp32 accumulation on the tcgen05 path; each operand may be
 * stored K-contiguous (kmajor=1) or M/N-contiguous (kmajor=0); replaces the cuBLAS calls behind the
 * generic `W*X` (src/gpt.jl:28) and batched_mul! (ext/FemtoChatCUDAExt.jl:121-125).  out_f32=1 writes
 * fp32, accumulate=1 adds to C (fp32 only). */
int32_t femto_gemm_bf16(const void* A, int32_t a_kmajor, int64_t lda, const void* B, int32_t b_kmajor,
                        int64_t ldb, void* C, int64_t ldc, int32_t M, int32_t N, int32_t K, int32_t batch,
                        int64_t strideA, int64_t strideB, int64_t strideC, int32_t out_f32,
                        int32_t accumulate, void* stream);
/* The tensor-core GEMM computes 256 x 256 output tiles with PAIRS of CTAs (tcgen05.mma.cta_group::2: each CTA holds
 * 128 rows of A and half of B's columns, a third less operand traffic per flop) wherever M >= 256, and 128 x 256
 * tiles with single CTAs otherwise.  mode 0 forces single CTAs, 1 restores the default, anything else only
 * queries; returns the previous mode.  A measurement and debugging aid with no counterpart in the reference. */
int32_t femto_gemm_pair_mode(int32_t mode);
/* embedding_gradient!(δ,dy,tokens) (src/kernels.jl:8-14): δ[tokens[n]] += dy[n], deterministic
 * (fixed summation order), tokens 0-based int32 [N], dy [N][D] of `dtype`, δ fp32 [rows][D]. */
int32_t femto_embedding_gradient(int32_t dtype, float* delta_table, const void* dy, const int32_t* tokens0,
                                 int32_t N, int32_t D, int32_t rows, void* stream);
/* cross_entropy(logits, targets, ignore, reduction) on materialised logits (src/gpt.jl:175-193; the
 * reference's GPU method ext/FemtoChatCUDAExt.jl:49-55): logits fp32 [N][ldl] (the (V,T,B) array, first V
 * columns used), targets0 0-based or -1.  out: one float (sum / mean over valid targets) or [N] floats
 * (FEMTO_REDUCTION_NONE, ignored rows 0).  Synchronises for sum / mean (its scratch is a grow-only buffer that the library keeps per device). */
int32_t femto_cross_entropy(const float* logits, int64_t ldl, const int32_t* targets0, int32_t N, int32_t V,
                            int32_t reduction, float* out, int32_t* n_valid_out, void* stream);
/* cross_entropy_gradient!(delta, logits, targets, dy, ignore, reduction) (src/kernels.jl:16-28; GPU method
 * ext/FemtoChatCUDAExt.jl:57-61): delta[N][ldd] += scale (softmax(logits) - onehot) on rows with a target,
 * scale = dy (sum), dy / n_valid (mean) or dy_rows[row] (none; device array [N]). */
int32_t femto_cross_entropy_gradient(float* delta, int64_t ldd, const float* logits, int64_t ldl,
                                     const int32_t* targets0, int32_t N, int32_t V, int32_t reduction, float dy,
                                     const float* dy_rows, void* stream);
/* Fused lm_head tail (src/gpt.jl:165-170,172-194; src/kernels.jl:16-28): loss = sum over valid
 * targets of logsumexp(z) - z[target], z = 15 tanh(x W / 15); dX and dW (+=) of that loss.
 * x: [N][D] dtype, W: [D][ldw] dtype (first V columns used), targets0: 0-based or -1,
 * dx: [N][D] dtype, dw: fp32 [D][ldw]. */
int32_t femto_xent_fused(int32_t dtype, const void* x, const void* W, int64_t ldw, const int32_t* targets0,
                         int32_t N, int32_t D, int32_t V, float scale, void* dx, float* dw,
                         float* loss_out, int32_t* n_valid_out, void* stream);
/* Polar Express / Newton-Schulz (src/optim.jl:131-149) on a stack of k row-major [rows][cols]
 * bf16 or fp32 matrices, in place; coeffs = steps x (a,b,c). */
int32_t femto_newton_schulz(int32_t dtype, void* X, int32_t k, int32_t rows, int32_t cols,
                            const float* h_coeffs, int32_t steps, void* stream);
/* AdamW on one flat range (src/optim.jl:33-39,75-87), one fused pass. */
int32_t femto_adamw(float* theta, const float* delta, float* m, float* v, int64_t n, float alpha,
                    float beta1, float beta2, float eps, float lambda, int32_t t, float n_tokens,
                    void* stream);

/* norm (src/gpt.jl:16-20): y = x / r, r = sqrt(mean(x^2) + eps) over each row of x [N][D]; r [N] is kept for the
 * reverse.  eps is the caller's eps(eltype): 2^-7 in a bf16 model, 2^-23 in fp32.  Asynchronous. */
int32_t femto_rmsnorm_fwd(int32_t dtype, const void* x, void* y, float* r, int32_t N, int32_t D, float eps,
                          void* stream);
/* Reverse of norm (ext/FemtoChatMooncakeExt.jl:248-255) from the saved output: dx = (dy - y mean(dy y)) / r,
 * which equals dy / r - x sum(dy x) / (D r^3).  Asynchronous. */
int32_t femto_rmsnorm_bwd(int32_t dtype, const void* dy, const void* y, const float* r, void* dx, int32_t N,
                          int32_t D, void* stream);
/* The Embedding call E[:, tokens] (src/gpt.jl:34; GPU kernel ext/FemtoChatCUDAExt.jl:63-75): out[n] = table[tokens0[n]],
 * table [rows][D] and out [N][D] of `dtype`, tokens 0-based.  An id outside 0..rows-1 is clamped and raises bit 1 of
 * the status word that femto_status_word(NULL, ..) reads.  Asynchronous. */
int32_t femto_embed_gather(int32_t dtype, void* out, const void* table, const int32_t* tokens0, int32_t N, int32_t D,
                           int32_t rows, void* stream);
/* muon_direction! (src/optim.jl:198-236) on a stack of k same-shape matrices: Nesterov momentum, MuonEq row
 * equilibration, Polar Express in `dtype`, Muon+ renormalisation and the NorMuon second-moment scaling.
 * G, momentum and X_out are fp32 [k][rows][cols] where a Julia (m, n) matrix is stored as rows = n, cols = m;
 * second_moment is fp32 [k][cols] when cols >= rows, else [k][rows]
 * (src/optim.jl:180).  momentum and second_moment are updated in place.  Synchronises before returning. */
int32_t femto_muon_direction(int32_t dtype, float* X_out, const float* G, float* momentum, float* second_moment,
                             int32_t k, int32_t rows, int32_t cols, float mu, float beta2, float n_tokens,
                             const float* h_coeffs, int32_t steps, void* stream);

/* ---- status --------------------------------------------------------------------------------- */
/* Device status word (0 = ok): bounded waits that ran out (bit 2), out-of-range token ids (bit 1), ...
 * h == NULL reads AND CLEARS the word of the stand-alone kernel-level entry points on the current device (after a
 * cudaDeviceSynchronize); a bit raised by an asynchronous entry point that nobody read is reported by the next
 * synchronising one as FEMTO_ERR_DEVICE_STATUS + word. */
int32_t femto_status_word(femto_handle* h, int32_t* h_out);
int32_t femto_sync(femto_handle* h, void* stream);
/* Number of kernels launched by this handle since creation (host counter). */
int64_t femto_launch_count(femto_handle* h);

/* Self test of the bounded waits that every warp-specialised kernel uses: one thread waits, with a poll limit of
 * `polls`, on a barrier that nothing completes.  It must give up and raise status bit 2 (*h_status), a second role
 * waiting on the same barrier must leave through the abort flag, and the kernel must return by itself:
 * h_result2[0] = waiter timed out, h_result2[1] = second role unwound.  Nothing traps or hangs. */
int32_t femto_selftest_bounded_wait(int32_t polls, int32_t* h_status, int32_t* h_result2);

/* Measurement aid (no counterpart in the reference): when enabled, every launch of the tensor-core
 * GEMM kernel is bracketed by CUDA events on its stream; the report returns the summed kernel time,
 * the summed 2*M*N*K and the launch count since the last femto_profile_gemm call. */
int32_t femto_profile_gemm(int32_t enable);
int32_t femto_profile_gemm_report(double* h_ms, double* h_flops, int32_t* h_launches);

#ifdef __cplusplus
}
#endif
#endif
