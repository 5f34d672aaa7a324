/*
 * lumen_moe.h -- C ABI of the B200 (sm_100a) MoE feed-forward operator.
 *
 * This is the boundary a lumen-runtime CUDA backend binds instead of launching
 * its NVRTC MoE kernels. Every entry point names the reference function it
 * replaces (paths relative to the reference project's root). All pointers named
 * d_* are device pointers; `stream` is a cudaStream_t passed as void*. Calls are
 * asynchronous on that stream and never synchronise it, except where stated.
 * No exceptions cross this boundary; every function returns a status code and
 * lumen_moe_last_error() gives the text of the last failure on the calling thread.
 *
 * There is no CPU fallback: if the CUDA library cannot run a request it returns
 * an error.
 */
#ifndef LUMEN_MOE_H
#define LUMEN_MOE_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define LUMEN_MOE_API __attribute__((visibility("default")))
#else
#define LUMEN_MOE_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Result<(), RuntimeError> of crates/lumen-runtime/src/error.rs:6-31:
 * INVALID_ARG / CUDA_ERROR ~ RuntimeError::Compute, UNSUPPORTED ~ RuntimeError::Unsupported. */
typedef enum {
    LUMEN_MOE_OK = 0,
    LUMEN_MOE_INVALID_ARG = 1,
    LUMEN_MOE_UNSUPPORTED = 2,
    LUMEN_MOE_CUDA_ERROR = 3,
    LUMEN_MOE_TIMEOUT = 4,
    LUMEN_MOE_NCCL_ERROR = 5
} lumen_moe_status_t;

/* lumen_format::quantization::QuantScheme tags accepted on this path
 * (cuda/moe.rs:1185-1191: gate and down must share one of these). */
typedef enum { LUMEN_MOE_Q8_0 = 0, LUMEN_MOE_Q4_0 = 1, LUMEN_MOE_BF16 = 2 } lumen_moe_quant_t;

/* SOFTMAX_RENORM: cuda/moe.rs:6464-6504 (CPU reference) and cuda/shaders/moe_router.cu:85-128.
 * SIGMOID_RENORM: cuda/shaders/topk_moe_fused.cu:118-129 (the CUDA backend's default). */
/* 0, 1: routed experts (softmax / sigmoid over E, top-k, weights renormalised).
 * 2, 3: the always-on shared expert as a context with num_experts = top_k = 1
 * (cuda/moe.rs:5455-5520): weight = sigmoid(dot(ffn_gate_inp_shexp, x)), or 1 when the
 * model has no gate vector. */
typedef enum {
    LUMEN_MOE_SOFTMAX_RENORM = 0,
    LUMEN_MOE_SIGMOID_RENORM = 1,
    LUMEN_MOE_SIGMOID_GATE = 2,
    LUMEN_MOE_UNIT_WEIGHT = 3
} lumen_moe_gating_t;

/* Activation element types of lumen_moe_prefill. */
/* LUMEN_MOE_ACT_F16 is accepted only where the caller supplies the routing
 * (lumen_moe_prefill_routed, lumen_moe_experts_routed_f16): it is the wire type of
 * f32 activations between expert-parallel ranks. */
typedef enum { LUMEN_MOE_ACT_F32 = 0, LUMEN_MOE_ACT_BF16 = 1, LUMEN_MOE_ACT_F16 = 2 } lumen_moe_act_t;

typedef struct {
    int32_t hidden_dim;   /* H, multiple of 32 */
    int32_t inter_dim;    /* I, multiple of 32 */
    int32_t num_experts;  /* E <= 256 (cuda/shaders/moe_router.cu:33) */
    int32_t top_k;        /* K <= 16  (cuda/shaders/moe_router.cu:34) */
    int32_t max_tokens;   /* initial prefill capacity; grows on demand */
    int32_t gating_mode;  /* lumen_moe_gating_t */
    int32_t device;       /* CUDA ordinal */
    int32_t flags;        /* 0, or LUMEN_MOE_FLAG_* or'ed together */
} lumen_moe_config;

/* Kernel selection is part of the configuration, never of the environment (the reference
 * selects its kernel generations through ~30 environment variables, cuda/moe.rs:1304-1561;
 * this library reads none).
 * DECODE_SPLIT: 1..4-token decode on the three-kernel chain instead of the persistent
 *   cooperative kernel (for a process that cannot give the kernel every SM of the device).
 * PREFILL_MMA: grouped products on mma.sync instead of tcgen05 (values outside f16 range).
 * SHORT_WAITS: device-side bounded waits give up after 2 ms instead of 1-2 s (tests).
 * PREFILL_F16_WEIGHTS: layers prepared on this context also keep their Q4_0 / Q8_0 expert weights
 *   as plain f16 matrices (2 more bytes per weight per layer: 1.2 GB at H=2048, I=768, E=128),
 *   and prefill feeds the tensor cores from them with TMA instead of dequantising in shared
 *   memory: memory traded for prefill speed. BF16 layers always work that way (nothing to
 *   dequantise). Decode is not affected.
 * TC_CTAS(n): cap of the persistent tcgen05 grid, n CTAs (one per SM), 0 = every SM. */
#define LUMEN_MOE_FLAG_DECODE_SPLIT 0x1
#define LUMEN_MOE_FLAG_PREFILL_MMA 0x2
#define LUMEN_MOE_FLAG_SHORT_WAITS 0x4
#define LUMEN_MOE_FLAG_PREFILL_F16_WEIGHTS 0x8
#define LUMEN_MOE_FLAG_TC_CTAS(n) (((n) & 0xff) << 8)

typedef struct lumen_moe_ctx lumen_moe_ctx;     /* ~ CudaMoeScratch, cuda/moe.rs:101-170 */
typedef struct lumen_moe_layer lumen_moe_layer; /* ~ CudaMoeMeta + CudaMoeBatchedOffsets + CudaMoeRepacked */

/* Replaces allocate_moe_scratch (cuda/moe.rs:968). Synchronous (allocates). */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_create(const lumen_moe_config* cfg, lumen_moe_ctx** out_ctx);
LUMEN_MOE_API void lumen_moe_destroy(lumen_moe_ctx* ctx);

/* Replaces ensure_prefill_grouped (cuda/moe.rs:1015): grow-only capacity for
 * `tokens` tokens. Synchronous when it has to reallocate. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_ensure_prefill(lumen_moe_ctx* ctx, int32_t tokens);

/* Replaces build_moe_meta (cuda/moe.rs:223) + build_batched_offsets (:272) +
 * build_repacked_down (:337). d_layer_blob is the layer's weight blob as uploaded
 * by the backend (router f32 [E,H] at router_off; expert e: gate [I,H] at
 * gate_offs[e], up [I,H] at up_offs[e], down [H,I] at down_offs[e]; raw GGML
 * Q8_0 / Q4_0 blocks or BF16, rows contiguous along the input dimension). The
 * offset arrays are HOST arrays of num_experts entries. The blob is left
 * untouched and must outlive the layer (the router weight is read in place when it
 * sits on a 16-byte boundary of device memory; a file's layer blob only promises
 * 4 bytes, and then the layer keeps its own aligned copy); the
 * expert weights are repacked once into aligned planes owned by the layer.
 * Passing NULL for all three offset tables prepares a router-only layer (nothing
 * repacked; valid for lumen_moe_route_only only), which is what an expert-parallel
 * rank uses for the replicated router.
 * Work is enqueued on `stream`; the function synchronises it before returning. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_layer_prepare(lumen_moe_ctx* ctx, const void* d_layer_blob,
                                           size_t blob_bytes, uint64_t router_off,
                                           const uint64_t* gate_offs, const uint64_t* up_offs,
                                           const uint64_t* down_offs, int32_t quant, void* stream,
                                           lumen_moe_layer** out_layer);
LUMEN_MOE_API void lumen_moe_layer_destroy(lumen_moe_layer* layer);

/* Replace encode_shared_expert_ffn_decode (cuda/moe.rs:5494) and
 * encode_shared_expert_ffn_prefill_batched (cuda/moe.rs:2788): the always-on shared expert,
 *   out[t] += g[t] * Down_sh(silu(Gate_sh x[t]) * Up_sh x[t]),
 *   g[t] = sigmoid(dot(ffn_gate_inp_shexp, x[t]))   (LUMEN_MOE_SIGMOID_GATE) or 1 (LUMEN_MOE_UNIT_WEIGHT),
 * accumulated INTO d_out, which already holds the routed experts' result. `ctx` is a
 * context created with num_experts = top_k = 1, inter_dim = the shared expert's inter
 * dim and gating_mode 2 or 3; `layer` was prepared on the same layer blob with
 * router_off = offset of ffn_gate_inp_shexp (F32 [H]; any valid offset in mode 3) and the
 * three shared-expert slices as one-element offset arrays. Decode: 1 <= T <= 16, f32. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_shared_expert_decode(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                                const float* d_normed, float* d_out,
                                                                int32_t tokens, void* stream);
LUMEN_MOE_API lumen_moe_status_t lumen_moe_shared_expert_prefill(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                                 const void* d_normed, float* d_out,
                                                                 int32_t tokens, int32_t act_dtype, void* stream);

/* Replaces encode_moe_ffn_decode (cuda/moe.rs:1119): out[t] = residual[t] +
 * sum_k w[t,k] * Down_e(silu(Gate_e x[t]) * Up_e x[t]), f32 [T,H] in and out,
 * 1 <= T <= 16. d_out may alias d_residual (the backend passes the same buffer,
 * cuda/backend_impl.rs:3570-3573) but not d_normed. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_decode(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                    const float* d_normed, const float* d_residual, float* d_out,
                                    int32_t tokens, void* stream);

/* Replaces encode_moe_ffn_decode_fused_norm (cuda/moe.rs:3184): normed =
 * rmsnorm(x; gamma, eps) (cuda/shaders/norm.cu:28-76), then as lumen_moe_decode
 * with residual = x. d_normed_out receives normed [T,H] (may be NULL). */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_decode_fused_norm(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                               const float* d_x, const float* d_gamma,
                                               float* d_normed_out, float* d_out, float eps,
                                               int32_t tokens, void* stream);

/* Replaces encode_moe_ffn_prefill_grouped (cuda/moe.rs:1900) without its host
 * round trip: routing, the stable counting sort (:2115-2147), the grouped expert
 * products and the scatter-accumulate all run on the device. d_normed is
 * [T,H] of act_dtype; d_residual and d_out are f32 [T,H]. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_prefill(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                     const void* d_normed, const float* d_residual, float* d_out,
                                     int32_t tokens, int32_t act_dtype, void* stream);

/* As lumen_moe_prefill, with the routing supplied by the caller instead of being
 * computed: d_ids u32 [T,K] (expert ids valid for THIS context, i.e. local ids on
 * an expert-parallel rank), d_weights f32 [T,K] or NULL (all 1). No counterpart in
 * the reference (it has no expert parallelism, cuda/ffi.rs:61-87): this is what a
 * rank runs on the rows it received in the dispatch all-to-all. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_prefill_routed(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                          const void* d_normed, const uint32_t* d_ids,
                                                          const float* d_weights, const float* d_residual,
                                                          float* d_out, int32_t tokens, int32_t act_dtype,
                                                          void* stream);

/* Expert-parallel building blocks (no counterpart in the reference).
 * lumen_moe_experts_routed_f16: on a context with top_k = 1, the expert FFN
 * Down_e(silu(Gate_e x) * Up_e x) of every row with its caller-supplied local expert id
 * d_ids[r]; output f16 [rows, H] in the caller's row order, unweighted.
 * lumen_moe_combine_f16: out[t] = residual[t] + sum_slot w[t,slot] * D[dst_to_col[t*K+slot]]
 * in slot order (moe_grouped_scatter_accum_q8_0, cuda/shaders/moe_grouped.cu:493-517) on
 * f16 rows D, e.g. those returned by the combine all-to-all. Needs no context. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_experts_routed_f16(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                              const void* d_rows, const uint32_t* d_ids,
                                                              void* d_out16, int32_t rows, int32_t act_dtype,
                                                              void* stream);
LUMEN_MOE_API lumen_moe_status_t lumen_moe_combine_f16(const void* d_d16, const float* d_residual,
                                                       const float* d_weights, const int32_t* d_dst_to_col,
                                                       float* d_out, int32_t tokens, int32_t hidden_dim,
                                                       int32_t top_k, void* stream);

/* Router only (moe_router_logits_v2 + finalize, cuda/shaders/moe_batched.cu:708,755;
 * batched: cuda/shaders/moe_grouped.cu:79 + topk_moe_fused.cu:172-296).
 * d_ids u32 [T,K] in selection (descending weight) order, row stride K;
 * d_weights f32 [T,K], each row sums to 1. d_logits_out [T,E] may be NULL. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_route_only(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                        const float* d_normed, int32_t tokens, uint32_t* d_ids,
                                        float* d_weights, float* d_logits_out, void* stream);

/* Gating + top-k + renormalisation on caller-supplied logits f32 [T,E]: the
 * arithmetic of cpu_router_softmax phases 2-3 (cuda/moe.rs:6464-6504), bit for
 * bit (ids and weights) for finite logits. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_topk_from_logits(lumen_moe_ctx* ctx, const float* d_logits,
                                              int32_t tokens, uint32_t* d_ids, float* d_weights,
                                              void* stream);

/* Routing for callers that cannot allocate device memory. No counterpart in the
 * reference (its router always works out of the CudaMoeScratch that
 * allocate_moe_scratch cudaMallocs). Same arithmetic and same results as
 * lumen_moe_topk_from_logits for 1..16 tokens, but it takes no context: its
 * working tables live in an 8 KiB array that is part of the library image on every
 * GPU that loads it, so the call performs no cudaMalloc / cudaFree at all. Meant
 * for hosts that pre-claim all device memory for their own pool, or that must not
 * enter the driver allocator from their decode loop (it synchronises the device).
 * Limits, fixed by that array and checked (LUMEN_MOE_INVALID_ARG otherwise):
 * tokens <= 16, num_experts <= 256, top_k <= 16.
 * d_logits f32 [T,E]; outputs d_ids u32 [T,K], d_weights f32 [T,K]; optional
 * d_dst_to_col i32 [T*K] and d_expert_bounds i32 [E+1] (NULL to skip).
 * The first call on a device looks up the array's device address; make that call
 * at start-up, before any stream capture begins. All calls on a GPU share the
 * array (it keeps the previous call's contents; the call clears what must start
 * at zero), so calls that could overlap on the GPU must be serialised by the caller. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_route_small_static(const float* d_logits, int32_t tokens,
                                                              int32_t num_experts, int32_t top_k,
                                                              int32_t gating_mode, uint32_t* d_ids,
                                                              float* d_weights, int32_t* d_dst_to_col,
                                                              int32_t* d_expert_bounds, void* stream);

/* Parity hook: while set (non-NULL), lumen_moe_decode / _prefill take the router
 * logits f32 [T,E] from this device buffer instead of computing them, so that
 * both sides of a parity test route on identical logits. NULL switches it off. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_set_logits_override(lumen_moe_ctx* ctx, const float* d_logits);

/* Readback of the routing tables of the most recent call (debug / parity; the
 * counterpart of the MOE_EXPERT_DUMP lines, cuda/moe.rs:1484-1492). Host output
 * arrays, any may be NULL: ids [T,K], weights [T,K], dst_to_col [T*K],
 * col_src_tok [T*K], expert_bounds [E+1] (cuda/moe.rs:2115-2147). Synchronises `stream`.
 * If the context's error word is set it returns that code and clears it (as
 * lumen_moe_clear_status does). */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_get_routing(lumen_moe_ctx* ctx, int32_t tokens, uint32_t* ids,
                                         float* weights, int32_t* dst_to_col, int32_t* col_src_tok,
                                         int32_t* expert_bounds, void* stream);

/* The ids of the most recent routing call in the layout of the reference's batched id
 * buffer: u32 [T, E] with row stride E, the first K entries of a row valid and the rest 0
 * (cuda/shaders/topk_moe_fused.cu:189-191, read back at cuda/moe.rs:2116-2121), for a
 * byte-level diff against a reference dump. Host output. Synchronises `stream`. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_get_routing_ids_stride_e(lumen_moe_ctx* ctx, int32_t tokens,
                                                                    uint32_t* ids_stride_e, void* stream);

/* Error state of the context (the counterpart of the Result<(), RuntimeError> every launch of
 * the reference returns, error.rs:6-31, cuda/moe.rs:1497-1502). Kernels cannot return a code, so a
 * kernel that gives up (a bounded wait that ran out: LUMEN_MOE_TIMEOUT; an expert id >= E in
 * caller-supplied routing: LUMEN_MOE_INVALID_ARG) records the code in a word of pinned host
 * memory owned by the context. lumen_moe_poll_status reads that word: no device work, no
 * synchronisation; it reflects every kernel that has finished. Once the word is set, every
 * entry point that would launch on the context fails with that code instead of launching
 * (outputs of the failed call and of calls enqueued behind it are undefined).
 * lumen_moe_clear_status synchronises `stream`, resets the word and the device-side barrier
 * state, and makes the context usable again. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_poll_status(const lumen_moe_ctx* ctx);
LUMEN_MOE_API lumen_moe_status_t lumen_moe_clear_status(lumen_moe_ctx* ctx, void* stream);

/* Test hook for the give-up paths, without faulting or hanging anything: the NEXT kernel of
 * the given kind launched on this context waits for something that cannot happen (which = 0:
 * the grid barrier of the persistent decode kernel expects one arrival more than there are
 * CTAs; which = 1: a stage barrier of the tcgen05 grouped GEMM expects one byte more than the
 * copies deliver), so its bounded wait runs out, the kernel records LUMEN_MOE_TIMEOUT, releases
 * what it holds and returns. Use with LUMEN_MOE_FLAG_SHORT_WAITS. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_debug_expire_next_wait(lumen_moe_ctx* ctx, int32_t which);

/* Device-to-device copy of the sort tables of the most recent routing call (no
 * synchronisation): dst_to_col [T*K], col_src_tok [T*K], col_expert [T*K],
 * expert_bounds [E+1] (cuda/moe.rs:2115-2147); any pointer may be NULL. The
 * expert-parallel dispatch uses them as its send plan. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_get_routing_device(lumen_moe_ctx* ctx, int32_t tokens,
                                                              int32_t* d_dst_to_col, int32_t* d_col_src_tok,
                                                              int32_t* d_col_expert, int32_t* d_expert_bounds,
                                                              void* stream);

/* Expert-parallel send side, after lumen_moe_route_only on the same context: in one launch,
 * d_rows16 [T*K, H] = the activation rows in compact-column order (rows for rank r are
 * contiguous, experts being contiguous per rank) as 16-bit values: bf16 (exact) when the
 * activations are bf16, f16 (the rounding the single-GPU grouped GEMM applies to its
 * operand) when they are f32; d_local_ids [T*K] = expert id relative to
 * its rank, d_send_counts [E / experts_per_rank] (int64) = rows per destination rank.
 * (The reference is single-GPU; this belongs to the additive expert-parallel form.) */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_ep_prepare(lumen_moe_ctx* ctx, const void* d_normed, int32_t act_dtype,
                                                      int32_t tokens, int32_t experts_per_rank, void* d_rows16,
                                                      int32_t* d_local_ids, int64_t* d_send_counts, void* stream);

/* ---- Expert-parallel prefill over several GPUs (one process per GPU) -------------------
 * No counterpart in the reference, which is single-GPU (one context, one stream,
 * cuda/ffi.rs:61-87): the multi-GPU form of encode_moe_ffn_prefill_grouped (cuda/moe.rs:1900)
 * for multi-token batches. Tokens are sharded over `world` ranks, experts E / world per rank
 * (rank r owns experts [r * E / world, (r + 1) * E / world)), the router weight is replicated.
 * The ranks exchange rows and results by plain stores into each other's device memory over
 * NVLink (CUDA IPC mappings); the library calls no collective and the host is not in the
 * loop: a layer call is one asynchronous call per rank on its stream.
 *
 * Set-up, once per rank, on a context created with the GLOBAL num_experts and top_k:
 *   lumen_moe_ep_create   allocates this rank's window (receive buffers and flags) and writes
 *                         its 64-byte IPC handle to handle_out. max_tokens = most tokens THIS
 *                         rank passes per call; recv_rows = rows this rank can receive per call,
 *                         0 = max_tokens * top_k * world (no routing skew can overflow that;
 *                         every rank must use the same values). Synchronous (allocates).
 *   (the host gathers the `world` handles in rank order: its own transport, e.g. the launcher's
 *    rendezvous; the handle of a rank's own slot is ignored)
 *   lumen_moe_ep_attach   maps the peers' windows. Synchronous.
 *   lumen_moe_ep_layer_prepare   as lumen_moe_layer_prepare, with the offset tables of ALL
 *                         num_experts experts: keeps the router weight and repacks only this
 *                         rank's experts.
 * Per layer call, on every rank (a collective call: all ranks make the same sequence of
 * calls, each on its own tokens; tokens may differ per rank, 1 <= tokens <= max_tokens):
 *   lumen_moe_prefill_ep  out[t] = residual[t] + sum_k w[t,k] * FFN_{e(t,k)}(normed[t]) for this
 *                         rank's tokens; bit-identical to lumen_moe_prefill on one GPU for the
 *                         same tokens. d_normed [T,H] f32 or bf16, 16-byte aligned.
 *   lumen_moe_stack_prefill_ep   the layer stack of lumen_moe_stack_prefill in this form.
 * Every cross-rank wait is bounded (2 s; 2 ms with LUMEN_MOE_FLAG_SHORT_WAITS): a rank whose
 * peer does not show up gets LUMEN_MOE_TIMEOUT through lumen_moe_poll_status, and an overflow
 * of recv_rows gives LUMEN_MOE_INVALID_ARG the same way; no index ever leaves a window.
 * A rank must not destroy its context while a peer may still write to it. */
#define LUMEN_MOE_EP_HANDLE_BYTES 64
LUMEN_MOE_API lumen_moe_status_t lumen_moe_ep_create(lumen_moe_ctx* ctx, int32_t rank, int32_t world,
                                                     int32_t max_tokens, int32_t recv_rows, void* handle_out);
LUMEN_MOE_API lumen_moe_status_t lumen_moe_ep_attach(lumen_moe_ctx* ctx, const void* handles, int32_t rank,
                                                     int32_t world);
LUMEN_MOE_API lumen_moe_status_t lumen_moe_ep_layer_prepare(lumen_moe_ctx* ctx, const void* d_layer_blob,
                                                            size_t blob_bytes, uint64_t router_off,
                                                            const uint64_t* gate_offs, const uint64_t* up_offs,
                                                            const uint64_t* down_offs, int32_t quant, void* stream,
                                                            lumen_moe_layer** out_layer);
LUMEN_MOE_API lumen_moe_status_t lumen_moe_prefill_ep(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                      const void* d_normed, const float* d_residual, float* d_out,
                                                      int32_t tokens, int32_t act_dtype, void* stream);
LUMEN_MOE_API lumen_moe_status_t lumen_moe_stack_prefill_ep(lumen_moe_ctx* ctx, const lumen_moe_layer* const* layers,
                                                            const float* const* d_gammas, int32_t n_layers,
                                                            float* d_x, float* d_normed, float eps, int32_t tokens,
                                                            void* stream);

/* Timing aid: with profiling on, lumen_moe_prefill_ep records CUDA events between its launches;
 * lumen_moe_ep_phase_ms waits for the last profiled call and returns its six phases in ms:
 * route + sort | counts + dispatch (includes waiting for every rank's counts) | waiting for
 * every rank's rows + tile plan | gate/up + SwiGLU + down | waiting for every rank's results |
 * combine. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_ep_profile(lumen_moe_ctx* ctx, int32_t enable);
LUMEN_MOE_API lumen_moe_status_t lumen_moe_ep_phase_ms(lumen_moe_ctx* ctx, float* out_ms6);

/* ---- LBC container: header and layer index (host only, no device work) ----------------
 * The reference's backend uploads a MoE layer's blob byte for byte
 * (cuda/gpu_buffers.rs:1404-1409) and derives the operator's offsets from the layer's
 * index entry (build_moe_meta, cuda/moe.rs:223-262). These two calls read the same
 * index from an LBC file held in host memory, so that a checkpoint's layer goes to
 * lumen_moe_layer_prepare with the offsets the file itself records. */

/* TensorSlice of crates/lumen-format/src/index.rs:158-164: a byte range relative to the
 * layer blob start and its scheme tag (quantization.rs:123-137: 0 F32, 1 F16, 2 BF16,
 * 3 Q8_0, 4 Q4_0, ...). present = 0 for an optional slice the entry does not carry. */
typedef struct {
    uint64_t offset;
    uint64_t length;
    uint32_t quant;
    uint32_t present;
} lumen_lbc_slice;

/* The header fields the operator's caller needs (header.rs:41-78, hyperparams of
 * reader.rs:383-481). */
typedef struct {
    uint32_t version;            /* <= 4 */
    uint32_t num_layers;
    uint32_t num_heads, num_kv_heads, head_dim;
    uint32_t hidden_dim;         /* H */
    uint32_t intermediate_dim;
    uint32_t vocab_size, max_seq_len;
    uint32_t num_experts;        /* 0 for a dense model */
    uint32_t num_active_experts; /* top-k; 0 for a dense model */
    float norm_eps;
    uint32_t primary_quant;      /* scheme tag of the primary descriptor */
    uint32_t has_expert_index;
    uint64_t alignment;
    uint64_t layer_index_offset;
    uint64_t payload_offset;
    uint64_t header_bytes;       /* 183 (v2), 207 (v3), 208 or 224 (v4) */
} lumen_lbc_header;

/* One layer's entry, reduced to the MoE feed-forward path (~ CudaMoeMeta, cuda/moe.rs:39-59). */
typedef struct {
    uint64_t layer_offset_bytes; /* absolute position of the layer blob in the file */
    uint64_t layer_length_bytes;
    uint32_t is_moe;             /* router present and at least one expert */
    uint32_t num_experts;
    uint32_t expert_gate_quant;  /* scheme tag of expert 0's gate (= up) and down slices */
    uint32_t expert_down_quant;
    uint64_t expert_gate_bytes;  /* length of expert 0's gate slice: I = bytes / row bytes(H) */
    uint64_t expert_down_bytes;
    lumen_lbc_slice router_weight;       /* F32 [E, H] */
    lumen_lbc_slice ffn_norm;            /* F32 [H] */
    lumen_lbc_slice shared_expert_gate, shared_expert_up, shared_expert_down;
    lumen_lbc_slice ffn_gate_inp_shexp;  /* F32 [H] */
    uint32_t has_layer_type;
    uint32_t layer_type;
} lumen_lbc_moe_layer;

/* Replaces the header half of LbcFile::from_bytes (reader.rs:134-170, parse_lbc :212-357):
 * magic, version, checksum, alignment and layer-count checks with the reference's error
 * cases (INVALID_ARG: bad magic, truncated, checksum mismatch, bad alignment, layer count
 * mismatch; UNSUPPORTED: version > 4, big-endian). `data` needs to hold the header only. */
LUMEN_MOE_API lumen_moe_status_t lumen_lbc_read_header(const void* data, size_t bytes, lumen_lbc_header* out);

/* Replaces parse_layer_index (reader.rs:522-760) + LayerIndex::validate (index.rs:229-378)
 * + build_moe_meta (cuda/moe.rs:223-262) for layer `layer`: `data` holds the file from byte
 * 0 through the end of the layer index at least. The three offset tables (host, `capacity`
 * entries each, all or none) receive the per-expert byte offsets relative to the layer
 * blob, ready for lumen_moe_layer_prepare. A dense layer returns OK with is_moe = 0. */
LUMEN_MOE_API lumen_moe_status_t lumen_lbc_read_moe_layer(const void* data, size_t bytes, uint32_t layer,
                                                          lumen_lbc_moe_layer* out, uint64_t* gate_offs,
                                                          uint64_t* up_offs, uint64_t* down_offs, uint32_t capacity);

/* LBC scheme tag -> lumen_moe_quant_t, or -1 when the operator has no kernel for it. */
LUMEN_MOE_API int32_t lumen_lbc_quant_to_moe(uint32_t lbc_tag);

/* Device restatement of quantize_f32_to_q4_0 / _q8_0
 * (crates/lumen-convert/src/dequant.rs:791-906) and of round-to-nearest-even BF16,
 * used to synthesise weights in HBM. n_elements multiple of 32. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_quantize(const float* d_src, int64_t n_elements, int32_t quant,
                                      void* d_dst, void* stream);

/* rmsnorm of cuda/shaders/norm.cu:28-76 over [T,H] rows (FFN norm before the MoE call). */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_rmsnorm(const float* d_x, const float* d_gamma, float* d_out,
                                     int32_t tokens, int32_t hidden_dim, float eps, void* stream);

/* Stack of n_layers MoE FFN layers with identity mixers:
 * x <- x + MoE_l(rmsnorm(x; gamma_l, eps)), in place on d_x f32 [T,H], T <= 16.
 * The decode loop of cuda/backend_impl.rs:2184 (compute_layer_gpu) restricted to
 * its FFN half (:3528-3580). */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_stack_decode(lumen_moe_ctx* ctx, const lumen_moe_layer* const* layers,
                                          const float* const* d_gammas, int32_t n_layers,
                                          float* d_x, float eps, int32_t tokens, void* stream);

/* The same stack for a multi-token batch (any number of tokens): per layer
 * normed <- rmsnorm(x; gamma_l, eps), x <- x + MoE_l(normed), in place on d_x f32 [T,H];
 * d_normed is caller-owned scratch f32 [T,H]. The FFN half of the prefill layer loop,
 * cuda/backend_impl.rs:9150-9176 (normed -> encode_moe_ffn_prefill_grouped -> x). */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_stack_prefill(lumen_moe_ctx* ctx, const lumen_moe_layer* const* layers,
                                           const float* const* d_gammas, int32_t n_layers, float* d_x,
                                           float* d_normed, float eps, int32_t tokens, void* stream);

/* Device check of the library's exp used by the router (see exact_expf.h). */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_debug_expf(const float* d_in, float* d_out, int64_t n, void* stream);

/* Instrumentation: re-launch ONE kernel of the most recent lumen_moe_decode call
 * on `layer` with the routing tables that call left in the context (phase 0 =
 * router, 1 = gate/up + SwiGLU, 2 = down + combine), so that a benchmark can time
 * a single kernel with CUDA events. No counterpart in the reference (its
 * profiler brackets whole stages, cuda/profiler.rs:1-80). */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_debug_decode_phase(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                              int32_t phase, void* stream);

/* Re-runs the most recent decode call through the fused persistent kernel (batches
 * of 1..4 tokens) and records, per CTA, globaltimer stamps (ns): 0 entry, 1 after the
 * wait on the previous kernel, 2 logits done, 3 barrier 1 passed, 4 routing done,
 * 5 gate/up done, 6 barrier 2 passed, 7 SwiGLU fragments staged, 8 down products
 * done, 9 end, 10 weight tiles requested (predicted expert set), 11 last staged
 * gate/up tile arrived. d_trace: [SM count][12] uint64 on the device, zeroed by the
 * caller.
 * LUMEN_MOE_UNSUPPORTED when the call's shape takes the three-kernel chain. */
LUMEN_MOE_API lumen_moe_status_t lumen_moe_debug_decode_trace(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                              uint64_t* d_trace, void* stream);

/* Bytes of device memory held by a prepared layer (repacked planes + tables). */
LUMEN_MOE_API size_t lumen_moe_layer_bytes(const lumen_moe_layer* layer);

/* Number of kernel launches issued by this library since the counter was last
 * read with reset != 0 (benchmark bookkeeping). */
LUMEN_MOE_API int64_t lumen_moe_launch_count(int32_t reset);

LUMEN_MOE_API const char* lumen_moe_last_error(void);
LUMEN_MOE_API const char* lumen_moe_version(void);

#ifdef __cplusplus
}
#endif
#endif /* LUMEN_MOE_H */
