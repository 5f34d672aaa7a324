// extern "C" boundary (include/lumen_moe.h): argument checks, handle
// management and error text; all work is delegated to the host layer.
#include "../../include/lumen_moe.h"
#include "host_moe.hpp"
#include <new>

namespace lumen {
long long read_launch_count(bool reset);
cudaError_t launch_scatter_accum(const __half* d16, const float* residual, const RouteDev& R, float* out, int T, int H,
                                 int K, cudaStream_t st);
}

struct lumen_moe_ctx {
    lumen::CudaMoeScratch scratch;
    lumen::EpState* ep = nullptr;  // expert-parallel state (lumen_moe_ep_create), or null
};
struct lumen_moe_layer {
    lumen::MoeLayer layer;
};

static thread_local std::string g_last_error;

namespace lumen {
// lets other translation units of the library report through lumen_moe_last_error()
void set_last_error(const std::string& msg) { g_last_error = msg; }
}  // namespace lumen

static lumen_moe_status_t fail(int code, const std::string& msg) {
    g_last_error = msg;
    return static_cast<lumen_moe_status_t>(code);
}
static lumen_moe_status_t done(const lumen::Status& s) {
    if (s.ok()) return LUMEN_MOE_OK;
    return fail(s.code, s.msg);
}

extern "C" {

const char* lumen_moe_last_error(void) { return g_last_error.c_str(); }
const char* lumen_moe_version(void) { return "lumen-moe-b200 0.1 (sm_100a)"; }

lumen_moe_status_t lumen_moe_create(const lumen_moe_config* cfg, lumen_moe_ctx** out_ctx) {
    if (!cfg || !out_ctx) return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
        return fail(LUMEN_MOE_CUDA_ERROR, "no CUDA device available; this library has no CPU path");
    if (cfg->device < 0 || cfg->device >= ndev) return fail(LUMEN_MOE_INVALID_ARG, "device ordinal out of range");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, cfg->device) != cudaSuccess)
        return fail(LUMEN_MOE_CUDA_ERROR, "cudaGetDeviceProperties failed");
    if (prop.major != 10)
        return fail(LUMEN_MOE_UNSUPPORTED, "this build contains sm_100a code only (Blackwell B200 required)");
    lumen_moe_ctx* ctx = new (std::nothrow) lumen_moe_ctx();
    if (!ctx) return fail(LUMEN_MOE_CUDA_ERROR, "out of host memory");
    if (cfg->flags & ~(0xf | 0xff00)) {
        delete ctx;
        return fail(LUMEN_MOE_INVALID_ARG, "unknown bits in lumen_moe_config.flags");
    }
    lumen::Status s = lumen::allocate_moe_scratch(cfg->device, cfg->hidden_dim, cfg->inter_dim, cfg->num_experts,
                                                  cfg->top_k, cfg->gating_mode, cfg->max_tokens, cfg->flags,
                                                  &ctx->scratch);
    if (!s.ok()) {
        delete ctx;
        return done(s);
    }
    *out_ctx = ctx;
    return LUMEN_MOE_OK;
}

void lumen_moe_destroy(lumen_moe_ctx* ctx) {
    if (!ctx) return;
    lumen::ep_free(ctx->ep);
    lumen::free_moe_scratch(&ctx->scratch);
    delete ctx;
}

lumen_moe_status_t lumen_moe_ensure_prefill(lumen_moe_ctx* ctx, int32_t tokens) {
    if (!ctx) return fail(LUMEN_MOE_INVALID_ARG, "null context");
    return done(lumen::ensure_prefill_grouped(&ctx->scratch, tokens));
}

lumen_moe_status_t lumen_moe_layer_prepare(lumen_moe_ctx* ctx, const void* d_layer_blob, size_t blob_bytes,
                                           uint64_t router_off, const uint64_t* gate_offs, const uint64_t* up_offs,
                                           const uint64_t* down_offs, int32_t quant, void* stream,
                                           lumen_moe_layer** out_layer) {
    if (!ctx || !d_layer_blob || !out_layer) return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    const lumen::CudaMoeScratch& sc = ctx->scratch;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    {
        int cur = -1;
        if (cudaGetDevice(&cur) != cudaSuccess || cur != sc.device)
            return fail(LUMEN_MOE_INVALID_ARG, "the context belongs to another CUDA device than the current one");
        cudaPointerAttributes pa;
        if (cudaPointerGetAttributes(&pa, d_layer_blob) != cudaSuccess || pa.type != cudaMemoryTypeDevice ||
            pa.device != sc.device)
            return fail(LUMEN_MOE_INVALID_ARG, "the layer blob is not device memory of the context's GPU");
    }
    if (!gate_offs && !up_offs && !down_offs) {
        // router-only layer: nothing is repacked; usable with lumen_moe_route_only
        if (router_off % 4 != 0 || router_off + (uint64_t)sc.E * sc.H * 4 > blob_bytes)
            return fail(LUMEN_MOE_INVALID_ARG, "router weight misaligned or outside the layer blob");
        lumen_moe_layer* r = new (std::nothrow) lumen_moe_layer();
        if (!r) return fail(LUMEN_MOE_CUDA_ERROR, "out of host memory");
        r->layer.dev.blob = static_cast<const uint8_t*>(d_layer_blob);
        {
            lumen::Status rs = lumen::aligned_router(d_layer_blob, router_off, sc.E, sc.H, st, &r->layer.repacked,
                                                     &r->layer.dev.router_w);
            if (rs.ok())
                rs = lumen::build_router_w16(r->layer.dev.router_w, sc.E, sc.H, st, &r->layer.repacked,
                                             &r->layer.dev.router_w16);
            if (rs.ok() && cudaStreamSynchronize(st) != cudaSuccess) rs = lumen::Status::Err(LUMEN_MOE_CUDA_ERROR, "copy of the router weight failed");
            if (!rs.ok()) {
                lumen::free_moe_layer(&r->layer);
                delete r;
                return fail(static_cast<lumen_moe_status_t>(rs.code), rs.msg);
            }
        }
        r->layer.dev.H = sc.H;
        r->layer.dev.I = sc.I;
        r->layer.dev.E = sc.E;
        r->layer.dev.quant = -1;
        r->layer.blob_bytes = blob_bytes;
        *out_layer = r;
        return LUMEN_MOE_OK;
    }
    if (!gate_offs || !up_offs || !down_offs) return fail(LUMEN_MOE_INVALID_ARG, "null offset table");
    if (quant < 0 || quant > 2) return fail(LUMEN_MOE_UNSUPPORTED, "unsupported quant scheme");
    lumen::SubtensorOffsets sub;
    sub.has_router = true;
    sub.router_weight.offset = router_off;
    sub.router_weight.length = (uint64_t)sc.E * sc.H * 4;
    sub.experts.resize(sc.E);
    for (int e = 0; e < sc.E; ++e) {
        sub.experts[e].gate.offset = gate_offs[e];
        sub.experts[e].up.offset = up_offs[e];
        sub.experts[e].down.offset = down_offs[e];
        sub.experts[e].gate.quant = sub.experts[e].up.quant = sub.experts[e].down.quant = quant;
    }
    lumen_moe_layer* l = new (std::nothrow) lumen_moe_layer();
    if (!l) return fail(LUMEN_MOE_CUDA_ERROR, "out of host memory");
    bool is_moe = false;
    lumen::Status s = lumen::build_moe_meta(sub, &l->layer.meta, &is_moe);
    if (s.ok() && !is_moe) s = lumen::Status::Err(LUMEN_MOE_INVALID_ARG, "layer has no experts");
    if (s.ok()) s = lumen::build_batched_offsets(l->layer.meta, st, &l->layer.offsets);
    if (s.ok())
        s = lumen::build_repacked(sc, d_layer_blob, blob_bytes, l->layer.meta, l->layer.offsets, sc.H, sc.I, sc.E, st,
                                  &l->layer.repacked, &l->layer.dev);
    if (s.ok()) {
        cudaError_t e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) s = lumen::Status::Err(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    }
    if (!s.ok()) {
        lumen::free_moe_layer(&l->layer);
        delete l;
        return done(s);
    }
    l->layer.blob_bytes = blob_bytes;
    *out_layer = l;
    return LUMEN_MOE_OK;
}

void lumen_moe_layer_destroy(lumen_moe_layer* layer) {
    if (!layer) return;
    lumen::free_moe_layer(&layer->layer);
    delete layer;
}

size_t lumen_moe_layer_bytes(const lumen_moe_layer* layer) {
    if (!layer) return 0;
    const size_t router_copy = layer->layer.repacked.router_copy ? (size_t)layer->layer.dev.E * layer->layer.dev.H * sizeof(float) : 0;
    const size_t router_w16 = layer->layer.repacked.router_w16 ? (size_t)2 * layer->layer.dev.E * layer->layer.dev.H * 2 : 0;
    const size_t f16w = layer->layer.repacked.gu16 ? (size_t)layer->layer.dev.E * 3 * layer->layer.dev.I * layer->layer.dev.H * 2 : 0;
    return layer->layer.repacked.q_bytes + layer->layer.repacked.s_bytes + router_copy + router_w16 + f16w +
           5 * sizeof(uint64_t) * layer->layer.dev.E;
}

lumen_moe_status_t lumen_moe_decode(lumen_moe_ctx* ctx, const lumen_moe_layer* layer, const float* d_normed,
                                    const float* d_residual, float* d_out, int32_t tokens, void* stream) {
    if (!ctx || !layer) return fail(LUMEN_MOE_INVALID_ARG, "null handle");
    return done(lumen::encode_moe_ffn_decode(&ctx->scratch, layer->layer, d_normed, d_residual, d_out, tokens,
                                             static_cast<cudaStream_t>(stream)));
}

static bool is_shared_ctx(const lumen_moe_ctx* ctx) {
    return ctx->scratch.E == 1 && ctx->scratch.K == 1 && (ctx->scratch.gating == 2 || ctx->scratch.gating == 3);
}

lumen_moe_status_t lumen_moe_shared_expert_decode(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                  const float* d_normed, float* d_out, int32_t tokens,
                                                  void* stream) {
    if (!ctx || !layer) return fail(LUMEN_MOE_INVALID_ARG, "null context or layer");
    if (!is_shared_ctx(ctx))
        return fail(LUMEN_MOE_INVALID_ARG, "not a shared-expert context (num_experts = top_k = 1, gating_mode 2 or 3)");
    return lumen_moe_decode(ctx, layer, d_normed, d_out, d_out, tokens, stream);
}

lumen_moe_status_t lumen_moe_shared_expert_prefill(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                   const void* d_normed, float* d_out, int32_t tokens,
                                                   int32_t act_dtype, void* stream) {
    if (!ctx || !layer) return fail(LUMEN_MOE_INVALID_ARG, "null context or layer");
    if (!is_shared_ctx(ctx))
        return fail(LUMEN_MOE_INVALID_ARG, "not a shared-expert context (num_experts = top_k = 1, gating_mode 2 or 3)");
    return lumen_moe_prefill(ctx, layer, d_normed, d_out, d_out, tokens, act_dtype, stream);
}

lumen_moe_status_t lumen_moe_decode_fused_norm(lumen_moe_ctx* ctx, const lumen_moe_layer* layer, const float* d_x,
                                               const float* d_gamma, float* d_normed_out, float* d_out, float eps,
                                               int32_t tokens, void* stream) {
    if (!ctx || !layer) return fail(LUMEN_MOE_INVALID_ARG, "null handle");
    return done(lumen::encode_moe_ffn_decode_fused_norm(&ctx->scratch, layer->layer, d_x, d_gamma, d_normed_out, d_out,
                                                        eps, tokens, static_cast<cudaStream_t>(stream)));
}

lumen_moe_status_t lumen_moe_prefill(lumen_moe_ctx* ctx, const lumen_moe_layer* layer, const void* d_normed,
                                     const float* d_residual, float* d_out, int32_t tokens, int32_t act_dtype,
                                     void* stream) {
    if (!ctx || !layer) return fail(LUMEN_MOE_INVALID_ARG, "null handle");
    return done(lumen::encode_moe_ffn_prefill_grouped(&ctx->scratch, layer->layer, d_normed, act_dtype, d_residual,
                                                      d_out, tokens, static_cast<cudaStream_t>(stream)));
}

lumen_moe_status_t lumen_moe_prefill_routed(lumen_moe_ctx* ctx, const lumen_moe_layer* layer, const void* d_normed,
                                            const uint32_t* d_ids, const float* d_weights, const float* d_residual,
                                            float* d_out, int32_t tokens, int32_t act_dtype, void* stream) {
    if (!ctx || !layer || !d_ids) return fail(LUMEN_MOE_INVALID_ARG, "null handle or ids");
    return done(lumen::encode_moe_ffn_prefill_grouped(&ctx->scratch, layer->layer, d_normed, act_dtype, d_residual,
                                                      d_out, tokens, static_cast<cudaStream_t>(stream), d_ids,
                                                      d_weights));
}

lumen_moe_status_t lumen_moe_experts_routed_f16(lumen_moe_ctx* ctx, const lumen_moe_layer* layer, const void* d_rows,
                                                const uint32_t* d_ids, void* d_out16, int32_t rows, int32_t act_dtype,
                                                void* stream) {
    if (!ctx || !layer || !d_ids || !d_out16) return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    return done(lumen::encode_moe_ffn_prefill_grouped(&ctx->scratch, layer->layer, d_rows, act_dtype, nullptr, nullptr,
                                                      rows, static_cast<cudaStream_t>(stream), d_ids, nullptr,
                                                      static_cast<__half*>(d_out16)));
}

lumen_moe_status_t lumen_moe_combine_f16(const void* d_d16, const float* d_residual, const float* d_weights,
                                         const int32_t* d_dst_to_col, float* d_out, int32_t tokens, int32_t hidden_dim,
                                         int32_t top_k, void* stream) {
    if (!d_d16 || !d_residual || !d_weights || !d_dst_to_col || !d_out || tokens < 1 || hidden_dim < 2 || hidden_dim % 2 ||
        top_k < 1)
        return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    lumen::RouteDev R{};
    R.weights = const_cast<float*>(d_weights);
    R.dst_to_col = const_cast<int32_t*>(d_dst_to_col);
    cudaError_t e = lumen::launch_scatter_accum(static_cast<const __half*>(d_d16), d_residual, R, d_out, tokens,
                                                hidden_dim, top_k, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_route_only(lumen_moe_ctx* ctx, const lumen_moe_layer* layer, const float* d_normed,
                                        int32_t tokens, uint32_t* d_ids, float* d_weights, float* d_logits_out,
                                        void* stream) {
    if (!ctx || !layer || !d_normed) return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    return done(lumen::encode_route_only(&ctx->scratch, &layer->layer, d_normed, nullptr, tokens, d_ids, d_weights,
                                         d_logits_out, static_cast<cudaStream_t>(stream)));
}

lumen_moe_status_t lumen_moe_topk_from_logits(lumen_moe_ctx* ctx, const float* d_logits, int32_t tokens,
                                              uint32_t* d_ids, float* d_weights, void* stream) {
    if (!ctx || !d_logits) return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    return done(lumen::encode_route_only(&ctx->scratch, nullptr, nullptr, d_logits, tokens, d_ids, d_weights, nullptr,
                                         static_cast<cudaStream_t>(stream)));
}

lumen_moe_status_t lumen_moe_set_logits_override(lumen_moe_ctx* ctx, const float* d_logits) {
    if (!ctx) return fail(LUMEN_MOE_INVALID_ARG, "null context");
    ctx->scratch.logits_override = d_logits;
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_get_routing(lumen_moe_ctx* ctx, int32_t tokens, uint32_t* ids, float* weights,
                                         int32_t* dst_to_col, int32_t* col_src_tok, int32_t* expert_bounds,
                                         void* stream) {
    if (!ctx) return fail(LUMEN_MOE_INVALID_ARG, "null context");
    const lumen::CudaMoeScratch& s = ctx->scratch;
    if (tokens < 1 || tokens > s.cap_tokens) return fail(LUMEN_MOE_INVALID_ARG, "tokens exceeds the last call's capacity");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t C = (size_t)tokens * s.K;
    cudaError_t e = cudaStreamSynchronize(st);
    if (e == cudaSuccess && ids) e = cudaMemcpy(ids, s.R.ids, C * 4, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && weights) e = cudaMemcpy(weights, s.R.weights, C * 4, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && dst_to_col) e = cudaMemcpy(dst_to_col, s.R.dst_to_col, C * 4, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && col_src_tok) e = cudaMemcpy(col_src_tok, s.R.col_src_tok, C * 4, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && expert_bounds)
        e = cudaMemcpy(expert_bounds, s.R.expert_bounds, (size_t)(s.E + 1) * 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    // the stream is idle: the host copy of the status word is final for everything enqueued so far
    lumen::Status st_word = lumen::check_status_word(&s);
    if (!st_word.ok()) {
        lumen::Status c = lumen::clear_status_word(&ctx->scratch, st);
        if (!c.ok()) return done(c);
        return done(st_word);
    }
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_get_routing_ids_stride_e(lumen_moe_ctx* ctx, int32_t tokens, uint32_t* ids_stride_e,
                                                      void* stream) {
    if (!ctx || !ids_stride_e) return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    const lumen::CudaMoeScratch& s = ctx->scratch;
    if (tokens < 1 || tokens > s.cap_tokens) return fail(LUMEN_MOE_INVALID_ARG, "tokens exceeds the last call's capacity");
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    // ids live with row stride K on the device: widen on the way out (a strided 2-D copy)
    if (e == cudaSuccess) {
        for (size_t i = 0; i < (size_t)tokens * s.E; ++i) ids_stride_e[i] = 0u;
        e = cudaMemcpy2D(ids_stride_e, (size_t)s.E * 4, s.R.ids, (size_t)s.K * 4, (size_t)s.K * 4, (size_t)tokens,
                         cudaMemcpyDeviceToHost);
    }
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_poll_status(const lumen_moe_ctx* ctx) {
    if (!ctx) return fail(LUMEN_MOE_INVALID_ARG, "null context");
    return done(lumen::check_status_word(&ctx->scratch));
}

lumen_moe_status_t lumen_moe_clear_status(lumen_moe_ctx* ctx, void* stream) {
    if (!ctx) return fail(LUMEN_MOE_INVALID_ARG, "null context");
    return done(lumen::clear_status_word(&ctx->scratch, static_cast<cudaStream_t>(stream)));
}

lumen_moe_status_t lumen_moe_debug_expire_next_wait(lumen_moe_ctx* ctx, int32_t which) {
    if (!ctx || which < 0 || which > 1) return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    if (ctx->scratch.wait_limit_us == 0)
        return fail(LUMEN_MOE_INVALID_ARG, "create the context with LUMEN_MOE_FLAG_SHORT_WAITS for this test hook");
    ctx->scratch.expire_next[which] = 1;
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_get_routing_device(lumen_moe_ctx* ctx, int32_t tokens, int32_t* d_dst_to_col,
                                                int32_t* d_col_src_tok, int32_t* d_col_expert,
                                                int32_t* d_expert_bounds, void* stream) {
    if (!ctx) return fail(LUMEN_MOE_INVALID_ARG, "null context");
    const lumen::CudaMoeScratch& s = ctx->scratch;
    if (tokens < 1 || tokens > s.cap_tokens) return fail(LUMEN_MOE_INVALID_ARG, "tokens exceeds the last call's capacity");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t C = (size_t)tokens * s.K;
    cudaError_t e = cudaSuccess;
    if (d_dst_to_col) e = cudaMemcpyAsync(d_dst_to_col, s.R.dst_to_col, C * 4, cudaMemcpyDeviceToDevice, st);
    if (e == cudaSuccess && d_col_src_tok) e = cudaMemcpyAsync(d_col_src_tok, s.R.col_src_tok, C * 4, cudaMemcpyDeviceToDevice, st);
    if (e == cudaSuccess && d_col_expert) e = cudaMemcpyAsync(d_col_expert, s.R.col_expert, C * 4, cudaMemcpyDeviceToDevice, st);
    if (e == cudaSuccess && d_expert_bounds)
        e = cudaMemcpyAsync(d_expert_bounds, s.R.expert_bounds, (size_t)(s.E + 1) * 4, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_ep_prepare(lumen_moe_ctx* ctx, const void* d_normed, int32_t act_dtype, int32_t tokens,
                                        int32_t experts_per_rank, void* d_rows16, int32_t* d_local_ids,
                                        int64_t* d_send_counts, void* stream) {
    if (!ctx || !d_normed || !d_rows16 || !d_local_ids || !d_send_counts)
        return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    const lumen::CudaMoeScratch& s = ctx->scratch;
    if (tokens < 1 || tokens > s.cap_tokens) return fail(LUMEN_MOE_INVALID_ARG, "tokens exceeds the last call's capacity");
    if (experts_per_rank < 1 || s.E % experts_per_rank != 0)
        return fail(LUMEN_MOE_INVALID_ARG, "experts_per_rank must divide num_experts");
    if (s.H % 8 != 0) return fail(LUMEN_MOE_UNSUPPORTED, "hidden_dim must be a multiple of 8");
    if (act_dtype != 0 && act_dtype != 1) return fail(LUMEN_MOE_INVALID_ARG, "unknown activation dtype");
    cudaError_t e = lumen::launch_ep_prepare(d_normed, act_dtype, s.R, tokens * s.K, s.H, s.E, experts_per_rank, d_rows16,
                                             d_local_ids, reinterpret_cast<long long*>(d_send_counts),
                                             static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_quantize(const float* d_src, int64_t n_elements, int32_t quant, void* d_dst,
                                      void* stream) {
    if (!d_src || !d_dst) return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    if (n_elements <= 0 || n_elements % 32) return fail(LUMEN_MOE_INVALID_ARG, "n_elements must be a positive multiple of 32");
    if (quant < 0 || quant > 2) return fail(LUMEN_MOE_UNSUPPORTED, "unsupported quant scheme");
    cudaError_t e = lumen::launch_quantize(d_src, n_elements, quant, d_dst, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_rmsnorm(const float* d_x, const float* d_gamma, float* d_out, int32_t tokens,
                                     int32_t hidden_dim, float eps, void* stream) {
    if (!d_x || !d_gamma || !d_out || tokens < 1 || hidden_dim < 1) return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    cudaError_t e = lumen::launch_rmsnorm(d_x, d_gamma, d_out, tokens, hidden_dim, eps, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_stack_decode(lumen_moe_ctx* ctx, const lumen_moe_layer* const* layers,
                                          const float* const* d_gammas, int32_t n_layers, float* d_x, float eps,
                                          int32_t tokens, void* stream) {
    if (!ctx || !layers || !d_gammas || !d_x || n_layers < 1) return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int l = 0; l < n_layers; ++l) {
        if (!layers[l] || !d_gammas[l]) return fail(LUMEN_MOE_INVALID_ARG, "null layer or gamma");
        // x <- x + MoE(rmsnorm(x)); residual and output are the same buffer (cuda/backend_impl.rs:3570-3573)
        lumen::Status s = lumen::encode_moe_ffn_decode_fused_norm(&ctx->scratch, layers[l]->layer, d_x, d_gammas[l],
                                                                  nullptr, d_x, eps, tokens, st);
        if (!s.ok()) return done(s);
    }
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_stack_prefill(lumen_moe_ctx* ctx, const lumen_moe_layer* const* layers,
                                           const float* const* d_gammas, int32_t n_layers, float* d_x, float* d_normed,
                                           float eps, int32_t tokens, void* stream) {
    if (!ctx || !layers || !d_gammas || !d_x || !d_normed || n_layers < 1 || tokens < 1)
        return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int l = 0; l < n_layers; ++l) {
        if (!layers[l] || !d_gammas[l]) return fail(LUMEN_MOE_INVALID_ARG, "null layer or gamma");
        cudaError_t e = lumen::launch_rmsnorm(d_x, d_gammas[l], d_normed, tokens, ctx->scratch.H, eps, st);
        if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
        // residual and output are the same buffer: the combine reads and writes each element in one thread
        lumen::Status s = lumen::encode_moe_ffn_prefill_grouped(&ctx->scratch, layers[l]->layer, d_normed, 0, d_x, d_x,
                                                                tokens, st, nullptr, nullptr, nullptr);
        if (!s.ok()) return done(s);
    }
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_debug_expf(const float* d_in, float* d_out, int64_t n, void* stream) {
    if (!d_in || !d_out || n <= 0) return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    cudaError_t e = lumen::launch_debug_expf(d_in, d_out, n, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_debug_decode_phase(lumen_moe_ctx* ctx, const lumen_moe_layer* layer, int32_t phase,
                                                void* stream) {
    if (!ctx || !layer || phase < 0 || phase > 2) return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    if (!ctx->scratch.has_last_decode) return fail(LUMEN_MOE_INVALID_ARG, "no decode call has been made yet");
    lumen::DecodeArgs a = ctx->scratch.last_decode;
    a.L = layer->layer.dev;
    cudaError_t e = lumen::launch_decode_phase(a, phase, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_debug_decode_trace(lumen_moe_ctx* ctx, const lumen_moe_layer* layer,
                                                uint64_t* d_trace, void* stream) {
    if (!ctx || !layer) return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    if (!ctx->scratch.has_last_decode) return fail(LUMEN_MOE_INVALID_ARG, "no decode call has been made yet");
    lumen::DecodeArgs a = ctx->scratch.last_decode;
    a.L = layer->layer.dev;
    a.trace = reinterpret_cast<unsigned long long*>(d_trace);
    if (!lumen::decode_fused_applicable(a)) return fail(LUMEN_MOE_UNSUPPORTED, "the fused decode kernel does not apply to this call");
    cudaError_t e = lumen::launch_decode_fused(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_ep_create(lumen_moe_ctx* ctx, int32_t rank, int32_t world, int32_t max_tokens,
                                       int32_t recv_rows, void* handle_out) {
    if (!ctx || !handle_out) return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    if (ctx->ep) return fail(LUMEN_MOE_INVALID_ARG, "the context already has an expert-parallel window");
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != ctx->scratch.device)
        return fail(LUMEN_MOE_INVALID_ARG, "the context belongs to another CUDA device than the current one");
    return done(lumen::ep_create(&ctx->scratch, rank, world, max_tokens, recv_rows, &ctx->ep, handle_out));
}

lumen_moe_status_t lumen_moe_ep_attach(lumen_moe_ctx* ctx, const void* handles, int32_t rank, int32_t world) {
    if (!ctx || !handles) return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    if (!ctx->ep) return fail(LUMEN_MOE_INVALID_ARG, "call lumen_moe_ep_create first");
    if (rank != lumen::ep_rank(ctx->ep) || world != lumen::ep_world(ctx->ep))
        return fail(LUMEN_MOE_INVALID_ARG, "rank / world differ from lumen_moe_ep_create");
    return done(lumen::ep_attach(ctx->ep, handles));
}

lumen_moe_status_t lumen_moe_ep_layer_prepare(lumen_moe_ctx* ctx, const void* d_layer_blob, size_t blob_bytes,
                                              uint64_t router_off, const uint64_t* gate_offs, const uint64_t* up_offs,
                                              const uint64_t* down_offs, int32_t quant, void* stream,
                                              lumen_moe_layer** out_layer) {
    if (!ctx || !d_layer_blob || !out_layer || !gate_offs || !up_offs || !down_offs)
        return fail(LUMEN_MOE_INVALID_ARG, "null argument");
    if (!ctx->ep) return fail(LUMEN_MOE_INVALID_ARG, "call lumen_moe_ep_create first");
    if (quant < 0 || quant > 2) return fail(LUMEN_MOE_UNSUPPORTED, "unsupported quant scheme");
    const lumen::CudaMoeScratch& sc = ctx->scratch;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != sc.device)
        return fail(LUMEN_MOE_INVALID_ARG, "the context belongs to another CUDA device than the current one");
    if (router_off % 4 != 0 || router_off + (uint64_t)sc.E * sc.H * 4 > blob_bytes)
        return fail(LUMEN_MOE_INVALID_ARG, "router weight misaligned or outside the layer blob");
    const int epr = lumen::ep_experts_per_rank(ctx->ep), first = lumen::ep_rank(ctx->ep) * epr;
    lumen_moe_layer* l = new (std::nothrow) lumen_moe_layer();
    if (!l) return fail(LUMEN_MOE_CUDA_ERROR, "out of host memory");
    lumen::CudaMoeMeta& m = l->layer.meta;
    m.router_weight_off = router_off;
    m.expert_gate_offs.assign(gate_offs + first, gate_offs + first + epr);
    m.expert_up_offs.assign(up_offs + first, up_offs + first + epr);
    m.expert_down_offs.assign(down_offs + first, down_offs + first + epr);
    m.expert_gate_quant = m.expert_down_quant = quant;
    lumen::Status s = lumen::build_batched_offsets(m, st, &l->layer.offsets);
    if (s.ok())
        s = lumen::build_repacked(sc, d_layer_blob, blob_bytes, m, l->layer.offsets, sc.H, sc.I, epr, st,
                                  &l->layer.repacked, &l->layer.dev);
    if (s.ok()) {
        // what build_repacked made of the router covers this rank's experts only: the router needs all E rows
        cudaStreamSynchronize(st);
        if (l->layer.repacked.router_copy) cudaFree(l->layer.repacked.router_copy);
        if (l->layer.repacked.router_w16) cudaFree(l->layer.repacked.router_w16);
        l->layer.repacked.router_copy = nullptr;
        l->layer.repacked.router_w16 = nullptr;
        s = lumen::aligned_router(d_layer_blob, router_off, sc.E, sc.H, st, &l->layer.repacked, &l->layer.dev.router_w);
        if (s.ok())
            s = lumen::build_router_w16(l->layer.dev.router_w, sc.E, sc.H, st, &l->layer.repacked, &l->layer.dev.router_w16);
    }
    if (s.ok()) {
        cudaError_t e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) s = lumen::Status::Err(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
    }
    if (!s.ok()) {
        lumen::free_moe_layer(&l->layer);
        delete l;
        return done(s);
    }
    l->layer.blob_bytes = blob_bytes;
    *out_layer = l;
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_prefill_ep(lumen_moe_ctx* ctx, const lumen_moe_layer* layer, const void* d_normed,
                                        const float* d_residual, float* d_out, int32_t tokens, int32_t act_dtype,
                                        void* stream) {
    if (!ctx || !layer) return fail(LUMEN_MOE_INVALID_ARG, "null handle");
    if (!ctx->ep) return fail(LUMEN_MOE_INVALID_ARG, "call lumen_moe_ep_create and lumen_moe_ep_attach first");
    return done(lumen::encode_moe_ffn_prefill_ep(&ctx->scratch, ctx->ep, layer->layer, d_normed, act_dtype, d_residual,
                                                 d_out, tokens, static_cast<cudaStream_t>(stream)));
}

lumen_moe_status_t lumen_moe_ep_profile(lumen_moe_ctx* ctx, int32_t enable) {
    if (!ctx || !ctx->ep) return fail(LUMEN_MOE_INVALID_ARG, "no expert-parallel window on this context");
    lumen::ep_set_profile(ctx->ep, enable != 0);
    return LUMEN_MOE_OK;
}

lumen_moe_status_t lumen_moe_ep_phase_ms(lumen_moe_ctx* ctx, float* out_ms6) {
    if (!ctx || !ctx->ep || !out_ms6) return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    return done(lumen::ep_phase_ms(ctx->ep, out_ms6));
}

lumen_moe_status_t lumen_moe_stack_prefill_ep(lumen_moe_ctx* ctx, const lumen_moe_layer* const* layers,
                                              const float* const* d_gammas, int32_t n_layers, float* d_x,
                                              float* d_normed, float eps, int32_t tokens, void* stream) {
    if (!ctx || !layers || !d_gammas || !d_x || !d_normed || n_layers < 1 || tokens < 1)
        return fail(LUMEN_MOE_INVALID_ARG, "bad argument");
    if (!ctx->ep) return fail(LUMEN_MOE_INVALID_ARG, "call lumen_moe_ep_create and lumen_moe_ep_attach first");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int l = 0; l < n_layers; ++l) {
        if (!layers[l] || !d_gammas[l]) return fail(LUMEN_MOE_INVALID_ARG, "null layer or gamma");
        cudaError_t e = lumen::launch_rmsnorm(d_x, d_gammas[l], d_normed, tokens, ctx->scratch.H, eps, st);
        if (e != cudaSuccess) return fail(LUMEN_MOE_CUDA_ERROR, cudaGetErrorString(e));
        lumen::Status s = lumen::encode_moe_ffn_prefill_ep(&ctx->scratch, ctx->ep, layers[l]->layer, d_normed, 0, d_x, d_x,
                                                           tokens, st);
        if (!s.ok()) return done(s);
    }
    return LUMEN_MOE_OK;
}

int64_t lumen_moe_launch_count(int32_t reset) { return lumen::read_launch_count(reset != 0); }

}  // extern "C"
