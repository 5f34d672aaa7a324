// Host layer: validation, layer preparation, scratch management and the
// sequencing of the kernels (see host_moe.hpp for the map onto the reference's
// cuda/moe.rs functions).
#include "host_moe.hpp"
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace lumen {

cudaError_t launch_grouped_mma(const DecodeArgs& a, __half* d16, cudaStream_t st);
cudaError_t launch_scatter_accum(const __half* d16, const float* residual, const RouteDev& R, float* out,
                                 int T, int H, int K, cudaStream_t st);
cudaError_t launch_build_xf(const void* x, int act_dtype, int T, int H, int nblk_pad, bool bf16_mode,
                            uint4* xf, cudaStream_t st);
cudaError_t launch_gather_permute_x16(const void* x, int act_dtype, const int32_t* col_src_tok, int C, int H, void* out,
                                      cudaStream_t st, bool natural);
cudaError_t launch_grouped_tc(const PrefillArgs& p, const void* x16, int grid, cudaStream_t st, __half* out16_rows,
                              const TcPlan* plan = nullptr, const TcPeerOut* peer = nullptr);
cudaError_t launch_rows_from_cols(const __half* d16, const int32_t* dst_to_col, __half* out16, int T, int H, cudaStream_t st);

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches += n; }
long long read_launch_count(bool reset) { return reset ? g_launches.exchange(0) : g_launches.load(); }

#define CUDA_TRY(expr)                                                                              \
    do {                                                                                            \
        cudaError_t _e = (expr);                                                                    \
        if (_e != cudaSuccess)                                                                      \
            return Status::Err(3, std::string(#expr) + ": " + cudaGetErrorString(_e));              \
    } while (0)

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static size_t row_bytes(int in_dim, int quant) {
    if (quant == Q8_0) return (size_t)(in_dim / 32) * 34;
    if (quant == Q4_0) return (size_t)(in_dim / 32) * 18;
    return (size_t)in_dim * 2;
}

// cuda/moe.rs:223-260
Status build_moe_meta(const SubtensorOffsets& st, CudaMoeMeta* out, bool* is_moe) {
    *is_moe = false;
    if (!st.has_router || st.experts.empty()) return Status::Ok();  // not an MoE layer (reference returns None)
    CudaMoeMeta m;
    m.router_weight_off = st.router_weight.offset;
    for (const auto& e : st.experts) {
        m.expert_gate_offs.push_back(e.gate.offset);
        m.expert_up_offs.push_back(e.up.offset);
        m.expert_down_offs.push_back(e.down.offset);
    }
    m.expert_gate_quant = st.experts[0].gate.quant;
    m.expert_down_quant = st.experts[0].down.quant;
    *out = std::move(m);
    *is_moe = true;
    return Status::Ok();
}

// cuda/moe.rs:272-296
Status build_batched_offsets(const CudaMoeMeta& meta, cudaStream_t st, CudaMoeBatchedOffsets* out) {
    const size_t E = meta.expert_gate_offs.size();
    if (meta.expert_up_offs.size() != E || meta.expert_down_offs.size() != E)
        return Status::Err(1, "build_batched_offsets: offset tables differ in length");
    std::vector<uint64_t> gu(2 * E);
    for (size_t i = 0; i < E; ++i) {
        gu[2 * i] = meta.expert_gate_offs[i];
        gu[2 * i + 1] = meta.expert_up_offs[i];
    }
    uint64_t* base = nullptr;
    CUDA_TRY(cudaMalloc(&base, sizeof(uint64_t) * 5 * E));
    out->gate_up_offsets = base;
    out->down_offsets = base + 2 * E;
    out->gate_offsets = base + 3 * E;
    out->up_offsets = base + 4 * E;
    CUDA_TRY(cudaMemcpyAsync(out->gate_up_offsets, gu.data(), sizeof(uint64_t) * 2 * E, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaMemcpyAsync(out->down_offsets, meta.expert_down_offs.data(), sizeof(uint64_t) * E, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaMemcpyAsync(out->gate_offsets, meta.expert_gate_offs.data(), sizeof(uint64_t) * E, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaMemcpyAsync(out->up_offsets, meta.expert_up_offs.data(), sizeof(uint64_t) * E, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaStreamSynchronize(st));  // the host vectors go out of scope
    return Status::Ok();
}

// cuda/moe.rs:337-394 (generalised to every quant and to gate/up/down)
Status build_repacked(const CudaMoeScratch& sc, const void* layer_buf, size_t blob_bytes, const CudaMoeMeta& meta,
                      const CudaMoeBatchedOffsets& offs, int H, int I, int E, cudaStream_t st,
                      CudaMoeRepacked* out, LayerDev* dev) {
    const int quant = meta.expert_gate_quant;
    // cuda/moe.rs:1185-1191: only (Q8_0,Q8_0), (Q4_0,Q4_0), (Bf16,Bf16)
    if (quant != meta.expert_down_quant || quant < 0 || quant > 2)
        return Status::Err(2, "unsupported expert quant combination (gate/down must both be Q8_0, Q4_0 or BF16)");
    if ((int)meta.expert_gate_offs.size() != E) return Status::Err(1, "expert count does not match the context");
    // cuda/moe.rs:1258-1271: router offset alignment and bounds
    if (meta.router_weight_off % 4 != 0) return Status::Err(1, "router weight offset is not 4-byte aligned");
    if (meta.router_weight_off + (uint64_t)E * H * 4 > blob_bytes)
        return Status::Err(1, "router weight exceeds the layer blob");
    const size_t gu_bytes = (size_t)I * row_bytes(H, quant), dn_bytes = (size_t)H * row_bytes(I, quant);
    for (int e = 0; e < E; ++e) {
        if (meta.expert_gate_offs[e] + gu_bytes > blob_bytes || meta.expert_up_offs[e] + gu_bytes > blob_bytes ||
            meta.expert_down_offs[e] + dn_bytes > blob_bytes)
            return Status::Err(1, "expert " + std::to_string(e) + " weight slice exceeds the layer blob");
    }
    LayerDev L{};
    L.blob = static_cast<const uint8_t*>(layer_buf);
    {
        Status rs = aligned_router(layer_buf, meta.router_weight_off, E, H, st, out, &L.router_w);
        if (rs.ok()) rs = build_router_w16(L.router_w, E, H, st, out, &L.router_w16);
        if (!rs.ok()) return rs;
    }
    L.quant = quant;
    L.H = H;
    L.I = I;
    L.E = E;
    L.kg_h = (H / 32 + 3) / 4;
    L.kg_i = (I / 32 + 3) / 4;
    L.rt_i = I / 16;
    L.rt_h = H / 16;
    L.nq = (quant == Q4_0) ? 2 : (quant == Q8_0) ? 4 : 8;
    L.q_gu = (size_t)L.rt_i * L.kg_h * L.nq * 32;
    L.q_dn = (size_t)L.rt_h * L.kg_i * L.nq * 32;
    L.q_exp = 2 * L.q_gu + L.q_dn;
    L.s_gu = (quant == BF16) ? 0 : (size_t)L.rt_i * L.kg_h * 8;
    L.s_dn = (quant == BF16) ? 0 : (size_t)L.rt_h * L.kg_i * 8;
    L.s_exp = 2 * L.s_gu + L.s_dn;
    out->q_bytes = L.q_exp * E * sizeof(uint4);
    out->s_bytes = L.s_exp * E * sizeof(uint4);
    CUDA_TRY(cudaMalloc(&out->q, out->q_bytes));
    if (out->s_bytes) CUDA_TRY(cudaMalloc(&out->s, out->s_bytes));
    L.q = out->q;
    L.s = out->s;
    CUDA_TRY(launch_repack(L.blob, offs.gate_offsets, offs.up_offsets, offs.down_offsets, L, out->q, out->s, st));
    // Plain f16 copies of the expert matrices: always for BF16 weights (there is nothing to
    // dequantise: TMA feeds the tensor cores directly, as it does the activations), and for
    // Q4_0 / Q8_0 when the context asks to trade memory for prefill speed
    // (LUMEN_MOE_FLAG_PREFILL_F16_WEIGHTS: 2 bytes per weight more per layer).
    if ((quant == BF16 || (sc.flags & 0x8)) && H % 256 == 0 && I % 128 == 0) {
        const size_t n = (size_t)E * 3 * I * H;
        CUDA_TRY(cudaMalloc(&out->gu16, (size_t)E * 2 * I * H * sizeof(__half)));
        CUDA_TRY(cudaMalloc(&out->dn16, (size_t)E * H * I * sizeof(__half)));
        (void)n;
        CUDA_TRY(launch_dequant_f16(L.blob, offs.gate_offsets, offs.up_offsets, offs.down_offsets, L, out->gu16, out->dn16, st));
        L.gu16 = out->gu16;
        L.dn16 = out->dn16;
    }
    *dev = L;
    return Status::Ok();
}

static size_t tok_arena_bytes(const CudaMoeScratch& s, int cap, size_t* offs) {
    // order: logits, ids, weights, col_expert, col_src_tok, dst_to_col, blk_hist, tiles, s16, d16, x16, xf, sf, w16, xq, xr16, rpart, sq
    const size_t C = (size_t)cap * s.K;
    const size_t nblk_h_pad = (size_t)((s.H / 32 + 3) / 4) * 4, nblk_i_pad = (size_t)((s.I / 32 + 3) / 4) * 4;
    const size_t max_ct = C / 128 + s.E, max_ct_dn = C / 128 + s.E;  // gate/up tiles of 128 or 256 columns (sized for 128), down tiles of 128
    const size_t n_tile_entries = max_ct * ((size_t)s.I / 128 + 1) + max_ct_dn * ((size_t)s.H / 256 + 1);
    size_t sizes[18] = {
        (size_t)cap * s.E * 4, C * 4, C * 4, C * 4, C * 4, C * 4,
        (size_t)((cap + 7) / 8) * s.E * 4,  // one histogram per chunk of 8 tokens (SORT_TOK in route_large.cu)
        n_tile_entries * sizeof(int4),
        C * s.I * 2, C * s.H * 2, C * s.H * 2,
        (size_t)cap * 2 * nblk_h_pad * 64, C * 2 * nblk_i_pad * 64,
        (size_t)s.E * s.H * 4,
        (size_t)DECODE_MAX_TOKENS * (18 * nblk_h_pad + 16) * 4,  // xq_tok_words(nblk_h_pad) words per token
        (size_t)cap * s.H * 2 * 2,
        (size_t)ROUTER_TC_MAX_KSPLIT * cap * s.E * 4,
        (size_t)DECODE_MAX_TOKENS * s.K * (18 * nblk_i_pad + 16) * 4};  // xq_tok_words(nblk_i_pad) words per decode column
    size_t off = 0;
    for (int i = 0; i < 18; ++i) {
        offs[i] = off;
        off += align_up(sizes[i], 256);
    }
    return off;
}

static Status alloc_tok_arena(CudaMoeScratch* s, int cap) {
    size_t offs[18];
    const size_t bytes = tok_arena_bytes(*s, cap, offs);
    void* p = nullptr;
    CUDA_TRY(cudaMalloc(&p, bytes));
    CUDA_TRY(cudaMemset(p, 0, bytes));  // fragment padding blocks must read as zero
    if (s->arena_tok) cudaFree(s->arena_tok);
    s->has_last_decode = false;  // its arguments pointed into the old arena
    s->arena_tok = p;
    s->arena_tok_bytes = bytes;
    s->cap_tokens = cap;
    uint8_t* b = static_cast<uint8_t*>(p);
    s->R.logits = reinterpret_cast<float*>(b + offs[0]);
    s->R.ids = reinterpret_cast<uint32_t*>(b + offs[1]);
    s->R.weights = reinterpret_cast<float*>(b + offs[2]);
    s->R.col_expert = reinterpret_cast<int32_t*>(b + offs[3]);
    s->R.col_src_tok = reinterpret_cast<int32_t*>(b + offs[4]);
    s->R.dst_to_col = reinterpret_cast<int32_t*>(b + offs[5]);
    s->blk_hist = reinterpret_cast<int32_t*>(b + offs[6]);
    s->tiles = reinterpret_cast<int4*>(b + offs[7]);
    s->s16 = reinterpret_cast<__half*>(b + offs[8]);
    s->d16 = reinterpret_cast<__half*>(b + offs[9]);
    s->x16 = reinterpret_cast<__half*>(b + offs[10]);
    s->xf = reinterpret_cast<uint4*>(b + offs[11]);
    s->sf = reinterpret_cast<uint4*>(b + offs[12]);
    s->w16 = reinterpret_cast<__half*>(b + offs[13]);
    s->xq = reinterpret_cast<unsigned*>(b + offs[14]);
    s->xr16 = reinterpret_cast<__half*>(b + offs[15]);
    s->rpart = reinterpret_cast<float*>(b + offs[16]);
    s->sq = reinterpret_cast<unsigned*>(b + offs[17]);
    return Status::Ok();
}

// cuda/moe.rs:968-1013
Status allocate_moe_scratch(int device, int H, int I, int E, int K, int gating, int max_tokens, int flags,
                            CudaMoeScratch* out) {
    if (H <= 0 || I <= 0 || H % 32 || I % 32) return Status::Err(1, "hidden_dim and inter_dim must be positive multiples of 32");
    if (E <= 0 || E > MAX_EXPERTS) return Status::Err(1, "num_experts must be in 1..256");
    if (K <= 0 || K > MAX_TOP_K || K > E) return Status::Err(1, "top_k must be in 1..16 and <= num_experts");
    if (gating < 0 || gating > 3) return Status::Err(1, "unknown gating mode");
    CUDA_TRY(cudaSetDevice(device));
    CudaMoeScratch s;
    s.device = device;
    s.H = H;
    s.I = I;
    s.E = E;
    s.K = K;
    s.gating = gating;
    const size_t fixed = align_up((size_t)(E + 1) * 4, 256) + align_up((size_t)E * 4, 256) + 256 * 4 +
                         (size_t)MAX_EXPERTS * 2 * sizeof(int4) + 1024 * 4;
    CUDA_TRY(cudaMalloc(&s.arena, fixed));
    CUDA_TRY(cudaMemset(s.arena, 0, fixed));
    uint8_t* b = static_cast<uint8_t*>(s.arena);
    s.R.expert_bounds = reinterpret_cast<int32_t*>(b);
    b += align_up((size_t)(E + 1) * 4, 256);
    s.R.uexp = reinterpret_cast<int32_t*>(b);
    b += align_up((size_t)E * 4, 256);
    s.R.n_uexp = reinterpret_cast<int32_t*>(b);
    s.R.ticket = reinterpret_cast<unsigned int*>(b + 256);
    s.n_tiles = reinterpret_cast<int32_t*>(b + 512);
    s.status = reinterpret_cast<int32_t*>(b + 768);
    s.any_lo = reinterpret_cast<int32_t*>(b + 772);
    s.R.work = reinterpret_cast<int4*>(b + 1024);
    s.bar = reinterpret_cast<unsigned int*>(b + 1024 + (size_t)MAX_EXPERTS * 2 * sizeof(int4));  // 1024 per-CTA flags
    s.flags = flags;
    s.decode_impl = (flags & 0x1) ? 1 : 0;   // LUMEN_MOE_FLAG_DECODE_SPLIT
    s.prefill_impl = (flags & 0x2) ? 1 : 0;  // LUMEN_MOE_FLAG_PREFILL_MMA
    s.wait_limit_us = (flags & 0x4) ? 2000u : 0u;  // LUMEN_MOE_FLAG_SHORT_WAITS
    s.tc_ctas = (flags >> 8) & 0xff;
    CUDA_TRY(cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, device));
    // the status word's host copy: kernels write it at most once per failure, the host reads it for free
    CUDA_TRY(cudaHostAlloc(&s.h_status, sizeof(int32_t), cudaHostAllocMapped));
    *s.h_status = 0;
    CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void**>(&s.status_host), s.h_status, 0));
    const int cap = max_tokens > DECODE_MAX_TOKENS ? max_tokens : DECODE_MAX_TOKENS;
    Status st = alloc_tok_arena(&s, cap);
    if (!st.ok()) {
        cudaFree(s.arena);
        cudaFreeHost(s.h_status);
        return st;
    }
    *out = s;
    return Status::Ok();
}

// cuda/moe.rs:1015-1100 (grow-only)
Status ensure_prefill_grouped(CudaMoeScratch* s, int batch) {
    if (batch <= s->cap_tokens) return Status::Ok();
    CUDA_TRY(cudaDeviceSynchronize());  // the old buffers may still be in use
    return alloc_tok_arena(s, batch);
}

Status check_status_word(const CudaMoeScratch* s) {
    const int code = s->h_status ? *reinterpret_cast<volatile int32_t*>(s->h_status) : 0;
    if (code == 0) return Status::Ok();
    if (code == 4)
        return Status::Err(4, "a device-side bounded wait expired in an earlier call on this context (grouped GEMM "
                              "pipeline or decode grid barrier); outputs since then are undefined; "
                              "lumen_moe_clear_status makes the context usable again");
    return Status::Err(code, "an earlier call on this context was given an expert id >= num_experts; "
                             "lumen_moe_clear_status makes the context usable again");
}

Status clear_status_word(CudaMoeScratch* s, cudaStream_t st) {
    CUDA_TRY(cudaStreamSynchronize(st));
    CUDA_TRY(cudaMemset(s->status, 0, 4));
    CUDA_TRY(cudaMemset(s->bar, 0, 1024 * 4));
    CUDA_TRY(cudaMemset(s->R.logits, 0, (size_t)s->cap_tokens * s->E * 4));  // tagged logit slots of the fused decode kernel
    CUDA_TRY(cudaDeviceSynchronize());
    *reinterpret_cast<volatile int32_t*>(s->h_status) = 0;
    return Status::Ok();
}

void free_moe_scratch(CudaMoeScratch* s) {
    if (s->h_status) cudaFreeHost(s->h_status);
    if (s->arena) cudaFree(s->arena);
    if (s->arena_tok) cudaFree(s->arena_tok);
    *s = CudaMoeScratch();
}

Status aligned_router(const void* layer_buf, uint64_t router_off, int E, int H, cudaStream_t st,
                      CudaMoeRepacked* out, const float** router_w) {
    const uint8_t* src = static_cast<const uint8_t*>(layer_buf) + router_off;
    if (reinterpret_cast<uintptr_t>(src) % 16 == 0) {
        *router_w = reinterpret_cast<const float*>(src);
        return Status::Ok();
    }
    const size_t bytes = (size_t)E * H * sizeof(float);
    CUDA_TRY(cudaMalloc(&out->router_copy, bytes));
    CUDA_TRY(cudaMemcpyAsync(out->router_copy, src, bytes, cudaMemcpyDeviceToDevice, st));
    *router_w = out->router_copy;
    return Status::Ok();
}

// f16 high / low planes of the router weight, once per layer (the batched router multiplies on tcgen05)
Status build_router_w16(const float* router_w, int E, int H, cudaStream_t st, CudaMoeRepacked* out, const __half** w16) {
    *w16 = nullptr;
    if (H % 64 != 0) return Status::Ok();  // the tcgen05 router does not take this shape
    CUDA_TRY(cudaMalloc(&out->router_w16, (size_t)2 * E * H * sizeof(__half)));
    CUDA_TRY(launch_split_router_w16(router_w, out->router_w16, E, H, st));
    *w16 = out->router_w16;
    return Status::Ok();
}

void free_moe_layer(MoeLayer* l) {
    if (l->repacked.router_copy) cudaFree(l->repacked.router_copy);
    if (l->repacked.router_w16) cudaFree(l->repacked.router_w16);
    if (l->repacked.gu16) cudaFree(l->repacked.gu16);
    if (l->repacked.dn16) cudaFree(l->repacked.dn16);
    if (l->offsets.gate_up_offsets) cudaFree(l->offsets.gate_up_offsets);
    if (l->repacked.q) cudaFree(l->repacked.q);
    if (l->repacked.s) cudaFree(l->repacked.s);
}

static Status check_device(const CudaMoeScratch* s) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != s->device)
        return Status::Err(1, "the context belongs to CUDA device " + std::to_string(s->device) +
                                  " but the calling thread's current device is " + std::to_string(cur));
    return Status::Ok();
}

static Status check_layer(const CudaMoeScratch* s, const MoeLayer& layer) {
    Status d = check_device(s);
    if (!d.ok()) return d;
    d = check_status_word(s);
    if (!d.ok()) return d;
    if (layer.dev.H != s->H || layer.dev.I != s->I || layer.dev.E != s->E)
        return Status::Err(1, "layer shape does not match the context");
    if (layer.dev.quant < 0) return Status::Err(1, "router-only layer: expert weights were not prepared");
    return Status::Ok();
}

static DecodeArgs make_decode_args(CudaMoeScratch* s, const MoeLayer& layer, int tokens) {
    DecodeArgs a{};
    a.L = layer.dev;
    a.R = s->R;
    a.xf = s->xf;
    a.xq = s->xq;
    a.sq = s->sq;
    a.sf = s->sf;
    a.s_f32 = nullptr;
    a.T = tokens;
    a.K = s->K;
    a.gating = s->gating;
    a.logits_override = s->logits_override;
    a.bar = (s->decode_impl == 0) ? s->bar : nullptr;
    a.status = s->status;
    a.status_host = s->status_host;
    a.wait_limit_us = s->wait_limit_us;
    a.debug_extra_arrivals = 0;
    a.trace = nullptr;
    return a;
}

// cuda/moe.rs:1119-1191
Status encode_moe_ffn_decode(CudaMoeScratch* s, const MoeLayer& layer, const float* normed_x, const float* residual,
                             float* output_x, int tokens, cudaStream_t st) {
    if (tokens < 1 || tokens > DECODE_MAX_TOKENS) return Status::Err(1, "decode handles 1..16 tokens; use prefill");
    if (!normed_x || !residual || !output_x) return Status::Err(1, "null activation pointer");
    if (normed_x == output_x) return Status::Err(1, "output must not alias the normed input");
    Status c = check_layer(s, layer);
    if (!c.ok()) return c;
    DecodeArgs a = make_decode_args(s, layer, tokens);
    a.x = normed_x;
    a.residual = residual;
    a.out = output_x;
    s->last_decode = a;
    s->has_last_decode = true;
    if (s->expire_next[0] && decode_uses_fused(a)) {
        a.debug_extra_arrivals = 1;
        s->expire_next[0] = 0;
    }
    CUDA_TRY(launch_decode(a, st));
    return Status::Ok();
}

// cuda/moe.rs:3184-3330
Status encode_moe_ffn_decode_fused_norm(CudaMoeScratch* s, const MoeLayer& layer, const float* attn_proj,
                                        const float* ffn_norm, float* normed_x, float* output_x, float eps,
                                        int tokens, cudaStream_t st) {
    if (tokens < 1 || tokens > DECODE_MAX_TOKENS) return Status::Err(1, "decode handles 1..16 tokens; use prefill");
    if (!attn_proj || !ffn_norm || !output_x) return Status::Err(1, "null activation pointer");
    Status c = check_layer(s, layer);
    if (!c.ok()) return c;
    DecodeArgs a = make_decode_args(s, layer, tokens);
    a.x = attn_proj;
    a.gamma = ffn_norm;
    a.normed_out = normed_x;
    a.eps = eps;
    a.residual = attn_proj;
    a.out = output_x;
    CUDA_TRY(launch_decode(a, st));
    return Status::Ok();
}

Status encode_route_only(CudaMoeScratch* s, const MoeLayer* layer, const float* normed, const float* logits_in,
                         int tokens, uint32_t* d_ids, float* d_weights, float* d_logits_out, cudaStream_t st) {
    if (tokens < 1) return Status::Err(1, "tokens must be positive");
    if (!logits_in && (!layer || !normed)) return Status::Err(1, "route_only needs a layer and activations");
    Status dv = check_device(s);
    if (!dv.ok()) return dv;
    dv = check_status_word(s);
    if (!dv.ok()) return dv;
    Status g = ensure_prefill_grouped(s, tokens);
    if (!g.ok()) return g;
    const size_t C = (size_t)tokens * s->K;
    if (tokens <= DECODE_MAX_TOKENS) {
        DecodeArgs a{};
        if (layer) a.L = layer->dev;
        a.L.H = s->H;
        a.L.E = s->E;
        a.R = s->R;
        a.x = normed;
        a.T = tokens;
        a.K = s->K;
        a.gating = s->gating;
        a.logits_override = logits_in;
        a.xf = nullptr;
        a.xq = nullptr;
        a.sq = nullptr;
        CUDA_TRY(launch_route_small(a, st));
    } else {
        PrefillArgs p{};
        if (layer) p.L = layer->dev;
        p.L.H = s->H;
        p.L.E = s->E;
        p.L.I = s->I;
        p.R = s->R;
        p.status = s->status;
        p.status_host = s->status_host;
        p.x = normed;
        p.act_dtype = 0;
        p.T = tokens;
        p.K = s->K;
        p.gating = s->gating;
        p.logits_override = logits_in;
        p.blk_hist = s->blk_hist;
        p.w16 = s->w16;
        p.xr16 = s->xr16;
        p.rpart = s->rpart;
        p.any_lo = s->any_lo;
        p.sms = s->sms;
        p.wait_limit_us = s->wait_limit_us;
        p.tiles = nullptr;
        p.n_tiles = s->n_tiles;
        CUDA_TRY(launch_route_large(p, st));
    }
    if (d_ids) CUDA_TRY(cudaMemcpyAsync(d_ids, s->R.ids, C * 4, cudaMemcpyDeviceToDevice, st));
    if (d_weights) CUDA_TRY(cudaMemcpyAsync(d_weights, s->R.weights, C * 4, cudaMemcpyDeviceToDevice, st));
    if (d_logits_out && !logits_in)
        CUDA_TRY(cudaMemcpyAsync(d_logits_out, s->R.logits, (size_t)tokens * s->E * 4, cudaMemcpyDeviceToDevice, st));
    return Status::Ok();
}

// cuda/moe.rs:1900-2760
Status encode_moe_ffn_prefill_grouped(CudaMoeScratch* s, const MoeLayer& layer, const void* normed, int act_dtype,
                                      const float* residual, float* output, int batch, cudaStream_t st,
                                      const uint32_t* ids_in, const float* weights_in, __half* out16_rows) {
    if (batch < 1) return Status::Err(1, "batch must be positive");
    if (out16_rows) {
        if (s->K != 1 || !ids_in) return Status::Err(1, "f16 row output needs top_k = 1 and caller-supplied ids");
        if (!normed) return Status::Err(1, "null activation pointer");
    } else if (!normed || !residual || !output) {
        return Status::Err(1, "null activation pointer");
    }
    if (act_dtype == 2 && !ids_in) return Status::Err(2, "f16 activations need caller-supplied routing");
    if (act_dtype < 0 || act_dtype > 2) return Status::Err(2, "activation dtype must be f32, bf16 or f16");
    Status c = check_layer(s, layer);
    if (!c.ok()) return c;
    Status g = ensure_prefill_grouped(s, batch);
    if (!g.ok()) return g;
    PrefillArgs p{};
    p.L = layer.dev;
    p.R = s->R;
    p.x = normed;
    p.act_dtype = act_dtype;
    p.residual = residual;
    p.out = output;
    p.logits_override = s->logits_override;
    p.ids_in = ids_in;
    p.weights_in = weights_in;
    p.T = batch;
    p.K = s->K;
    p.gating = s->gating;
    p.blk_hist = s->blk_hist;
    p.w16 = s->w16;
    p.xr16 = s->xr16;
    p.rpart = s->rpart;
    p.any_lo = s->any_lo;
    p.sms = s->sms;
    p.s16 = s->s16;
    p.d16 = s->d16;
    p.tiles = s->tiles;
    p.n_tiles = s->n_tiles;
    p.status = s->status;
    p.status_host = s->status_host;
    p.wait_limit_us = s->wait_limit_us;
    p.tc_ctas = s->tc_ctas;
    // the tcgen05 path reads activation rows with 16-byte loads (8-byte for 16-bit rows)
    // and stores f16 output rows 32 bytes at a time
    const bool tc_ok = (s->H % 256 == 0) && (s->I % 128 == 0) && (reinterpret_cast<uintptr_t>(normed) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(out16_rows) % 32 == 0);
    p.impl = (s->prefill_impl == 1 || !tc_ok) ? 1 : 0;
    CUDA_TRY(launch_route_large(p, st));
    const bool bf16_mode = (layer.dev.quant == BF16);
    if (p.impl == 0) {
        CUDA_TRY(launch_gather_permute_x16(normed, act_dtype, s->R.col_src_tok, batch * s->K, s->H, s->x16, st,
                                           layer.dev.gu16 != nullptr));
        // persistent grid, one CTA per SM; LUMEN_MOE_FLAG_TC_CTAS leaves some SMs to kernels that run beside it
        int sms = s->sms;
        if (s->tc_ctas > 0 && s->tc_ctas < sms) sms = s->tc_ctas;
        if (s->expire_next[1]) {
            p.debug_extra_tx = 1;
            s->expire_next[1] = 0;
        }
        CUDA_TRY(launch_grouped_tc(p, s->x16, sms, st, out16_rows));
    } else {
        CUDA_TRY(launch_build_xf(normed, act_dtype, batch, s->H, layer.dev.kg_h * 4, bf16_mode, s->xf, st));
        DecodeArgs a = make_decode_args(s, layer, batch);
        CUDA_TRY(launch_grouped_mma(a, s->d16, st));
    }
    if (out16_rows) {
        if (p.impl != 0) CUDA_TRY(launch_rows_from_cols(s->d16, s->R.dst_to_col, out16_rows, batch, s->H, st));
        return Status::Ok();
    }
    CUDA_TRY(launch_scatter_accum(s->d16, residual, s->R, output, batch, s->H, s->K, st));
    return Status::Ok();
}

}  // namespace lumen
