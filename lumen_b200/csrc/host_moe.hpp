// Host layer of the MoE operator. The functions mirror, name for name, the
// crate-internal interface of the reference's CUDA backend
// (crates/lumen-runtime/src/cuda/moe.rs) so that a call site there maps one to
// one onto a call here; the extern "C" functions of include/lumen_moe.h are thin
// wrappers around them.
//
//   reference (cuda/moe.rs)                     here
//   build_moe_meta                    :223      lumen::build_moe_meta
//   build_batched_offsets             :272      lumen::build_batched_offsets
//   build_repacked_down               :337      lumen::build_repacked
//   allocate_moe_scratch              :968      lumen::allocate_moe_scratch
//   ensure_prefill_grouped            :1015     lumen::ensure_prefill_grouped
//   encode_moe_ffn_decode             :1119     lumen::encode_moe_ffn_decode
//   encode_moe_ffn_decode_fused_norm  :3184     lumen::encode_moe_ffn_decode_fused_norm
//   encode_moe_ffn_prefill_grouped    :1900     lumen::encode_moe_ffn_prefill_grouped
//
// Error behaviour follows the reference: every function returns a status
// (Result<_, RuntimeError>), validation happens on the host before any launch
// (router offset alignment and bounds, cuda/moe.rs:1258-1271; scratch capacity,
// :1497-1502; quant combinations, :1185-1191), nothing synchronises the stream on
// the hot path.
#pragma once
#include <string>
#include <vector>
#include "moe_internal.cuh"

namespace lumen {

struct Status {
    int code = 0;  // lumen_moe_status_t
    std::string msg;
    bool ok() const { return code == 0; }
    static Status Ok() { return Status(); }
    static Status Err(int c, std::string m) {
        Status s;
        s.code = c;
        s.msg = std::move(m);
        return s;
    }
};

// lumen_format::index::TensorSlice / ExpertSlice / SubtensorOffsets restricted to
// the fields this path reads (crates/lumen-format/src/index.rs).
struct TensorSlice {
    uint64_t offset = 0, length = 0;
    int quant = 0;
};
struct ExpertSlice {
    TensorSlice gate, up, down;
};
struct SubtensorOffsets {
    bool has_router = false;
    TensorSlice router_weight;
    std::vector<ExpertSlice> experts;
};

// CudaMoeMeta, cuda/moe.rs:39-59 (shared-expert fields are outside this path).
struct CudaMoeMeta {
    uint64_t router_weight_off = 0;
    std::vector<uint64_t> expert_gate_offs, expert_up_offs, expert_down_offs;
    int expert_gate_quant = 0, expert_down_quant = 0;
};

// CudaMoeBatchedOffsets, cuda/moe.rs:70-76: device u64 tables. The reference
// interleaves gate/up as [g0,u0,g1,u1,...]; the same table is built here and the
// repack kernels index it with a stride of two.
struct CudaMoeBatchedOffsets {
    uint64_t* gate_up_offsets = nullptr;  // [2E]
    uint64_t* down_offsets = nullptr;     // [E]
    uint64_t* gate_offsets = nullptr;     // [E] (de-interleaved copies for the repack kernels)
    uint64_t* up_offsets = nullptr;       // [E]
};

// CudaMoeRepacked, cuda/moe.rs:89-97: aligned planes built once per layer.
struct CudaMoeRepacked {
    uint4* q = nullptr;
    uint4* s = nullptr;
    size_t q_bytes = 0, s_bytes = 0;
    // 16-byte-aligned copy of the router weight, made only when the blob holds it at an
    // address the vector loads cannot take (a file's layer blob aligns tensors to 4 bytes)
    float* router_copy = nullptr;
    __half* router_w16 = nullptr;  // f16 high / low planes of the router weight for the batched tcgen05 router
    __half* gu16 = nullptr;        // plain f16 expert matrices for the TMA-fed prefill products (see LayerDev)
    __half* dn16 = nullptr;
};

// Router weight pointer for the kernels: in place when 16-byte aligned in device memory,
// else a copy owned by `out` (enqueued on `st`).
Status aligned_router(const void* layer_buf, uint64_t router_off, int E, int H, cudaStream_t st,
                      CudaMoeRepacked* out, const float** router_w);
Status build_router_w16(const float* router_w, int E, int H, cudaStream_t st, CudaMoeRepacked* out, const __half** w16);

// CudaMoeScratch + CudaMoePrefillGrouped, cuda/moe.rs:101-210.
struct CudaMoeScratch {
    int device = 0;
    int H = 0, I = 0, E = 0, K = 0, gating = 0;
    int cap_tokens = 0;  // capacity of the token-sized buffers below
    RouteDev R{};
    uint4* xf = nullptr;    // decode activation fragments
    unsigned* xq = nullptr; // decode activations as two-term int8 blocks (Q4_0 gate/up of the three-kernel chain)
    unsigned* sq = nullptr; // SwiGLU outputs of a 5..16-token Q4_0 decode in the same form, per compact column
    uint4* sf = nullptr;    // decode SwiGLU fragments
    float* s_f32 = nullptr; // optional debug copy
    // prefill (grow-only)
    int32_t* blk_hist = nullptr;
    __half* w16 = nullptr;
    __half* s16 = nullptr;
    __half* d16 = nullptr;
    __half* x16 = nullptr;  // permuted 16-bit activations for the tcgen05 path
    __half* xr16 = nullptr; // f16 high / low planes of the batch for the tcgen05 router
    float* rpart = nullptr; // partial logits of the tcgen05 router
    int32_t* any_lo = nullptr;
    int4* tiles = nullptr;
    int32_t* n_tiles = nullptr;
    unsigned int* tile_counter = nullptr;
    int32_t* status = nullptr;
    int32_t* h_status = nullptr;       // pinned host word the kernels mirror the status code into
    int32_t* status_host = nullptr;    // device-side address of h_status
    int flags = 0;                     // lumen_moe_config.flags
    unsigned wait_limit_us = 0;        // 0 = the kernels' defaults (1-2 s); 2000 with LUMEN_MOE_FLAG_SHORT_WAITS
    int tc_ctas = 0;                   // cap of the persistent tcgen05 grid (0 = every SM)
    int sms = 0;                       // multiprocessors of the device
    int expire_next[2] = {0, 0};       // test hook (lumen_moe_debug_expire_next_wait): one-shot per kernel kind
    const float* logits_override = nullptr;
    DecodeArgs last_decode{};   // arguments of the most recent decode call (instrumentation)
    bool has_last_decode = false;
    int prefill_impl = 0;
    int decode_impl = 0;            // 0 = fused persistent kernel where it applies, 1 = three-kernel chain
    unsigned int* bar = nullptr;    // grid barrier words of the fused decode kernel
    void* arena = nullptr;       // one allocation for the fixed-size part
    void* arena_tok = nullptr;   // one allocation for the token-sized part
    size_t arena_tok_bytes = 0;
};

struct MoeLayer {
    CudaMoeMeta meta;
    CudaMoeBatchedOffsets offsets;
    CudaMoeRepacked repacked;
    LayerDev dev{};
    size_t blob_bytes = 0;
};

Status build_moe_meta(const SubtensorOffsets& subtensors, CudaMoeMeta* out, bool* is_moe);
Status build_batched_offsets(const CudaMoeMeta& meta, cudaStream_t st, CudaMoeBatchedOffsets* out);
Status build_repacked(const CudaMoeScratch& scratch, const void* layer_buf, size_t blob_bytes,
                      const CudaMoeMeta& meta, const CudaMoeBatchedOffsets& offs, int H, int I, int E,
                      cudaStream_t st, CudaMoeRepacked* out, LayerDev* dev);
Status allocate_moe_scratch(int device, int H, int expert_I, int E, int K, int gating, int max_tokens, int flags,
                            CudaMoeScratch* out);
// LUMEN_MOE_TIMEOUT / LUMEN_MOE_INVALID_ARG once a kernel of this context has given up (host read, no sync)
Status check_status_word(const CudaMoeScratch* scratch);
Status clear_status_word(CudaMoeScratch* scratch, cudaStream_t st);
Status ensure_prefill_grouped(CudaMoeScratch* scratch, int batch);
void free_moe_scratch(CudaMoeScratch* scratch);
void free_moe_layer(MoeLayer* layer);

Status encode_moe_ffn_decode(CudaMoeScratch* scratch, const MoeLayer& layer, const float* normed_x,
                             const float* residual, float* output_x, int tokens, cudaStream_t st);
Status encode_moe_ffn_decode_fused_norm(CudaMoeScratch* scratch, const MoeLayer& layer,
                                        const float* attn_proj, const float* ffn_norm, float* normed_x,
                                        float* output_x, float eps, int tokens, cudaStream_t st);
Status encode_moe_ffn_prefill_grouped(CudaMoeScratch* scratch, const MoeLayer& layer, const void* normed,
                                      int act_dtype, const float* residual, float* output, int batch,
                                      cudaStream_t st, const uint32_t* ids_in = nullptr,
                                      const float* weights_in = nullptr, __half* out16_rows = nullptr);
Status encode_route_only(CudaMoeScratch* scratch, const MoeLayer* layer, const float* normed,
                         const float* logits_in, int tokens, uint32_t* d_ids, float* d_weights,
                         float* d_logits_out, cudaStream_t st);


// Expert-parallel prefill (ep_push.cu): per-rank state behind lumen_moe_ep_create / _attach.
struct EpState;
Status ep_create(CudaMoeScratch* scratch, int rank, int world, int max_tokens, int recv_rows, EpState** out,
                 void* handle64);
Status ep_attach(EpState* ep, const void* handles64);
void ep_free(EpState* ep);
int ep_rank(const EpState* ep);
int ep_world(const EpState* ep);
int ep_experts_per_rank(const EpState* ep);
size_t ep_window_bytes(const EpState* ep);
void ep_set_profile(EpState* ep, bool on);
Status ep_phase_ms(EpState* ep, float* out6);
Status encode_moe_ffn_prefill_ep(CudaMoeScratch* scratch, EpState* ep, const MoeLayer& layer, const void* normed,
                                 int act_dtype, const float* residual, float* output, int batch, cudaStream_t st);

}  // namespace lumen
