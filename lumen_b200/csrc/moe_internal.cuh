// Internal declarations shared by the kernels and the host layer of the MoE
// operator: device-side layouts, scratch buffers and launch prototypes.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>

namespace lumen {

enum Quant : int { Q8_0 = 0, Q4_0 = 1, BF16 = 2 };

constexpr int MAX_EXPERTS = 256;  // cuda/shaders/moe_router.cu:33
// Columns per tile of the tcgen05 gate/up product (the down tiles of a one-GPU call follow it): 256 once the
// experts average more than 128 columns (each dequantised weight tile then serves twice the
// columns), else 128 (fewer empty columns in ragged tiles, epilogue overlapped).
inline int tc_gu_tile_cols(int columns, int experts) { return (columns > 128 * experts) ? 256 : 128; }
constexpr int MAX_TOP_K = 16;     // cuda/shaders/moe_router.cu:34
constexpr int DECODE_MAX_TOKENS = 16;

// ---------------------------------------------------------------------------
// Repacked expert weights ("fragment planes").
//
// A matrix [R rows, Kdim] (rows = outputs, Kdim = inputs, 32-element blocks along
// Kdim) is cut into tiles of 16 rows x 4 blocks (128 inputs). Tile (rt, kg) is
// stored as NQ consecutive 512-byte vectors (one uint4 per lane of a warp), laid
// out so that lane (g = lane/4, t = lane%4) finds in its own uint4s exactly the
// words the m16n8k16 A fragment of rows {16rt+g, 16rt+g+8} needs:
//   Q4_0 (NQ=2): vector j holds blocks 2j, 2j+1 of the group:
//        {w(g,2j,t), w(g+8,2j,t), w(g,2j+1,t), w(g+8,2j+1,t)}, w(r,b,t) = 32-bit
//        word t of the block's 16 nibble bytes (elements 4t..4t+3 low nibbles,
//        16+4t..16+4t+3 high nibbles).
//   Q8_0 (NQ=4): vector b holds block b: {w(g,b,t), w(g,b,4+t), w(g+8,b,t), w(g+8,b,4+t)},
//        w(r,b,i) = 32-bit word i of the block's 32 int8 (elements 4i..4i+3).
//   BF16 (NQ=8): vector 2b+r holds, for row g+8r, the 8 bf16 elements
//        {4t..4t+3, 16+4t..16+4t+3} of block b.
// Scales (Q4_0/Q8_0): per tile 8 uint4, one per g: f16 {row g: blocks 0..3, row g+8: blocks 0..3}.
// Blocks past Kdim inside the last group are zero (scale 0).
// ---------------------------------------------------------------------------
struct LayerDev {
    const uint8_t* blob;
    const float* router_w;  // blob + router_off, [E,H] f32
    const __half* router_w16;  // [2][E][H] f16 high / low parts of router_w (batched router on tcgen05), or null
    const uint4* q;         // all experts' quant planes
    const uint4* s;         // all experts' scale planes (unused for BF16)
    // optional plain f16 matrices of all experts (scale folded in) for the TMA-fed prefill products:
    // gu16 [E][2 I rows: gate then up][H], dn16 [E][H rows][I]; null = dequantise in shared memory
    const __half* gu16;
    const __half* dn16;
    int quant, H, I, E;
    int kg_h, kg_i;  // 128-input groups along H (gate/up) and I (down)
    int rt_i, rt_h;  // 16-row tiles of gate/up (I rows) and down (H rows)
    int nq;          // uint4 per lane per tile
    size_t q_gu, q_dn, q_exp;  // uint4 counts: one gate (or up) matrix, one down matrix, one expert
    size_t s_gu, s_dn, s_exp;

    __host__ __device__ const uint4* gate_q(int e) const { return q + (size_t)e * q_exp; }
    __host__ __device__ const uint4* up_q(int e) const { return q + (size_t)e * q_exp + q_gu; }
    __host__ __device__ const uint4* down_q(int e) const { return q + (size_t)e * q_exp + 2 * q_gu; }
    __host__ __device__ const uint4* gate_s(int e) const { return s + (size_t)e * s_exp; }
    __host__ __device__ const uint4* up_s(int e) const { return s + (size_t)e * s_exp + s_gu; }
    __host__ __device__ const uint4* down_s(int e) const { return s + (size_t)e * s_exp + 2 * s_gu; }
};

// Routing tables of one call (device pointers into the context's scratch).
struct RouteDev {
    float* logits;         // [T,E]
    uint32_t* ids;         // [T,K] selection order
    float* weights;        // [T,K]
    int32_t* expert_bounds;  // [E+1]
    int32_t* col_expert;   // [C]
    int32_t* col_src_tok;  // [C]
    int32_t* dst_to_col;   // [C] indexed t*K+slot
    int32_t* uexp;         // [E] distinct experts, ascending
    int32_t* n_uexp;       // [1]
    unsigned int* ticket;  // [1] last-block election counter (zero between launches)
    int4* work;            // [2*E] decode work descriptors: {expert | -1, first column, columns, 0}, {tok0..tok3}
};

// Activation fragments: for token (or compact column) c, half hl (0 = high part,
// 1 = low part of the f32 value split into two f16), block b, t in 0..3: one uint4
//   {pack(v[4t],v[4t+2]), pack(v[4t+1],v[4t+3]), pack(v[16+4t],v[16+4t+2]), pack(v[16+4t+1],v[16+4t+3])}
// i.e. the m16n8k16 B fragments (b0,b1) of the low-nibble MMA then of the
// high-nibble MMA of that block. Index: ((c*2 + hl)*nblk_pad + b)*4 + t.
struct DecodeArgs {
    LayerDev L;
    RouteDev R;
    const float* x;         // normed [T,H] (or raw x when gamma != null)
    const float* gamma;     // fused FFN norm weight or null
    float* normed_out;      // optional normed output when gamma != null
    float eps;
    const float* residual;  // [T,H]
    float* out;             // [T,H]
    const float* logits_override;  // [T,E] or null
    uint4* xf;              // activation fragments [T][2][kg_h*4][4]
    unsigned* xq;           // two-term int8 activations [T][xq_tok_words] of the three-kernel chain's Q4_0 gate/up (null = f16 fragments in xf)
    unsigned* sq;           // two-term int8 SwiGLU outputs [C][xq_tok_words(kg_i*4)]: down operand of the 5..16-token Q4_0 chain (null = f16 fragments in sf)
    uint4* sf;              // SwiGLU fragments     [C][2][kg_i*4][4]
    float* s_f32;           // optional [C,I] f32 copy of the SwiGLU output (null = skip)
    int T, K, gating;
    unsigned int* bar;      // grid barrier of the fused kernel: arrival counter + per-CTA barrier counts (1024 words); null = three-kernel chain
    int32_t* status;        // context status word (non-zero after a bounded wait expired)
    int32_t* status_host;   // the same code for the host: a word of mapped pinned host memory (null = none)
    unsigned wait_limit_us; // limit of every device-side wait of this launch (0 = one second)
    int debug_extra_arrivals;  // test hook: the grid barrier expects this many arrivals more than there are CTAs
    unsigned long long* trace;  // optional [grid][12] globaltimer stamps of the fused kernel's phases (null = off)
};

#ifdef __CUDACC__
// A kernel that gives up records why: the first code wins; the host copy is written once.
__device__ __forceinline__ void raise_status(int32_t* status, int32_t* status_host, int code) {
    if (atomicCAS(status, 0, code) == 0 && status_host != nullptr) {
        *reinterpret_cast<volatile int32_t*>(status_host) = code;
        __threadfence_system();
    }
}

// Programmatic dependent launch for the chains of small kernels around the grouped products. A
// kernel launched with launch_dep() may be scheduled while the kernel before it in the stream
// is still running; it calls grid_dep_sync() as its first statement (every thread, before any
// early return, before touching anything an earlier kernel wrote): that returns once the
// preceding kernel has completed and its writes are visible, so the order of the stream is
// kept, and because every kernel of a chain does so, completion of one implies completion of
// all before it. What overlaps is the launch itself and whatever the kernel does before the call.
__device__ __forceinline__ void grid_dep_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dep(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

// launchers (kernels.cu files)
cudaError_t launch_repack(const uint8_t* blob, const uint64_t* d_gate_offs, const uint64_t* d_up_offs,
                          const uint64_t* d_down_offs, const LayerDev& L, uint4* q, uint4* s,
                          cudaStream_t st);
cudaError_t launch_dequant_f16(const uint8_t* blob, const uint64_t* d_gate_offs, const uint64_t* d_up_offs,
                               const uint64_t* d_down_offs, const LayerDev& L, __half* gu16, __half* dn16,
                               cudaStream_t st);
cudaError_t launch_decode(const DecodeArgs& a, cudaStream_t st);
cudaError_t launch_ep_prepare(const void* x, int act_dtype, const RouteDev& R, int C, int H, int E, int epr, void* rows,
                              int32_t* local_ids, long long* send_counts, cudaStream_t st);
cudaError_t launch_route_small(const DecodeArgs& a, cudaStream_t st);  // router + tables only (T <= 16)
bool decode_fused_applicable(const DecodeArgs& a);
bool decode_uses_fused(const DecodeArgs& a);  // whether launch_decode takes the fused kernel for this call
cudaError_t launch_decode_fused(const DecodeArgs& a, cudaStream_t st);
cudaError_t launch_decode_phase(const DecodeArgs& a, int phase, cudaStream_t st);  // one kernel of the three-kernel chain: 0 router, 1 gate/up, 2 down
cudaError_t launch_quantize(const float* src, int64_t n, int quant, void* dst, cudaStream_t st);
cudaError_t launch_rmsnorm(const float* x, const float* gamma, float* out, int T, int H, float eps,
                           cudaStream_t st);
cudaError_t launch_debug_expf(const float* in, float* out, int64_t n, cudaStream_t st);

// prefill path
struct PrefillArgs {
    LayerDev L;
    RouteDev R;
    const void* x;          // normed [T,H], f32 or bf16
    int act_dtype;          // 0 f32, 1 bf16
    const float* residual;
    float* out;
    const float* logits_override;
    int T, K, gating;
    // scratch
    int32_t* blk_hist;      // [nchunks, E]
    __half* w16;            // [2, E, H] router weight split into f16 high and low planes (per call, when the layer has none)
    __half* xr16;           // [2, T, H] activations split into f16 high and low planes (tcgen05 router)
    float* rpart;           // [ksplit, T, E] partial logits of the tcgen05 router
    int32_t* any_lo;        // [1] some low part of the activations is non-zero
    int sms;                // multiprocessors of the device
    __half* s16;            // [C, I] f16 SwiGLU output, row-major by compact column
    __half* d16;            // [C, H] f16 down output by compact column
    int4* tiles;            // tile list for the grouped GEMMs
    int32_t* n_tiles;       // [4]: gate/up tiles, down tiles, and the two kernels' tile counters
    unsigned int* tile_counter;  // [2] dynamic tile scheduler counters
    int32_t* status;        // [1] device-side error flag (bounded waits, invalid caller-supplied ids)
    int32_t* status_host;   // the same code in mapped pinned host memory (null = none)
    unsigned wait_limit_us; // limit of the device-side waits (0 = two seconds)
    int debug_extra_tx;     // test hook: the first stage barrier expects this many bytes more than arrive
    int tc_ctas;            // cap of the persistent tcgen05 grid (0 = every SM)
    int impl;               // 0 = tcgen05 path, 1 = mma.sync grouped fallback
    const uint32_t* ids_in;  // caller-supplied routing [T,K] (null = route here)
    const float* weights_in; // [T,K] or null (= 1)
};
cudaError_t launch_route_large(const PrefillArgs& a, cudaStream_t st);
// tcgen05 router (route_tc.cu)
cudaError_t launch_split_router_w16(const float* w, __half* w16, int E, int H, cudaStream_t st);
int router_tc_ksplit(int T, int E, int H, int sms);
bool router_tc_applicable(int T, int E, int H, const void* x);
cudaError_t launch_router_logits_tc(const void* x, int act_dtype, const __half* w16, int T, int E, int H, int ksplit,
                                    __half* x16, int32_t* any_lo, float* part, int32_t* status, int32_t* status_host,
                                    unsigned wait_limit_us, cudaStream_t st);
constexpr int ROUTER_TC_MAX_KSPLIT = 4;

// Expert-parallel form of the grouped products: the rows of the activation operand are not this
// rank's T*K compact columns but whatever the peers pushed into its receive window, and the down
// product's output rows go back to the ranks they came from.
constexpr int MAX_EP_RANKS = 16;
struct TcPeerOut {
    const int32_t* ret_map;        // [rows] (source rank << 24) | row in that rank's return buffer; null = off
    __half* base[MAX_EP_RANKS];    // every rank's return buffer [rows_cap, H] f16 as mapped into this process
    int world;
    int rows_cap;                  // rows of a return buffer: indices are checked against it
};
struct TcPlan {
    int rows;      // rows of the activation operand = capacity the tile lists were laid out for
    int gu_cols;   // columns per gate/up tile the tile lists were built with (128 or 256)
};
// tile lists {expert, col_start, ncols, m_tile} of both grouped GEMMs from per-expert column counts
// left in R.expert_bounds[0..E) (turned into bounds in place), plus R.uexp / R.n_uexp
cudaError_t launch_tile_plan(const RouteDev& R, int E, int H, int I, int rows_cap, int gu_cols, int4* tiles,
                             int32_t* n_tiles, cudaStream_t st);
cudaError_t launch_prefill(const PrefillArgs& a, cudaStream_t st);

void count_launch(int n = 1);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the CURRENT device only, and one
// process may own contexts on several GPUs: the opt-in is remembered per device ordinal
// (`cache` is a function-local static of the launcher, one per kernel instantiation).
struct SmemOptIn {
    size_t bytes[64] = {};
};
template <typename Kern>
inline cudaError_t ensure_dyn_smem(Kern kern, size_t bytes, SmemOptIn& cache) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (bytes <= cache.bytes[device & 63]) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) cache.bytes[device & 63] = bytes;
    return e;
}

}  // namespace lumen
