// lumen_moe_route_small_static: routing (gating, top-k, renormalisation and the
// stable counting sort) for 1..16 tokens WITHOUT a context and WITHOUT any device
// allocation.
//
// Who needs this. The regular routing entry points work out of a lumen_moe_ctx,
// and creating a context calls cudaMalloc. Some hosts cannot do that: a serving
// process that claims all of its device memory once at start-up and hands it out
// from its own pool (so nothing is left for the driver allocator, or any later
// cudaMalloc is a policy violation), and a latency-critical decode loop in which
// cudaMalloc/cudaFree are off limits because they synchronise the whole device
// and stall every other stream of the process. Such a caller owns its input and
// output buffers already; what it lacks is a place for the kernel's working
// tables. Here those tables live in a fixed array inside the library image.
//
// The working memory. `g_route_scratch` below is a file-scope __device__ array of
// ROUTE_SCRATCH_BYTES (8 KiB). Every GPU on which this library's module gets
// loaded carries its own copy from load time until the process exits. The limits
// it imposes are stated in the header and checked at run time: at most 16 tokens,
// 256 experts and top-16 (the array has room for exactly that case).
//
// Host code must not hand the array's NAME to a kernel: on the host that name is
// only a handle for the runtime's symbol table, not a device address. The device
// address is looked up with cudaGetSymbolAddress, once per device, with that
// device current, and cached. The first call on a device does this look-up; make
// that first call during start-up, before any stream capture is begun.
//
// Sharing. All calls on one GPU use the same 8 KiB and find in it whatever the
// previous call left there. The per-expert counters must start at zero, so every
// call clears them on its stream before the kernel runs. Two calls whose kernels
// overlap on the GPU (different streams, or different host threads) would
// trample each other's tables: callers must serialise them.
//
// This entry point never calls cudaMalloc, cudaFree, or any library routine that
// allocates (no torch, no cudaMallocAsync, no context creation).
#include "../../include/lumen_moe.h"
#include "moe_internal.cuh"
#include "router.cuh"
#include <mutex>
#include <string>

namespace lumen {

constexpr int RS_MAX_T = 16, RS_MAX_E = 256, RS_MAX_K = 16;
constexpr int RS_MAX_C = RS_MAX_T * RS_MAX_K;
// layout (int32 words): counts[E] | bounds[E+1] (padded to E+64) | col_src_tok[C] | dst_to_col[C] | ids[C]
constexpr int RS_OFF_COUNTS = 0;
constexpr int RS_OFF_BOUNDS = RS_OFF_COUNTS + RS_MAX_E;
constexpr int RS_OFF_SRC = RS_OFF_BOUNDS + RS_MAX_E + 64;
constexpr int RS_OFF_D2C = RS_OFF_SRC + RS_MAX_C;
constexpr int RS_OFF_IDS = RS_OFF_D2C + RS_MAX_C;
constexpr int RS_WORDS = RS_OFF_IDS + RS_MAX_C;
constexpr size_t ROUTE_SCRATCH_BYTES = 8192;
static_assert(RS_WORDS * 4 <= ROUTE_SCRATCH_BYTES, "scratch layout exceeds the static array");

static __device__ __align__(256) unsigned char g_route_scratch[ROUTE_SCRATCH_BYTES];

// One CTA. Same arithmetic as the last-CTA section of router_small_kernel (decode.cu):
// warp_topk per token, then the stable counting sort of (token, slot) pairs by expert.
// `scratch` is the device address of g_route_scratch; the counts region arrives zeroed.
__global__ void __launch_bounds__(256)
route_small_static_kernel(const float* __restrict__ logits, int T, int E, int K, int gating,
                          uint32_t* __restrict__ ids_out, float* __restrict__ w_out,
                          int32_t* __restrict__ scratch) {
    __shared__ __align__(16) float p_s[8][MAX_EXPERTS];
    __shared__ __align__(16) float lg_s[8][MAX_EXPERTS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int32_t* counts = scratch + RS_OFF_COUNTS;
    int32_t* bounds = scratch + RS_OFF_BOUNDS;
    int32_t* col_src_tok = scratch + RS_OFF_SRC;
    int32_t* dst_to_col = scratch + RS_OFF_D2C;
    int32_t* ids_g = scratch + RS_OFF_IDS;
    for (int t = warp; t < T; t += 8) {
        for (int i = lane; i < E; i += 32) lg_s[warp][i] = logits[(size_t)t * E + i];
        __syncwarp();
        warp_topk(lg_s[warp], E, K, gating, p_s[warp], nullptr, ids_out + (size_t)t * K, w_out + (size_t)t * K);
        if (lane < K) {
            const int e = (int)ids_out[(size_t)t * K + lane];
            ids_g[t * K + lane] = e;
            atomicAdd(&counts[e], 1);  // counts start at zero: cleared by the host before the launch
        }
    }
    __threadfence_block();
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            bounds[e] = run;
            run += counts[e];
        }
        bounds[E] = run;
    }
    __syncthreads();
    const int C = T * K;
    if (tid < E) {
        int cur = bounds[tid];
        for (int p = 0; p < C; ++p) {
            if (ids_g[p] == tid) {
                col_src_tok[cur] = p / K;
                dst_to_col[p] = cur;
                ++cur;
            }
        }
    }
}

static std::mutex g_setup_mutex;
static void* g_scratch_addr[64] = {nullptr};

// Device address of g_route_scratch on the current device (looked up once per device).
static cudaError_t scratch_address(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_route_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return cudaSuccess;
}

}  // namespace lumen

namespace lumen {
void set_last_error(const std::string& msg);  // api.cu: text returned by lumen_moe_last_error()
}

extern "C" lumen_moe_status_t lumen_moe_route_small_static(const float* d_logits, int32_t tokens,
                                                           int32_t num_experts, int32_t top_k,
                                                           int32_t gating_mode, uint32_t* d_ids,
                                                           float* d_weights, int32_t* d_dst_to_col,
                                                           int32_t* d_expert_bounds, void* stream) {
    using namespace lumen;
    if (!d_logits || !d_ids || !d_weights) {
        set_last_error("null logits / ids / weights pointer");
        return LUMEN_MOE_INVALID_ARG;
    }
    if (tokens < 1 || tokens > RS_MAX_T || num_experts < 1 || num_experts > RS_MAX_E || top_k < 1 ||
        top_k > RS_MAX_K || top_k > num_experts) {
        set_last_error(std::string("lumen_moe_route_small_static is limited by its 8 KiB static scratch to tokens <= 16, "
                       "num_experts <= 256, top_k <= 16 (got tokens=" + std::to_string(tokens) +
                       ", num_experts=" + std::to_string(num_experts) + ", top_k=" + std::to_string(top_k) + ")"));
        return LUMEN_MOE_INVALID_ARG;
    }
    if (gating_mode != 0 && gating_mode != 1) {
        set_last_error("unknown gating mode");
        return LUMEN_MOE_INVALID_ARG;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void* scratch = nullptr;
    cudaError_t e = scratch_address(&scratch);
    if (e == cudaSuccess)  // the counters must start at zero; the array keeps the previous call's contents
        e = cudaMemsetAsync(static_cast<int32_t*>(scratch) + RS_OFF_COUNTS, 0, sizeof(int32_t) * RS_MAX_E, st);
    if (e == cudaSuccess) {
        count_launch();
        route_small_static_kernel<<<1, 256, 0, st>>>(d_logits, tokens, num_experts, top_k, gating_mode, d_ids,
                                                     d_weights, static_cast<int32_t*>(scratch));
        e = cudaGetLastError();
    }
    const size_t C = (size_t)tokens * top_k;
    if (e == cudaSuccess && d_dst_to_col)
        e = cudaMemcpyAsync(d_dst_to_col, static_cast<int32_t*>(scratch) + RS_OFF_D2C, C * 4,
                            cudaMemcpyDeviceToDevice, st);
    if (e == cudaSuccess && d_expert_bounds)
        e = cudaMemcpyAsync(d_expert_bounds, static_cast<int32_t*>(scratch) + RS_OFF_BOUNDS,
                            (size_t)(num_experts + 1) * 4, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) {
        set_last_error(std::string("CUDA error: ") + cudaGetErrorString(e));
        return LUMEN_MOE_CUDA_ERROR;
    }
    return LUMEN_MOE_OK;
}
