// Expert-parallel prefill as ONE library call per rank, with no host round trip and no
// collective library in the data path. The reference is single-GPU (one context, one stream,
// cuda/ffi.rs:61-87): this is the additive multi-GPU form of encode_moe_ffn_prefill_grouped
// (cuda/moe.rs:1900) for multi-token batches. Tokens are sharded over the ranks, experts are
// sharded E / world per rank, the router weight is replicated.
//
// Every rank owns a "window": one device allocation that its peers map through CUDA IPC
// (cudaIpcGetMemHandle / cudaIpcOpenMemHandle) and write with plain stores over NVLink:
//
//   flags     [3][16] u32   counts / rows / results of call number `epoch` have arrived from rank s
//   cnt       [world][E]    pairs per global expert on each source rank (every rank gets every row)
//   ret_map   [rows_cap]    for each received row: (source rank << 24) | compact column there
//   x16       [rows_cap][H] received activation rows, f16, already in the order the grouped GEMM's
//                           weight producer emits (what gather_permute_x16_kernel writes locally)
//   back      [C_cap][H]    f16 expert outputs of MY (token, slot) pairs, by my compact column
//
// One call = this stream of kernels on every rank (all waits bounded; a wait that runs out
// raises the context's status word and the remaining kernels only keep every index in range):
//
//   route + stable counting sort of my tokens         (route_large.cu, unchanged)
//   ep_dispatch_kernel    CTA 0: my per-expert counts -> every rank's cnt[me][*], then their count
//                         flag. All CTAs: wait for all count flags; from the count matrix every rank derives the
//                         same layout of every receive window (rows grouped by expert, inside an
//                         expert by source rank, inside a source in its compact-column order, i.e.
//                         the stable order of cuda/moe.rs:2115-2147 applied globally); push my
//                         rows (+ ret_map entries) straight to their final place; last CTA done
//                         sets my row flag on every rank
//   ep_plan_kernel        wait for all row flags; per-expert column counts of MY experts
//   tile plan + grouped gate/up + SwiGLU + down on tcgen05 (prefill_tc.cu): operands in this
//                         GPU's own memory; the down epilogue sends each token's outputs, 256
//                         bytes per m-tile as one cp.async.bulk copy from a staging tile in
//                         shared memory, into the `back` buffer of the rank the row came from
//   ep_signal_wait_kernel my result flag on every rank, then wait for all result flags
//   scatter_accum_kernel  out[t] = residual[t] + sum_slot w * back[dst_to_col[t, slot]]
//
// Reuse of the single-buffered window is safe in stream order: a rank leaves call n only after
// every rank's results arrived, i.e. after every rank finished reading what call n pushed to it.
// No TMA or tensor-core operand ever lies in another GPU's memory; no multicast anywhere.
#include "host_moe.hpp"
#include <cstring>

namespace lumen {

cudaError_t launch_grouped_tc(const PrefillArgs& p, const void* x16, int grid, cudaStream_t st, __half* out16_rows,
                              const TcPlan* plan, const TcPeerOut* peer);
cudaError_t launch_scatter_accum(const __half* d16, const float* residual, const RouteDev& R, float* out, int T, int H,
                                 int K, cudaStream_t st);

namespace ep {

constexpr int FLAG_STRIDE = 16;  // = MAX_EP_RANKS

struct WindowLayout {
    size_t flags, cnt, ret_map, x16, back, bytes;
};

static inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

static WindowLayout window_layout(int world, int E, int H, int rows_cap, int cols_cap) {
    WindowLayout w{};
    size_t off = 0;
    w.flags = off;
    off += up256(3 * FLAG_STRIDE * sizeof(uint32_t));
    w.cnt = off;
    off += up256((size_t)world * E * sizeof(int32_t));
    w.ret_map = off;
    off += up256((size_t)rows_cap * sizeof(int32_t));
    w.x16 = off;
    off += up256((size_t)rows_cap * H * 2);
    w.back = off;
    off += up256((size_t)cols_cap * H * 2);
    w.bytes = off;
    return w;
}

struct Peers {
    uint8_t* win[MAX_EP_RANKS];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Thread s < world waits until rank s's flag of this kind carries this call's number. Bounded;
// returns false for the whole CTA (through `fail_s`) when a wait ran out or the status word is
// already raised.
__device__ __forceinline__ bool wait_flags(const uint32_t* flags, int world, uint32_t epoch, unsigned long long limit_ns,
                                           int32_t* status, int32_t* status_host, int* fail_s) {
    if (threadIdx.x == 0) *fail_s = 0;
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const uint32_t* f = flags + threadIdx.x;
        unsigned long long t0 = 0;
        unsigned spins = 0;
        // flags only grow: a rank that is already one call ahead has certainly finished this one
        while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
            if ((++spins & 31u) == 0) {
                if (t0 == 0) t0 = now_ns();
                if (now_ns() - t0 > limit_ns || *reinterpret_cast<volatile int32_t*>(status) != 0) {
                    raise_status(status, status_host, 4);  // LUMEN_MOE_TIMEOUT
                    *fail_s = 1;
                    break;
                }
            }
        }
    }
    __syncthreads();
    return *fail_s == 0;
}

// ---------------------------------------------------------------------------
// my counts -> every rank
// ---------------------------------------------------------------------------
// ---------------------------------------------------------------------------
// push my rows to their final place in the owners' windows
// ---------------------------------------------------------------------------
template <typename XT>
__device__ __forceinline__ uint16_t to_f16_bits(XT v);
template <>
__device__ __forceinline__ uint16_t to_f16_bits<float>(float v) { return __half_as_ushort(__float2half_rn(v)); }
template <>
__device__ __forceinline__ uint16_t to_f16_bits<__nv_bfloat16>(__nv_bfloat16 v) {
    return __half_as_ushort(__float2half_rn(__bfloat162float(v)));
}

struct DispatchArgs {
    const void* x;                 // my activations [T, H]
    const int32_t* col_expert;     // my sort tables (route_large.cu)
    const int32_t* col_src_tok;
    const int32_t* expert_bounds;  // [E + 1]
    uint8_t* my_win;
    Peers peers;
    WindowLayout wl;
    int C, H, E, epr, world, me, rows_cap;
    int natural;                   // rows in the natural input order (TMA-fed weights) instead of the dequantiser's order
    uint32_t* epoch_dev;           // number of the previous call; this kernel's last CTA advances it
    unsigned long long limit_ns;
    int32_t* status;
    int32_t* status_host;
    unsigned int* done_counter;    // local: CTAs that finished pushing
};

template <typename XT>
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __grid_constant__ DispatchArgs a) {
    grid_dep_sync();
    __shared__ int base_s[MAX_EXPERTS];   // first row, in the owner's window, of MY pairs of expert e
    __shared__ int tot_s[MAX_EXPERTS];    // pairs of expert e over all ranks
    __shared__ int mine_s[MAX_EXPERTS + 1];
    __shared__ int fail_s;
    __shared__ int over_s;
    const int tid = threadIdx.x;
    // The number of the call that tags every flag lives in device memory, so that a captured call
    // can be replayed from a CUDA graph (a host-side counter would be frozen into the graph). Every
    // CTA reads the previous call's number here; the last CTA to finish stores this call's.
    const uint32_t epoch = *a.epoch_dev + 1u;
    if (blockIdx.x == 0) {
        // my per-expert pair counts into every rank's count matrix, then my count flag there
        for (int i = tid; i < a.world * a.E; i += 256) {
            const int r = i / a.E, e = i - r * a.E;
            int32_t* cnt = reinterpret_cast<int32_t*>(a.peers.win[r] + a.wl.cnt) + (size_t)a.me * a.E;
            cnt[e] = a.expert_bounds[e + 1] - a.expert_bounds[e];
        }
        __threadfence_system();
        __syncthreads();
        if (tid < a.world)
            st_release_sys(reinterpret_cast<uint32_t*>(a.peers.win[tid] + a.wl.flags) + 0 * FLAG_STRIDE + a.me, epoch);
    }
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(a.my_win + a.wl.flags);
    const bool ok = wait_flags(flags + 0 * FLAG_STRIDE, a.world, epoch, a.limit_ns, a.status, a.status_host, &fail_s);
    if (tid == 0) over_s = 0;
    const int32_t* cnt = reinterpret_cast<const int32_t*>(a.my_win + a.wl.cnt);
    const int cols_cap = a.rows_cap;  // no count can exceed the window
    for (int e = tid; e < a.E; e += 256) {
        int tot = 0, before = 0;
        for (int s = 0; s < a.world; ++s) {
            int c = ok ? __ldcg(cnt + (size_t)s * a.E + e) : 0;
            c = min(max(c, 0), cols_cap);
            if (s < a.me) before += c;
            tot += c;
        }
        tot_s[e] = tot;
        base_s[e] = before;
        mine_s[e] = a.expert_bounds[e];
    }
    if (tid == 0) mine_s[a.E] = a.expert_bounds[a.E];
    __syncthreads();
    for (int e = tid; e < a.E; e += 256) {
        const int first = (e / a.epr) * a.epr;
        long long lower = 0;
        for (int q = first; q < e; ++q) lower += tot_s[q];
        const long long b = lower + base_s[e];
        // the owner's window must hold everything it is sent
        if (lower + tot_s[e] > (long long)a.rows_cap) over_s = 1;
        base_s[e] = (int)min(b, (long long)a.rows_cap);
    }
    __syncthreads();
    if (over_s && tid == 0) raise_status(a.status, a.status_host, 1);  // receive capacity exceeded: LUMEN_MOE_INVALID_ARG
    const bool push = ok && !over_s;

    if (push) {
        // start with the columns of the NEXT rank and wrap around, so that at any moment the ranks
        // write to different owners instead of all converging on rank 0's ingress
        const int start = mine_s[((a.me + 1) % a.world) * a.epr];
        const XT* x = static_cast<const XT*>(a.x);
        struct __align__(4 * sizeof(XT)) Run { XT v[4]; };
        // Four rows per step: where they go is worked out first, then all of a thread's loads are in
        // flight together before the peer stores (one row per step was a chain of dependent latencies).
        constexpr int R = 4;
        for (int ci0 = blockIdx.x * R; ci0 < a.C; ci0 += gridDim.x * R) {
            uint16_t* dstrow[R];
            const XT* srcrow[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                dstrow[r] = nullptr;
                srcrow[r] = x;
                const int ci = ci0 + r;
                if (ci >= a.C) continue;
                int c = ci + start;
                if (c >= a.C) c -= a.C;
                const int e = a.col_expert[c];
                const int tok = a.col_src_tok[c];
                if ((unsigned)e >= (unsigned)a.E) continue;
                const int owner = e / a.epr;
                const int drow = base_s[e] + (c - mine_s[e]);
                if (drow >= a.rows_cap) continue;
                uint8_t* w = a.peers.win[owner];
                dstrow[r] = reinterpret_cast<uint16_t*>(w + a.wl.x16) + (size_t)drow * a.H;
                srcrow[r] = x + (size_t)tok * a.H;
                if (tid == 0) reinterpret_cast<int32_t*>(w + a.wl.ret_map)[drow] = (a.me << 24) | c;
            }
            // chunk t of a 32-block holds inputs (4t, 4t+2, 16+4t, 16+4t+2, 4t+1, 4t+3, 16+4t+1, 16+4t+3),
            // or, for TMA-fed weights, chunk ch holds inputs 8 ch .. 8 ch + 7 as they are
            for (int ch = tid; ch < a.H / 8; ch += 256) {
                const int blk = ch >> 2, t = ch & 3;
                const int oa = a.natural ? ch * 8 : blk * 32 + 4 * t, ob = a.natural ? ch * 8 + 4 : blk * 32 + 16 + 4 * t;
                Run p[R], q[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    p[r] = *reinterpret_cast<const Run*>(srcrow[r] + oa);
                    q[r] = *reinterpret_cast<const Run*>(srcrow[r] + ob);
                }
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (dstrow[r] == nullptr) continue;
                    uint4 o;
                    if (a.natural) {
                        o.x = (uint32_t)to_f16_bits<XT>(p[r].v[0]) | ((uint32_t)to_f16_bits<XT>(p[r].v[1]) << 16);
                        o.y = (uint32_t)to_f16_bits<XT>(p[r].v[2]) | ((uint32_t)to_f16_bits<XT>(p[r].v[3]) << 16);
                        o.z = (uint32_t)to_f16_bits<XT>(q[r].v[0]) | ((uint32_t)to_f16_bits<XT>(q[r].v[1]) << 16);
                        o.w = (uint32_t)to_f16_bits<XT>(q[r].v[2]) | ((uint32_t)to_f16_bits<XT>(q[r].v[3]) << 16);
                    } else {
                        o.x = (uint32_t)to_f16_bits<XT>(p[r].v[0]) | ((uint32_t)to_f16_bits<XT>(p[r].v[2]) << 16);
                        o.y = (uint32_t)to_f16_bits<XT>(q[r].v[0]) | ((uint32_t)to_f16_bits<XT>(q[r].v[2]) << 16);
                        o.z = (uint32_t)to_f16_bits<XT>(p[r].v[1]) | ((uint32_t)to_f16_bits<XT>(p[r].v[3]) << 16);
                        o.w = (uint32_t)to_f16_bits<XT>(q[r].v[1]) | ((uint32_t)to_f16_bits<XT>(q[r].v[3]) << 16);
                    }
                    *reinterpret_cast<uint4*>(dstrow[r] + blk * 32 + t * 8) = o;
                }
            }
        }
    }
    // my rows are out once every CTA's stores are: the last CTA to get here tells every rank
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(a.done_counter, 1u);
        fail_s = (prev == gridDim.x - 1) ? 1 : 0;  // (reused as "I am last")
    }
    __syncthreads();
    if (fail_s) {
        __threadfence_system();
        if (tid < a.world)
            st_release_sys(reinterpret_cast<uint32_t*>(a.peers.win[tid] + a.wl.flags) + 1 * FLAG_STRIDE + a.me, epoch);
        if (tid == 0) {
            *a.done_counter = 0u;
            *a.epoch_dev = epoch;
        }
    }
}

// ---------------------------------------------------------------------------
// receive side: column counts of my experts once every rank's rows are in
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
ep_plan_kernel(const uint8_t* my_win, WindowLayout wl, int E, int epr, int world, int me, int rows_cap,
               const uint32_t* epoch_dev, unsigned long long limit_ns, int32_t* status, int32_t* status_host,
               int32_t* counts_out) {
    grid_dep_sync();
    __shared__ int fail_s;
    __shared__ int tot_s[MAX_EXPERTS];
    const uint32_t epoch = *epoch_dev;
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(my_win + wl.flags);
    const bool ok = wait_flags(flags + 1 * FLAG_STRIDE, world, epoch, limit_ns, status, status_host, &fail_s);
    const int32_t* cnt = reinterpret_cast<const int32_t*>(my_win + wl.cnt);
    const int tid = threadIdx.x;
    if (tid < epr) {
        int tot = 0;
        for (int s = 0; s < world; ++s) {
            int c = ok ? __ldcg(cnt + (size_t)s * E + me * epr + tid) : 0;
            tot += min(max(c, 0), rows_cap);
        }
        tot_s[tid] = tot;
    }
    __syncthreads();
    if (tid == 0) {
        // keep the running total inside the window whatever the counts say
        int run = 0;
        for (int e = 0; e < epr; ++e) {
            const int c = min(tot_s[e], rows_cap - run);
            counts_out[e] = c;
            run += c;
        }
    }
}

// my result flag on every rank (the grouped GEMMs of this stream have completed), then wait for everyone's
__global__ void ep_signal_wait_kernel(Peers peers, const uint8_t* my_win, WindowLayout wl, int world, int me,
                                      const uint32_t* epoch_dev, unsigned long long limit_ns, int32_t* status,
                                      int32_t* status_host) {
    grid_dep_sync();
    __shared__ int fail_s;
    const uint32_t epoch = *epoch_dev;
    __threadfence_system();
    if ((int)threadIdx.x < world)
        st_release_sys(reinterpret_cast<uint32_t*>(peers.win[threadIdx.x] + wl.flags) + 2 * FLAG_STRIDE + me, epoch);
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(my_win + wl.flags);
    wait_flags(flags + 2 * FLAG_STRIDE, world, epoch, limit_ns, status, status_host, &fail_s);
}

}  // namespace ep

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
struct EpState {
    int rank = 0, world = 1, epr = 0;
    int cap_tokens = 0;   // tokens of this rank per call, at most
    int cols_cap = 0;     // cap_tokens * K
    int rows_cap = 0;     // rows this rank can receive per call
    ep::WindowLayout wl{};
    uint8_t* win = nullptr;
    ep::Peers peers{};
    bool attached = false;
    bool opened[MAX_EP_RANKS] = {};
    // local-only buffers of the expert side
    void* local = nullptr;
    __half* s16 = nullptr;
    int4* tiles = nullptr;
    int32_t* n_tiles = nullptr;
    RouteDev RX{};        // expert_bounds / uexp / n_uexp of MY experts (the other fields unused)
    unsigned int* done_counter = nullptr;
    uint32_t* epoch_dev = nullptr;  // number of the current call, in device memory
    // optional phase timing of a call (lumen_moe_ep_profile): events between the launches
    bool profile = false;
    cudaEvent_t ev[7] = {};
    bool ev_made = false, ev_valid = false;
};

#define CUDA_TRY(expr)                                                                              \
    do {                                                                                            \
        cudaError_t _e = (expr);                                                                    \
        if (_e != cudaSuccess)                                                                      \
            return Status::Err(3, std::string(#expr) + ": " + cudaGetErrorString(_e));              \
    } while (0)

void ep_free(EpState* s) {
    if (!s) return;
    for (int r = 0; r < s->world; ++r)
        if (s->opened[r] && s->peers.win[r]) cudaIpcCloseMemHandle(s->peers.win[r]);
    if (s->win) cudaFree(s->win);
    if (s->local) cudaFree(s->local);
    if (s->ev_made)
        for (cudaEvent_t e : s->ev) cudaEventDestroy(e);
    delete s;
}

Status ep_create(CudaMoeScratch* sc, int rank, int world, int max_tokens, int recv_rows, EpState** out, void* handle64) {
    if (world < 1 || world > MAX_EP_RANKS || rank < 0 || rank >= world)
        return Status::Err(1, "rank / world out of range (at most 16 ranks)");
    if (sc->E % world) return Status::Err(1, "num_experts must be divisible by the number of ranks");
    if (max_tokens < 1) return Status::Err(1, "max_tokens must be positive");
    if (sc->H % 256 || sc->I % 128) return Status::Err(2, "the expert-parallel path needs hidden_dim % 256 == 0 and inter_dim % 128 == 0");
    if ((size_t)max_tokens * sc->K >= (1u << 24)) return Status::Err(1, "max_tokens * top_k must stay below 2^24");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI passes IPC handles as 64 bytes");
    EpState* s = new EpState();
    s->rank = rank;
    s->world = world;
    s->epr = sc->E / world;
    s->cap_tokens = max_tokens;
    s->cols_cap = max_tokens * sc->K;
    // default: room for every pair of every rank (no routing skew can overflow it)
    s->rows_cap = recv_rows > 0 ? recv_rows : s->cols_cap * world;
    s->rows_cap = (s->rows_cap + 127) / 128 * 128;
    s->wl = ep::window_layout(world, sc->E, sc->H, s->rows_cap, s->cols_cap);
    cudaError_t e = cudaMalloc(&s->win, s->wl.bytes);
    if (e == cudaSuccess) e = cudaMemset(s->win, 0, s->wl.bytes);
    // local: s16 [rows_cap, I], tile lists, expert tables
    const int gu_ct = s->rows_cap / 128 + s->epr, dn_ct = s->rows_cap / 128 + s->epr;
    const size_t n_tiles = (size_t)gu_ct * (sc->I / 128 + 1) + (size_t)dn_ct * (sc->H / 256 + 1);
    size_t off = 0, o_s16 = 0, o_tiles, o_misc;
    off += ep::up256((size_t)s->rows_cap * sc->I * 2);
    o_tiles = off;
    off += ep::up256(n_tiles * sizeof(int4));
    o_misc = off;
    off += 4096;
    if (e == cudaSuccess) e = cudaMalloc(&s->local, off);
    if (e == cudaSuccess) e = cudaMemset(s->local, 0, off);
    if (e != cudaSuccess) {
        const std::string msg = std::string("expert-parallel buffers: ") + cudaGetErrorString(e);
        ep_free(s);
        return Status::Err(3, msg);
    }
    uint8_t* b = static_cast<uint8_t*>(s->local);
    s->s16 = reinterpret_cast<__half*>(b + o_s16);
    s->tiles = reinterpret_cast<int4*>(b + o_tiles);
    int32_t* misc = reinterpret_cast<int32_t*>(b + o_misc);
    s->RX.expert_bounds = misc;            // [epr + 1] <= 257
    s->RX.uexp = misc + 264;               // [epr]
    s->RX.n_uexp = misc + 528;
    s->n_tiles = misc + 536;               // [4]: tile counts and the tile counters of the two products
    s->done_counter = reinterpret_cast<unsigned int*>(misc + 544);
    s->epoch_dev = reinterpret_cast<uint32_t*>(misc + 552);
    s->peers.win[rank] = s->win;
    if (world == 1) s->attached = true;
    if (handle64) {
        cudaIpcMemHandle_t h;
        e = cudaIpcGetMemHandle(&h, s->win);
        if (e != cudaSuccess) {
            const std::string msg = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e);
            ep_free(s);
            return Status::Err(3, msg);
        }
        std::memcpy(handle64, &h, 64);
    }
    *out = s;
    return Status::Ok();
}

Status ep_attach(EpState* s, const void* handles64) {
    if (s->attached) return Status::Ok();
    for (int r = 0; r < s->world; ++r) {
        if (r == s->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const uint8_t*>(handles64) + (size_t)r * 64, 64);
        void* p = nullptr;
        CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        s->peers.win[r] = static_cast<uint8_t*>(p);
        s->opened[r] = true;
    }
    s->attached = true;
    return Status::Ok();
}

// One expert-parallel layer call on this rank (see the head of the file). `layer` holds the
// replicated router weight and the planes of this rank's experts only (L.E = epr).
Status encode_moe_ffn_prefill_ep(CudaMoeScratch* sc, EpState* s, const MoeLayer& layer, const void* normed, int act_dtype,
                                 const float* residual, float* output, int batch, cudaStream_t st) {
    if (!s->attached) return Status::Err(1, "lumen_moe_ep_attach has not been called");
    if (batch < 1 || batch > s->cap_tokens) return Status::Err(1, "tokens outside 1..max_tokens of lumen_moe_ep_create");
    if (!normed || !residual || !output) return Status::Err(1, "null activation pointer");
    if (act_dtype != 0 && act_dtype != 1) return Status::Err(2, "activation dtype must be f32 or bf16");
    if (reinterpret_cast<uintptr_t>(normed) % 16) return Status::Err(1, "activations must be 16-byte aligned");
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != sc->device) return Status::Err(1, "the context belongs to another CUDA device than the current one");
    Status w = check_status_word(sc);
    if (!w.ok()) return w;
    if (layer.dev.H != sc->H || layer.dev.I != sc->I || layer.dev.E != s->epr || layer.dev.quant < 0)
        return Status::Err(1, "not a layer prepared by lumen_moe_ep_layer_prepare for this context");
    Status g = ensure_prefill_grouped(sc, batch);
    if (!g.ok()) return g;

    const unsigned long long limit_ns = sc->wait_limit_us ? (unsigned long long)sc->wait_limit_us * 1000ull : 2000000000ull;
    if (s->profile && !s->ev_made) {
        for (cudaEvent_t& e : s->ev) CUDA_TRY(cudaEventCreate(&e));
        s->ev_made = true;
    }
    auto mark = [&](int i) {
        if (s->profile) cudaEventRecord(s->ev[i], st);
    };
    mark(0);
    // 1. route my tokens over ALL experts and sort the pairs (no tile lists: the GEMMs run on received rows)
    PrefillArgs p{};
    p.L = layer.dev;
    p.L.E = sc->E;
    p.R = sc->R;
    p.x = normed;
    p.act_dtype = act_dtype;
    p.T = batch;
    p.K = sc->K;
    p.gating = sc->gating;
    p.logits_override = sc->logits_override;
    p.blk_hist = sc->blk_hist;
    p.w16 = sc->w16;
    p.xr16 = sc->xr16;
    p.rpart = sc->rpart;
    p.any_lo = sc->any_lo;
    p.sms = sc->sms;
    p.wait_limit_us = sc->wait_limit_us;
    p.tiles = nullptr;
    p.n_tiles = sc->n_tiles;
    p.status = sc->status;
    p.status_host = sc->status_host;
    CUDA_TRY(launch_route_large(p, st));
    mark(1);
    const int C = batch * sc->K;
    // 2. counts to everyone, 3. rows to their owners (one kernel)
    count_launch(1);
    ep::DispatchArgs d{};
    d.x = normed;
    d.col_expert = sc->R.col_expert;
    d.col_src_tok = sc->R.col_src_tok;
    d.expert_bounds = sc->R.expert_bounds;
    d.my_win = s->win;
    d.peers = s->peers;
    d.wl = s->wl;
    d.C = C;
    d.H = sc->H;
    d.E = sc->E;
    d.epr = s->epr;
    d.world = s->world;
    d.me = s->rank;
    d.rows_cap = s->rows_cap;
    d.natural = layer.dev.gu16 != nullptr ? 1 : 0;
    d.epoch_dev = s->epoch_dev;
    d.limit_ns = limit_ns;
    d.status = sc->status;
    d.status_host = sc->status_host;
    d.done_counter = s->done_counter;
    const int dgrid = (C + 3) / 4 < sc->sms * 8 ? (C + 3) / 4 : sc->sms * 8;  // four rows per CTA step
    CUDA_TRY(act_dtype == 0 ? launch_dep(ep::ep_dispatch_kernel<float>, dim3(dgrid), dim3(256), 0, st, d)
                            : launch_dep(ep::ep_dispatch_kernel<__nv_bfloat16>, dim3(dgrid), dim3(256), 0, st, d));
    mark(2);
    // 4. what arrived for my experts
    count_launch(1);
    CUDA_TRY(launch_dep(ep::ep_plan_kernel, dim3(1), dim3(256), 0, st, (const uint8_t*)s->win, s->wl, sc->E, s->epr, s->world,
                        s->rank, s->rows_cap, (const uint32_t*)s->epoch_dev, limit_ns, sc->status, sc->status_host,
                        s->RX.expert_bounds));
    // expected rows per expert under balanced routing decide the gate/up tile width
    const int gu_cols = ((long long)C > 128ll * s->epr) ? 256 : 128;
    CUDA_TRY(launch_tile_plan(s->RX, s->epr, sc->H, sc->I, s->rows_cap, gu_cols, s->tiles, s->n_tiles, st));
    mark(3);
    // 5. grouped products on my experts; outputs go back to the pairs' home ranks
    PrefillArgs q{};
    q.L = layer.dev;
    q.R = s->RX;
    q.T = s->rows_cap;
    q.K = 1;
    q.s16 = s->s16;
    q.d16 = nullptr;
    q.tiles = s->tiles;
    q.n_tiles = s->n_tiles;
    q.status = sc->status;
    q.status_host = sc->status_host;
    q.wait_limit_us = sc->wait_limit_us;
    TcPlan plan{s->rows_cap, gu_cols};
    TcPeerOut po{};
    po.ret_map = reinterpret_cast<const int32_t*>(s->win + s->wl.ret_map);
    for (int r = 0; r < s->world; ++r) po.base[r] = reinterpret_cast<__half*>(s->peers.win[r] + s->wl.back);
    po.world = s->world;
    po.rows_cap = s->cols_cap;
    int grid = sc->sms;
    if (sc->tc_ctas > 0 && sc->tc_ctas < grid) grid = sc->tc_ctas;
    CUDA_TRY(launch_grouped_tc(q, s->win + s->wl.x16, grid, st, nullptr, &plan, &po));
    mark(4);
    // 6. results are out; wait for everyone's; combine
    count_launch(1);
    CUDA_TRY(launch_dep(ep::ep_signal_wait_kernel, dim3(1), dim3(32), 0, st, s->peers, (const uint8_t*)s->win, s->wl, s->world,
                        s->rank, (const uint32_t*)s->epoch_dev, limit_ns, sc->status, sc->status_host));
    CUDA_TRY(cudaGetLastError());
    mark(5);
    CUDA_TRY(launch_scatter_accum(reinterpret_cast<const __half*>(s->win + s->wl.back), residual, sc->R, output, batch,
                                  sc->H, sc->K, st));
    mark(6);
    s->ev_valid = s->profile;
    return Status::Ok();
}

void ep_set_profile(EpState* s, bool on) {
    s->profile = on;
    if (!on) s->ev_valid = false;
}

// ms of the last profiled call: route+sort | counts+dispatch (includes waiting for every rank's
// counts) | wait for every rank's rows + tile plan | gate/up+SwiGLU+down | wait for every rank's
// results | combine
Status ep_phase_ms(EpState* s, float* out6) {
    if (!s->ev_valid) return Status::Err(1, "no profiled call yet (lumen_moe_ep_profile)");
    CUDA_TRY(cudaEventSynchronize(s->ev[6]));
    for (int i = 0; i < 6; ++i) CUDA_TRY(cudaEventElapsedTime(&out6[i], s->ev[i], s->ev[i + 1]));
    return Status::Ok();
}

int ep_rank(const EpState* s) { return s->rank; }
int ep_world(const EpState* s) { return s->world; }
int ep_experts_per_rank(const EpState* s) { return s->epr; }
size_t ep_window_bytes(const EpState* s) { return s->wl.bytes; }

}  // namespace lumen
