// Routing and dispatch tables for multi-token batches (prefill), entirely on the
// device: the reference does this part of encode_moe_ffn_prefill_grouped with a
// blocking device-to-host copy, a host loop and four to six uploads per layer
// (crates/lumen-runtime/src/cuda/moe.rs:2105-2207).
//
//   router_logits_large_kernel  logits[T,E] = X[T,H] W_r[E,H]^T, f32 accumulate
//                               (moe_router_logits_batched, cuda/shaders/moe_grouped.cu:79)
//   topk_large_kernel           one warp per token (router.cuh)
//   sort_hist / sort_scan / sort_place
//                               stable counting sort of (token, slot) pairs by
//                               expert, tokens ascending then slots ascending:
//                               expert_bounds, col_expert, col_src_tok, dst_to_col
//                               exactly as cuda/moe.rs:2115-2147; sort_scan also
//                               emits the list of experts with work and the tile
//                               lists of the grouped GEMMs (cuda/moe.rs:2188-2207).
//   scatter_accum_kernel        out[t] = residual[t] + sum_slot w[t,slot] * D[dst_to_col[t,slot]]
//                               in slot order (moe_grouped_scatter_accum_q8_0,
//                               cuda/shaders/moe_grouped.cu:493-517).
#include "moe_internal.cuh"
#include "router.cuh"
#include "mma_frag.cuh"

#define CUDA_RET(expr)                         \
    do {                                       \
        const cudaError_t e_ = (expr);         \
        if (e_ != cudaSuccess) return e_;      \
    } while (0)

namespace lumen {

// ---------------------------------------------------------------------------
// logits: 64 tokens x 64 experts per CTA, BK = 32, 256 threads, 4x4 per thread
// ---------------------------------------------------------------------------
template <typename XT>
__device__ __forceinline__ float x_to_f32(XT v);
template <>
__device__ __forceinline__ float x_to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float x_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float x_to_f32<__half>(__half v) { return __half2float(v); }

template <typename XT>
__global__ void __launch_bounds__(256)
router_logits_large_kernel(const XT* __restrict__ x, const float* __restrict__ w, float* __restrict__ logits,
                           int T, int H, int E) {
    constexpr int BM = 64, BN = 64, BK = 32;
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    const int tid = threadIdx.x;
    const int t0 = blockIdx.x * BM, e0 = blockIdx.y * BN;
    const int tx = tid & 15, ty = tid >> 4;  // tx: experts, ty: tokens
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < H; k0 += BK) {
        for (int i = tid; i < BM * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int t = t0 + r;
            xs[c][r] = (t < T) ? x_to_f32<XT>(x[(size_t)t * H + k0 + c]) : 0.0f;
        }
        for (int i = tid; i < BN * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int e = e0 + r;
            ws[c][r] = (e < E) ? w[(size_t)e * H + k0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = e0 + tx * 4 + j;
            if (e < E) logits[(size_t)t * E + e] = acc[i][j];
        }
    }
}

// ---------------------------------------------------------------------------
// logits on the tensor cores with f32-grade accuracy: X and W_r are each split into
// a high and a low f16 part and up to three m16n8k16 products (hi*hi + hi*lo + lo*hi)
// are accumulated in f32; the dropped lo*lo term is ~2^-22 relative. W_r is split
// once per call into two [E,H] f16 planes; X is split in registers (the lo*hi
// product is skipped for a fragment whose low parts are all zero, which is the
// usual case for bf16 activations).
// CTA = 64 tokens x (up to) 64 experts, 4 warps of 16 tokens (small tiles: at a few
// thousand tokens the grid must still cover the SMs). Per 32-input slab
// lane (g,t) owns inputs 8t..8t+7 of token rows g and g+8 (one 16-byte load each
// for bf16) and of expert row 8n+g (one 16-byte shared load per plane): the same
// input -> k-slot assignment on both operands, so the contraction is unchanged.
// ---------------------------------------------------------------------------
__global__ void split_router_w_kernel(const float* __restrict__ w, __half* __restrict__ w16, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = w[i];
    const __half hi = __float2half_rn(v);
    w16[i] = hi;
    w16[n + i] = __float2half_rn(v - __half2float(hi));
}

__device__ __forceinline__ void cp_async16_rl(void* smem_dst, const void* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}

template <typename XT>
struct XSlab;  // 8 consecutive inputs of one token row
template <>
struct XSlab<__nv_bfloat16> {
    uint4 v;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void get(float* f) const {
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(u[i] << 16);
            f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
};
template <>
struct XSlab<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = *reinterpret_cast<const float4*>(p);
        b = *reinterpret_cast<const float4*>(p + 4);
    }
    __device__ __forceinline__ void get(float* f) const {
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
};

__device__ __forceinline__ void split_pair(float v0, float v1, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(v0, v1);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(v0 - hf.x, v1 - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// NE = experts per CTA: 64, or 32 for batches that would otherwise leave most SMs with a few warps
template <typename XT, int NE>
__global__ void __launch_bounds__(128)
router_logits_mma_kernel(const XT* __restrict__ x, const __half* __restrict__ w16, float* __restrict__ logits,
                         int T, int H, int E) {
    constexpr int BM = 64, BK = 32;
    // [buffer][plane][expert row][32 inputs]: 64-byte rows, 16-byte fragment loads are conflict-free
    __shared__ __align__(16) __half ws[2][2][NE][BK];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int t0 = blockIdx.x * BM, e0 = blockIdx.y * NE;
    const int ne = min(NE, E - e0);
    const int ntile = (ne + 7) >> 3;
    const size_t plane = (size_t)E * H;
    float acc[NE / 8][4];
#pragma unroll
    for (int n = 0; n < NE / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    const int ra = t0 + warp * 16 + g, rb = ra + 8;
    const XT* xa = x + (size_t)min(ra, T - 1) * H + 8 * t4;
    const XT* xb = x + (size_t)min(rb, T - 1) * H + 8 * t4;
    auto stage_w = [&](int buf, int k0) {
        // NE rows x 4 chunks x 2 planes = 512 16-byte copies, 4 per thread
#pragma unroll
        for (int i = 0; i < NE / 16; ++i) {
            const int c = tid + i * 128;
            const int pl = c / (NE * 4), row = (c >> 2) % NE, ch = c & 3;
            const __half* src = w16 + pl * plane + (size_t)min(e0 + row, E - 1) * H + k0 + ch * 8;
            cp_async16_rl(&ws[buf][pl][row][ch * 8], src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int nslab = H / BK;
    XSlab<XT> na, nb;
    stage_w(0, 0);
    na.load(xa);
    nb.load(xb);
    for (int sidx = 0; sidx < nslab; ++sidx) {
        const int buf = sidx & 1;
        XSlab<XT> ca = na, cb = nb;
        if (sidx + 1 < nslab) {
            stage_w(buf ^ 1, (sidx + 1) * BK);
            na.load(xa + (sidx + 1) * BK);
            nb.load(xb + (sidx + 1) * BK);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        float fa[8], fb[8];
        ca.get(fa);
        cb.get(fb);
        uint32_t ah[2][4], al[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            split_pair(fa[4 * j], fa[4 * j + 1], ah[j][0], al[j][0]);
            split_pair(fb[4 * j], fb[4 * j + 1], ah[j][1], al[j][1]);
            split_pair(fa[4 * j + 2], fa[4 * j + 3], ah[j][2], al[j][2]);
            split_pair(fb[4 * j + 2], fb[4 * j + 3], ah[j][3], al[j][3]);
        }
        uint32_t lo_or = 0;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) lo_or |= al[j][i];
        const bool use_lo = __any_sync(0xffffffffu, (lo_or & 0x7fff7fffu) != 0);
#pragma unroll
        for (int n = 0; n < NE / 8; ++n) {
            if (n < ntile) {
                const uint4 bh = *reinterpret_cast<const uint4*>(&ws[buf][0][n * 8 + g][8 * t4]);
                const uint4 bl = *reinterpret_cast<const uint4*>(&ws[buf][1][n * 8 + g][8 * t4]);
                if (use_lo) {
                    mma_f16(acc[n], al[0], bh.x, bh.y);
                    mma_f16(acc[n], al[1], bh.z, bh.w);
                }
                mma_f16(acc[n], ah[0], bl.x, bl.y);
                mma_f16(acc[n], ah[1], bl.z, bl.w);
                mma_f16(acc[n], ah[0], bh.x, bh.y);
                mma_f16(acc[n], ah[1], bh.z, bh.w);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int n = 0; n < NE / 8; ++n) {
        if (n < ntile) {
            const int ec = e0 + n * 8 + 2 * t4;
            if (ra < T) {
                if (ec < E) logits[(size_t)ra * E + ec] = acc[n][0];
                if (ec + 1 < E) logits[(size_t)ra * E + ec + 1] = acc[n][1];
            }
            if (rb < T) {
                if (ec < E) logits[(size_t)rb * E + ec] = acc[n][2];
                if (ec + 1 < E) logits[(size_t)rb * E + ec + 1] = acc[n][3];
            }
        }
    }
}

// nparts > 0: the logits arrive as `nparts` partial sums [nparts][T][E] (k ranges of the tcgen05
// router); they are added in a fixed order and the sum is left in logits_out.
constexpr int TK_WARPS = 8;
// blk_hist (null = none): the per-expert pair counts of this block's TK_WARPS tokens, the first
// step of the counting sort (one histogram per chunk of SORT_TOK = TK_WARPS tokens), written here
// instead of by a launch of its own.
__global__ void __launch_bounds__(TK_WARPS * 32)
topk_large_kernel(const float* __restrict__ logits, int nparts, float* __restrict__ logits_out, int T, int E, int K,
                  int gating, uint32_t* __restrict__ ids, float* __restrict__ weights, int32_t* __restrict__ blk_hist) {
    grid_dep_sync();
    __shared__ __align__(16) float p_s[TK_WARPS][MAX_EXPERTS];
    __shared__ __align__(16) float lg_s[TK_WARPS][MAX_EXPERTS];
    __shared__ int h[MAX_EXPERTS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * TK_WARPS + warp;
    for (int e = threadIdx.x; e < E; e += TK_WARPS * 32) h[e] = 0;
    __syncthreads();
    if (t < T) {
        for (int i = lane; i < E; i += 32) {
            float v = logits[(size_t)t * E + i];
            for (int q = 1; q < nparts; ++q) v += logits[((size_t)q * T + t) * E + i];
            if (nparts > 0) logits_out[(size_t)t * E + i] = v;
            lg_s[warp][i] = v;
        }
        __syncwarp();
        warp_topk(lg_s[warp], E, K, gating, p_s[warp], nullptr, ids + (size_t)t * K, weights + (size_t)t * K);
        if (blk_hist != nullptr && lane < K) atomicAdd(&h[ids[(size_t)t * K + lane]], 1);  // (the lane's own store)
    }
    if (blk_hist == nullptr) return;
    __syncthreads();
    // layout [expert][chunk]: a warp of sort_rowscan then scans one expert's row with coalesced loads
    for (int e = threadIdx.x; e < E; e += TK_WARPS * 32) blk_hist[(size_t)e * gridDim.x + blockIdx.x] = h[e];
}

// ---------------------------------------------------------------------------
// stable counting sort
// ---------------------------------------------------------------------------
constexpr int SORT_TOK = TK_WARPS;  // tokens per chunk: one block of the top-k kernel; small chunks also spread the
                                   // placement (one warp per chunk) over the machine

__global__ void __launch_bounds__(256)
sort_hist_kernel(const uint32_t* __restrict__ ids, int T, int K, int E, int32_t* __restrict__ blk_hist) {
    grid_dep_sync();
    __shared__ int h[MAX_EXPERTS];
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += 256) h[e] = 0;
    __syncthreads();
    const int t0 = blockIdx.x * SORT_TOK;
    const int n = min(SORT_TOK, T - t0) * K;
    for (int p = tid; p < n; p += 256) atomicAdd(&h[ids[(size_t)t0 * K + p]], 1);
    __syncthreads();
    // layout [expert][chunk]: a warp of sort_scan then scans one expert's row with coalesced loads
    for (int e = tid; e < E; e += 256) blk_hist[(size_t)e * gridDim.x + blockIdx.x] = h[e];
}

// One warp per expert: exclusive scan over the chunk counts of the expert's row (in place);
// the row total goes to expert_bounds[e] for sort_scan_kernel.
__global__ void __launch_bounds__(32)
sort_rowscan_kernel(int32_t* __restrict__ blk_hist, int nchunks, RouteDev R) {
    grid_dep_sync();
    const int e = blockIdx.x, lane = threadIdx.x;
    int32_t* rowp = blk_hist + (size_t)e * nchunks;
    int run = 0;
    for (int c0 = 0; c0 < nchunks; c0 += 128) {
        int v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = c0 + u * 32 + lane;
            v[u] = (c < nchunks) ? rowp[c] : 0;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = c0 + u * 32 + lane;
            int inc = v[u];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int w = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += w;
            }
            if (c < nchunks) rowp[c] = run + inc - v[u];
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
    }
    if (lane == 0) R.expert_bounds[e] = run;
}

// One CTA of 256 threads (E <= 256): expert segment bounds from the row totals and the
// tile lists. tile entry: {expert, col_start, ncols, m_tile}.
__global__ void __launch_bounds__(256)
sort_scan_kernel(int nchunks, int E, RouteDev R, int tile_cols, int tile_cols_dn,
                 int mt_gu, int mt_dn, int4* __restrict__ tiles_gu, int4* __restrict__ tiles_dn,
                 int32_t* __restrict__ n_tiles, int max_tiles_gu, int max_tiles_dn) {
    grid_dep_sync();
    __shared__ int cnt_s[MAX_EXPERTS];
    __shared__ int bounds_s[MAX_EXPERTS + 1];
    __shared__ int tile_off_s[MAX_EXPERTS + 1];
    __shared__ int tile_off_dn_s[MAX_EXPERTS + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < E) cnt_s[tid] = R.expert_bounds[tid];
    __syncthreads();
    if (warp == 0) {
        int local[8], ltiles[8], ltiles_dn[8], lsum = 0, lnz = 0, ltl = 0, ltd = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int ee = lane * 8 + j;
            local[j] = (ee < E) ? cnt_s[ee] : 0;
            ltiles[j] = (local[j] + tile_cols - 1) / tile_cols;
            ltiles_dn[j] = (local[j] + tile_cols_dn - 1) / tile_cols_dn;
            lsum += local[j];
            lnz += (local[j] > 0);
            ltl += ltiles[j];
            ltd += ltiles_dn[j];
        }
        int isum = lsum, inz = lnz, itl = ltl, itd = ltd;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v1 = __shfl_up_sync(0xffffffffu, isum, o);
            const int v2 = __shfl_up_sync(0xffffffffu, inz, o);
            const int v3 = __shfl_up_sync(0xffffffffu, itl, o);
            const int v4 = __shfl_up_sync(0xffffffffu, itd, o);
            if (lane >= o) {
                isum += v1;
                inz += v2;
                itl += v3;
                itd += v4;
            }
        }
        int run = isum - lsum, unz = inz - lnz, trun = itl - ltl, drun = itd - ltd;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int ee = lane * 8 + j;
            if (ee < E) {
                bounds_s[ee] = run;
                tile_off_s[ee] = trun;
                tile_off_dn_s[ee] = drun;
                R.expert_bounds[ee] = run;
                if (local[j] > 0) R.uexp[unz++] = ee;
                run += local[j];
                trun += ltiles[j];
                drun += ltiles_dn[j];
            }
        }
        if (lane == 31) {
            bounds_s[E] = isum;
            tile_off_s[E] = itl;
            tile_off_dn_s[E] = itd;
            R.expert_bounds[E] = isum;
            *R.n_uexp = inz;
            n_tiles[0] = min(itl * mt_gu, max_tiles_gu);
            n_tiles[1] = min(itd * mt_dn, max_tiles_dn);
            n_tiles[2] = 0;  // tile counters of the two grouped products (tiles are claimed dynamically)
            n_tiles[3] = 0;
        }
    }
    __syncthreads();
    // Column tiles in expert order, all threads emitting: thread takes column chunk c, finds its
    // expert by bisection of the chunk offsets, writes the chunk's m-tiles. The m-tile is the fastest
    // index so that CTAs running side by side share the same activation tile. (One thread per
    // expert used to emit all of a loaded expert's tiles alone: 8.7 us of a 4096-token call.)
    auto emit = [&](const int* off_s, int tcols, int mt_n, int4* __restrict__ tiles, int max_tiles) {
        if (tiles == nullptr) return;
        const int total = off_s[E];
        for (int c = tid; c < total; c += 256) {
            int lo = 0, hi = E;  // largest e with off_s[e] <= c
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (off_s[mid] <= c) lo = mid;
                else hi = mid;
            }
            const int e = lo, ct = c - off_s[e];
            const int cs = bounds_s[e] + ct * tcols;
            const int nc = min(tcols, cnt_s[e] - ct * tcols);
            for (int mt = 0; mt < mt_n; ++mt) {
                const int idx = c * mt_n + mt;
                if (idx < max_tiles) tiles[idx] = make_int4(e, cs, nc, mt);
            }
        }
    };
    emit(tile_off_s, tile_cols, mt_gu, tiles_gu, max_tiles_gu);
    emit(tile_off_dn_s, tile_cols_dn, mt_dn, tiles_dn, max_tiles_dn);
}

// One warp per chunk of SORT_TOK tokens: the chunk's (token, slot) pairs are taken 32 at
// a time in order; lanes holding the same expert find each other with match.any, the
// position inside the expert's segment is the expert's running cursor plus the number
// of lower lanes with the same expert, so the placement is stable.
__global__ void __launch_bounds__(256)
sort_place_kernel(const uint32_t* __restrict__ ids, int T, int K, int E, const int32_t* __restrict__ blk_hist,
                  int nchunks, RouteDev R) {
    grid_dep_sync();
    __shared__ int cursor[8][MAX_EXPERTS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunk = blockIdx.x * 8 + warp;
    if (chunk >= nchunks) return;
    for (int e = lane; e < E; e += 32) cursor[warp][e] = R.expert_bounds[e] + blk_hist[(size_t)e * nchunks + chunk];
    __syncwarp();
    const int t0 = chunk * SORT_TOK;
    const int n = min(SORT_TOK, T - t0) * K;
    for (int p0 = 0; p0 < n; p0 += 32) {
        const int p = p0 + lane;
        const bool valid = p < n;
        const int e = valid ? (int)ids[(size_t)t0 * K + p] : -1 - lane;  // invalid lanes match nobody
        const unsigned int same = __match_any_sync(0xffffffffu, e);
        if (valid) {
            const int rank = __popc(same & ((1u << lane) - 1u));
            const int col = cursor[warp][e] + rank;
            R.col_expert[col] = e;
            R.col_src_tok[col] = t0 + p / K;
            R.dst_to_col[(size_t)t0 * K + p] = col;
        }
        __syncwarp();
        if (valid && (same & ((1u << lane) - 1u)) == 0u) cursor[warp][e] += __popc(same);  // one leader per expert
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------
// activation fragments for the mma.sync grouped path (any T)
// ---------------------------------------------------------------------------
template <typename XT>
__global__ void __launch_bounds__(256)
build_xf_kernel(const XT* __restrict__ x, int T, int H, int nblk_pad, bool bf16_mode, uint4* __restrict__ xf) {
    const int nblk = H >> 5;
    const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;
    const size_t total = (size_t)T * nblk * 8;
    if (idx >= total) return;
    const int sub = (int)(idx & 7), hl = sub >> 2, t4 = sub & 3;
    const size_t item = idx >> 3;
    const int t = (int)(item / nblk), b = (int)(item % nblk);
    const XT* xr = x + (size_t)t * H + b * 32;
    float4 lo4, hi4;
    lo4.x = x_to_f32<XT>(xr[4 * t4]);
    lo4.y = x_to_f32<XT>(xr[4 * t4 + 1]);
    lo4.z = x_to_f32<XT>(xr[4 * t4 + 2]);
    lo4.w = x_to_f32<XT>(xr[4 * t4 + 3]);
    hi4.x = x_to_f32<XT>(xr[16 + 4 * t4]);
    hi4.y = x_to_f32<XT>(xr[16 + 4 * t4 + 1]);
    hi4.z = x_to_f32<XT>(xr[16 + 4 * t4 + 2]);
    hi4.w = x_to_f32<XT>(xr[16 + 4 * t4 + 3]);
    xf[((size_t)(t * 2 + hl) * nblk_pad + b) * 4 + t4] = make_act_frag(lo4, hi4, hl, bf16_mode);
}

// ---------------------------------------------------------------------------
// scatter-accumulate
// ---------------------------------------------------------------------------
// One thread per 8 consecutive outputs (16-byte loads of the f16 rows); the slots are taken four
// at a time so that their rows are in flight together, and added in slot order.
__global__ void __launch_bounds__(256)
scatter_accum_kernel(const __half* __restrict__ d16, const float* residual,
                     const float* __restrict__ weights, const int32_t* __restrict__ dst_to_col,
                     float* out, int T, int H, int K) {  // residual may be out (in-place layer stacks)
    grid_dep_sync();
    const int t = blockIdx.x;  // tokens on grid.x: the y dimension is limited to 65535
    const int h8 = blockIdx.y * 256 + threadIdx.x;  // group of 8 outputs
    if (h8 * 8 >= H) return;
    const size_t o = (size_t)t * H + h8 * 8;
    float acc[8];
    {
        const float4 r0 = *reinterpret_cast<const float4*>(residual + o);
        const float4 r1 = *reinterpret_cast<const float4*>(residual + o + 4);
        acc[0] = r0.x; acc[1] = r0.y; acc[2] = r0.z; acc[3] = r0.w;
        acc[4] = r1.x; acc[5] = r1.y; acc[6] = r1.z; acc[7] = r1.w;
    }
    for (int s0 = 0; s0 < K; s0 += 4) {
        uint4 d[4];
        float w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int slot = min(s0 + j, K - 1);
            const int col = dst_to_col[(size_t)t * K + slot];
            w[j] = weights[(size_t)t * K + slot];
            d[j] = *reinterpret_cast<const uint4*>(d16 + (size_t)col * H + h8 * 8);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (s0 + j < K) {
                const __half2* hp = reinterpret_cast<const __half2*>(&d[j]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(hp[i]);
                    acc[2 * i] = __fadd_rn(acc[2 * i], __fmul_rn(w[j], f.x));
                    acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], __fmul_rn(w[j], f.y));
                }
            }
        }
    }
    *reinterpret_cast<float4*>(out + o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(out + o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

cudaError_t launch_scatter_accum(const __half* d16, const float* residual, const RouteDev& R, float* out,
                                 int T, int H, int K, cudaStream_t st) {
    count_launch();
    return launch_dep(scatter_accum_kernel, dim3(T, (H / 8 + 255) / 256), dim3(256), 0, st, d16, residual, R.weights,
                      R.dst_to_col, out, T, H, K);
}

__global__ void __launch_bounds__(256)
rows_from_cols_kernel(const __half* __restrict__ d16, const int32_t* __restrict__ dst_to_col, __half* __restrict__ out16,
                      int H) {
    const int t = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(d16 + (size_t)dst_to_col[t] * H);
    uint4* dst = reinterpret_cast<uint4*>(out16 + (size_t)t * H);
    for (int i = threadIdx.x; i < H / 8; i += 256) dst[i] = src[i];
}

cudaError_t launch_rows_from_cols(const __half* d16, const int32_t* dst_to_col, __half* out16, int T, int H,
                                  cudaStream_t st) {
    count_launch();
    rows_from_cols_kernel<<<T, 256, 0, st>>>(d16, dst_to_col, out16, H);
    return cudaGetLastError();
}

cudaError_t launch_build_xf(const void* x, int act_dtype, int T, int H, int nblk_pad, bool bf16_mode,
                            uint4* xf, cudaStream_t st) {
    const size_t total = (size_t)T * (H / 32) * 8;
    count_launch();
    if (act_dtype == 0)
        build_xf_kernel<float><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const float*)x, T, H, nblk_pad,
                                                                               bf16_mode, xf);
    else if (act_dtype == 2)
        build_xf_kernel<__half><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const __half*)x, T, H, nblk_pad,
                                                                                bf16_mode, xf);
    else
        build_xf_kernel<__nv_bfloat16><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
            (const __nv_bfloat16*)x, T, H, nblk_pad, bf16_mode, xf);
    return cudaGetLastError();
}

// Caller-supplied routing (expert-parallel ranks receive rows that were routed
// elsewhere): copy the ids, weights default to 1. The reference checks expert_id < E on
// its host path (cuda/moe.rs:1776-1780); here the ids are device data, so the check runs
// on the device: an id >= E raises the context's status word (LUMEN_MOE_INVALID_ARG) and
// the pair is routed to expert 0 with weight 0, so that no table or histogram is ever
// indexed out of range.
__global__ void set_routing_kernel(const uint32_t* __restrict__ ids_in, const float* __restrict__ w_in, int n, int E,
                                   uint32_t* __restrict__ ids, float* __restrict__ w, int32_t* status,
                                   int32_t* status_host) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < n) {
        uint32_t id = ids_in[i];
        float wt = w_in ? w_in[i] : 1.0f;
        if (id >= (uint32_t)E) {
            if (status != nullptr) raise_status(status, status_host, 1);
            id = 0u;
            wt = 0.0f;
        }
        ids[i] = id;
        w[i] = wt;
    }
}

// Router + tables for any T. tile lists are optional (tiles == nullptr skips them).
cudaError_t launch_route_large(const PrefillArgs& a, cudaStream_t st) {
    const int T = a.T, E = a.L.E, H = a.L.H, K = a.K;
    const float* lg = a.logits_override;
    int nparts = 0;
    if (a.ids_in != nullptr) {
        count_launch();
        set_routing_kernel<<<(T * K + 255) / 256, 256, 0, st>>>(a.ids_in, a.weights_in, T * K, E, a.R.ids, a.R.weights,
                                                                a.status, a.status_host);
    } else if (lg == nullptr && a.L.router_w16 != nullptr && a.xr16 != nullptr && a.rpart != nullptr &&
               router_tc_applicable(T, E, H, a.x)) {
        // tcgen05 router: partial logits per k range, summed by the top-k kernel
        nparts = router_tc_ksplit(T, E, H, a.sms > 0 ? a.sms : 148);
        cudaError_t e = launch_router_logits_tc(a.x, a.act_dtype, a.L.router_w16, T, E, H, nparts, a.xr16, a.any_lo,
                                                a.rpart, a.status, a.status_host, a.wait_limit_us, st);
        if (e != cudaSuccess) return e;
        lg = a.rpart;
    } else if (lg == nullptr) {
        count_launch();
        if (H % 32 == 0 && a.w16 != nullptr && reinterpret_cast<uintptr_t>(a.x) % 16 == 0) {
            const size_t n = (size_t)E * H;
            split_router_w_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a.L.router_w, a.w16, n);
            count_launch(1);
            // experts per CTA: fewer for small batches, so that every SM still gets several warps
            const int ne = (T <= 2048) ? 16 : (T <= 16384) ? 32 : 64;
            const dim3 grid((T + 63) / 64, (E + ne - 1) / ne);
#define LUMEN_LAUNCH_LOGITS(XT, NE_) \
    router_logits_mma_kernel<XT, NE_><<<grid, 128, 0, st>>>((const XT*)a.x, a.w16, a.R.logits, T, H, E)
            if (a.act_dtype == 0) {
                if (ne == 16) LUMEN_LAUNCH_LOGITS(float, 16);
                else if (ne == 32) LUMEN_LAUNCH_LOGITS(float, 32);
                else LUMEN_LAUNCH_LOGITS(float, 64);
            } else {
                if (ne == 16) LUMEN_LAUNCH_LOGITS(__nv_bfloat16, 16);
                else if (ne == 32) LUMEN_LAUNCH_LOGITS(__nv_bfloat16, 32);
                else LUMEN_LAUNCH_LOGITS(__nv_bfloat16, 64);
            }
#undef LUMEN_LAUNCH_LOGITS
        } else {
            const dim3 grid((T + 63) / 64, (E + 63) / 64);
            if (a.act_dtype == 0)
                router_logits_large_kernel<float><<<grid, 256, 0, st>>>((const float*)a.x, a.L.router_w, a.R.logits, T, H, E);
            else
                router_logits_large_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a.x, a.L.router_w,
                                                                               a.R.logits, T, H, E);
        }
        lg = a.R.logits;
    }
    count_launch(4);
    const int nchunks = (T + SORT_TOK - 1) / SORT_TOK;
    if (a.ids_in == nullptr)
        CUDA_RET(launch_dep(topk_large_kernel, dim3(nchunks), dim3(TK_WARPS * 32), 0, st, lg, nparts, a.R.logits, T, E, K,
                            a.gating, a.R.ids, a.R.weights, a.blk_hist));
    else
        CUDA_RET(launch_dep(sort_hist_kernel, dim3(nchunks), dim3(256), 0, st, a.R.ids, T, K, E, a.blk_hist));
    const int C = T * K;
    // columns per grouped-GEMM tile: 128 or 256, the same for gate/up and down
    const int tile_cols = tc_gu_tile_cols(C, E), tile_cols_dn = tile_cols;
    const int max_ct = C / tile_cols + E, max_ct_dn = C / tile_cols_dn + E;
    const int mt_gu = a.L.I / 128, mt_dn = a.L.H / 256;  // m-tiles: 128 gate + 128 up rows | 256 down rows
    int4* tiles_gu = a.tiles;
    int4* tiles_dn = a.tiles ? a.tiles + (size_t)max_ct * (mt_gu > 0 ? mt_gu : 1) : nullptr;
    CUDA_RET(launch_dep(sort_rowscan_kernel, dim3(E), dim3(32), 0, st, a.blk_hist, nchunks, a.R));
    CUDA_RET(launch_dep(sort_scan_kernel, dim3(1), dim3(256), 0, st, nchunks, E, a.R, tile_cols, tile_cols_dn, mt_gu, mt_dn,
                        tiles_gu, tiles_dn, a.n_tiles, max_ct * mt_gu, max_ct_dn * mt_dn));
    return launch_dep(sort_place_kernel, dim3((nchunks + 7) / 8), dim3(256), 0, st, a.R.ids, T, K, E, a.blk_hist, nchunks,
                      a.R);
}

cudaError_t launch_tile_plan(const RouteDev& R, int E, int H, int I, int rows_cap, int gu_cols, int4* tiles,
                             int32_t* n_tiles, cudaStream_t st) {
    const int max_ct = rows_cap / gu_cols + E, max_ct_dn = rows_cap / 128 + E;
    const int mt_gu = I / 128, mt_dn = H / 256;
    count_launch();
    // (down tiles of 128 tokens here: an expert-parallel down product stores its rows into other GPUs'
    // memory, which only the always-overlapped epilogue of the 128-token form hides)
    return launch_dep(sort_scan_kernel, dim3(1), dim3(256), 0, st, 0, E, R, gu_cols, 128, mt_gu, mt_dn, tiles,
                      tiles + (size_t)max_ct * (mt_gu > 0 ? mt_gu : 1), n_tiles, max_ct * mt_gu, max_ct_dn * mt_dn);
}

// ---------------------------------------------------------------------------
// Expert-parallel send side in one launch: activation rows gathered in compact-column
// order (= destination-rank order, experts being contiguous per rank) as bf16, the
// expert id of every row relative to its rank, and the number of rows per rank.
// ---------------------------------------------------------------------------
// XT = float: rows leave as f16 (round to nearest, what the grouped GEMM's gather applies to
// f32 activations); XT = bf16: rows leave as bf16, unchanged.
template <typename XT>
__global__ void __launch_bounds__(256)
ep_prepare_kernel(const XT* __restrict__ x, RouteDev R, int H, int E, int epr, uint16_t* __restrict__ rows,
                  int32_t* __restrict__ local_ids, long long* __restrict__ send_counts) {
    const int col = blockIdx.x;
    const int tok = R.col_src_tok[col];
    const XT* src = x + (size_t)tok * H;
    uint16_t* dst = rows + (size_t)col * H;
    for (int i = threadIdx.x * 8; i < H; i += 256 * 8) {
        __align__(16) uint16_t v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (sizeof(XT) == 4) v[j] = __half_as_ushort(__float2half_rn(x_to_f32<XT>(src[i + j])));
            else v[j] = reinterpret_cast<const uint16_t*>(src)[i + j];
        }
        *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(v);
    }
    if (threadIdx.x == 0) local_ids[col] = R.col_expert[col] % epr;
    if (col == 0) {
        for (int r = threadIdx.x; r * epr < E; r += 256)
            send_counts[r] = (long long)(R.expert_bounds[min((r + 1) * epr, E)] - R.expert_bounds[r * epr]);
    }
}

cudaError_t launch_ep_prepare(const void* x, int act_dtype, const RouteDev& R, int C, int H, int E, int epr, void* rows,
                              int32_t* local_ids, long long* send_counts, cudaStream_t st) {
    count_launch();
    if (act_dtype == 0)
        ep_prepare_kernel<float><<<C, 256, 0, st>>>((const float*)x, R, H, E, epr, (uint16_t*)rows, local_ids, send_counts);
    else
        ep_prepare_kernel<__nv_bfloat16><<<C, 256, 0, st>>>((const __nv_bfloat16*)x, R, H, E, epr, (uint16_t*)rows,
                                                            local_ids, send_counts);
    return cudaGetLastError();
}

}  // namespace lumen
