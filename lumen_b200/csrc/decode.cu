// Decode path (1..16 tokens) of the MoE FFN: three kernels chained with
// programmatic dependent launch.
//
//   router_small_kernel   one CTA per expert: router logit(s) W_r[e]·x[t]
//                         (moe_router_logits_v2, cuda/shaders/moe_batched.cu:708),
//                         optional fused FFN RMSNorm (cuda/shaders/norm.cu:28-76),
//                         activation fragments; the last CTA to finish (fence +
//                         ticket, no spinning) does gating/top-k/renorm
//                         (cuda/moe.rs:6464-6504) and the stable counting sort
//                         (cuda/moe.rs:2115-2147).
//   gate_up_kernel        per (distinct expert, 16 rows of I): gate and up rows
//                         times the tokens routed to the expert, SwiGLU
//                         (cuda/shaders/moe_expert_q4_0.cu:58-108, moe_expert.cu:62-97).
//                         The general form; Q4_0 layers take gate_up_stream_kernel and the
//                         other small-batch forms of decode_small.cu.
//   down_combine_kernel   per 16 rows of H: down rows of every selected expert
//                         (moe_expert_q4_0.cu:118-151; integer tensor cores on int8 SwiGLU
//                         values after gate_up_stream_kernel) and the weighted combine
//                         out = residual + sum_k w_k d_k in slot order
//                         (cuda/shaders/moe_accum.cu:22-46, cuda/moe.rs:6508-6524).
//
// All three are HBM-bound: each weight byte is read exactly once with 128-bit
// streaming loads, every load of a warp's share is in flight before the first
// use, and the arithmetic runs on the tensor cores (mma_frag.cuh).
#include "decode_common.cuh"
#include <type_traits>
#include "router.cuh"

namespace lumen {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

constexpr int RS_THREADS = 512;  // 16 warps: the last CTA gates one token per warp at batches up to 16
constexpr int RS_WARPS = RS_THREADS / 32;

__global__ void __launch_bounds__(RS_THREADS)
router_small_kernel(const __grid_constant__ DecodeArgs a) {
    __shared__ float red_s[RS_WARPS][DECODE_MAX_TOKENS];
    __shared__ float scale_s[DECODE_MAX_TOKENS];
    __shared__ __align__(16) float p_s[RS_WARPS][MAX_EXPERTS];
    __shared__ __align__(16) float lg_s[RS_WARPS][MAX_EXPERTS];
    __shared__ int ids_s[DECODE_MAX_TOKENS * MAX_TOP_K];
    __shared__ int cnt_s[MAX_EXPERTS];
    __shared__ int cntw_s[DECODE_MAX_TOKENS * MAX_TOP_K / 32][MAX_EXPERTS];
    __shared__ int bounds_s[MAX_EXPERTS + 1];
    __shared__ int uidx_s[MAX_EXPERTS];
    __shared__ int is_last_s;
    __shared__ unsigned long long tab_s[32];

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int e = blockIdx.x;
    const int H = a.L.H, E = a.L.E, T = a.T, K = a.K;
    const int H4 = H >> 2;
    const bool want_logits = (a.logits_override == nullptr);

    // Router row in registers before waiting on the previous kernel (weights are static).
    constexpr int MAXV = 4;  // covers H <= 4096 without re-reading
    float4 wv[MAXV];
    const float4* wrow = reinterpret_cast<const float4*>(a.L.router_w + (size_t)e * H);
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i4 = tid + j * RS_THREADS;
        wv[j] = (want_logits && i4 < H4) ? __ldg(wrow + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();

    // fused FFN RMSNorm scale per token
    if (a.gamma != nullptr) {
        for (int t = 0; t < T; ++t) {
            const float4* xr = reinterpret_cast<const float4*>(a.x + (size_t)t * H);
            float ss = 0.0f;
            for (int i4 = tid; i4 < H4; i4 += RS_THREADS) {
                const float4 v = xr[i4];
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red_s[warp][t] = ss;
        }
        __syncthreads();
        if (tid < T) {
            float ss = 0.0f;
            for (int w = 0; w < RS_WARPS; ++w) ss += red_s[w][tid];
            scale_s[tid] = 1.0f / sqrtf(ss / (float)H + a.eps);
        }
        __syncthreads();
    }
    auto load_x4 = [&](int t, int i4) -> float4 {
        float4 v = reinterpret_cast<const float4*>(a.x + (size_t)t * H)[i4];
        if (a.gamma != nullptr) {
            const float4 g = __ldg(reinterpret_cast<const float4*>(a.gamma) + i4);
            const float sc = scale_s[t];
            v.x = v.x * sc * g.x;
            v.y = v.y * sc * g.y;
            v.z = v.z * sc * g.z;
            v.w = v.w * sc * g.w;
        }
        return v;
    };

    // logits for this expert row, all tokens (token loop rolled: the code of this kernel runs
    // once per launch, so its size is paid in instruction fetches)
    if (want_logits) {
#pragma unroll 4
        for (int t = 0; t < T; ++t) {
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < MAXV; ++j) {
                const int i4 = tid + j * RS_THREADS;
                if (i4 < H4) {
                    const float4 xv = load_x4(t, i4);
                    acc += wv[j].x * xv.x + wv[j].y * xv.y + wv[j].z * xv.z + wv[j].w * xv.w;
                }
            }
#pragma unroll 1
            for (int i4 = tid + MAXV * RS_THREADS; i4 < H4; i4 += RS_THREADS) {  // H > 4096
                const float4 w4 = __ldg(wrow + i4);
                const float4 xv = load_x4(t, i4);
                acc += w4.x * xv.x + w4.y * xv.y + w4.z * xv.z + w4.w * xv.w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) red_s[warp][t] = acc;
        }
        __syncthreads();
        if (tid < T) {
            float v = 0.0f;
            for (int w = 0; w < RS_WARPS; ++w) v += red_s[w][tid];
            a.R.logits[(size_t)tid * E + e] = v;
        }
    }

    // activation operand of the gate/up kernel (and the normed output of the fused-norm entry
    // point): two-term int8 blocks for Q4_0 weights, f16 hi+lo fragments otherwise
    if (a.xq != nullptr) {
        const int nblk = H >> 5, nblk_pad = a.L.kg_h * 4;
        const int sub = tid & 7;
        const int xq_tok = dcommon::xq_tok_words(nblk_pad);
        for (int item = blockIdx.x * (RS_THREADS / 8) + (tid >> 3); item < T * nblk;
             item += gridDim.x * (RS_THREADS / 8)) {
            const int t = item / nblk, b = item - t * nblk;
            const float4 v = load_x4(t, b * 8 + sub);
            dcommon::build_xq_block(v, sub, lane, a.xq + (size_t)t * xq_tok, nblk_pad, b);
            if (a.gamma != nullptr && a.normed_out != nullptr)
                reinterpret_cast<float4*>(a.normed_out + (size_t)t * H)[b * 8 + sub] = v;
        }
    } else if (a.xf != nullptr) {
        const int nblk = H >> 5, nblk_pad = a.L.kg_h * 4;
        const bool bf16_mode = (a.L.quant == BF16);
        const int sub = tid & 7, hl = sub >> 2, t4 = sub & 3;
        for (int item = blockIdx.x * (RS_THREADS / 8) + (tid >> 3); item < T * nblk;
             item += gridDim.x * (RS_THREADS / 8)) {
            const int t = item / nblk, b = item - t * nblk;
            const float4 lo4 = load_x4(t, b * 8 + t4);
            const float4 hi4 = load_x4(t, b * 8 + 4 + t4);
            a.xf[((size_t)(t * 2 + hl) * nblk_pad + b) * 4 + t4] = make_act_frag(lo4, hi4, hl, bf16_mode);
            if (a.gamma != nullptr && a.normed_out != nullptr) {
                float4* o = reinterpret_cast<float4*>(a.normed_out + (size_t)t * H);
                o[b * 8 + (hl ? 4 : 0) + t4] = hl ? hi4 : lo4;
            }
        }
    }

    // last-CTA election: the CTA barrier orders every thread's stores before
    // thread 0's device-scope fence and ticket (fences are cumulative)
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned int ticket = atomicAdd(a.R.ticket, 1u);
        is_last_s = (ticket == gridDim.x - 1);
        if (is_last_s) __threadfence();
    }
    __syncthreads();
    if (!is_last_s) return;

    const float* lg = want_logits ? a.R.logits : a.logits_override;
    if (tid < 32) tab_s[tid] = lumen_exact::exp2_tab_entry(tid);
    __syncthreads();
    // The exact exps are the long part: the 16 warps share a token's exps 4-, 2- or 1-way
    // (consecutive warps form a token's group), then the group's first warp selects.
    {
        const int nsub = (T <= 4) ? 4 : (T <= 8) ? 2 : 1;
        const int t = warp / nsub, sub = warp - t * nsub;
        if (t < T) {
            for (int i = lane; i < E; i += 32) lg_s[warp][i] = __ldcg(lg + (size_t)t * E + i);
            __syncwarp();
            float* p = p_s[warp - sub];
            warp_gate_probs(lg_s[warp], E, a.gating, p, tab_s, sub, nsub);
            if (nsub > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "r"(nsub * 32) : "memory");
            else __syncwarp();
            if (sub == 0) {
                warp_select(p, E, K, a.gating, a.R.ids + (size_t)t * K, a.R.weights + (size_t)t * K);
                if (lane < K) ids_s[t * K + lane] = (int)a.R.ids[(size_t)t * K + lane];
            }
        }
    }
    __syncthreads();
    // Stable counting sort of the C = T*K <= 128 pairs by expert, one pair per thread: pairs
    // of one warp that share an expert rank themselves with a match, and a small table of
    // per-warp counts orders the warps; no loop over the pairs anywhere.
    const int C = T * K;
    const int npw = (C + 31) >> 5;
    for (int i = tid; i < npw * E; i += RS_THREADS) cntw_s[i / E][i % E] = 0;
    __syncthreads();
    int my_e = -1, my_rank = 0;
    if (warp < npw) {
        const int p = warp * 32 + lane;
        my_e = (p < C) ? ids_s[p] : -1 - lane;  // padding lanes match nobody
        const unsigned same = __match_any_sync(0xffffffffu, my_e);
        my_rank = __popc(same & ((1u << lane) - 1u));
        if (p < C && my_rank == 0) cntw_s[warp][my_e] = __popc(same);
    }
    __syncthreads();
    if (tid < E) {
        int c = 0;
        for (int w = 0; w < npw; ++w) c += cntw_s[w][tid];
        cnt_s[tid] = c;
    }
    __syncthreads();
    if (warp == 0) {
        // exclusive scan over experts, 8 per lane (E <= 256), and the ascending
        // list of experts that received at least one token
        int local[8], lsum = 0, lnz = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int ee = lane * 8 + j;
            local[j] = (ee < E) ? cnt_s[ee] : 0;
            lsum += local[j];
            lnz += (local[j] > 0);
        }
        int isum = lsum, inz = lnz;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v1 = __shfl_up_sync(0xffffffffu, isum, o);
            const int v2 = __shfl_up_sync(0xffffffffu, inz, o);
            if (lane >= o) {
                isum += v1;
                inz += v2;
            }
        }
        int run = isum - lsum, unz = inz - lnz;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int ee = lane * 8 + j;
            if (ee < E) {
                bounds_s[ee] = run;
                a.R.expert_bounds[ee] = run;
                uidx_s[ee] = -1;
                if (local[j] > 0) {
                    // work descriptor of the unz-th expert with work: one 32-byte record that a
                    // consumer CTA reads in a single round trip {expert, first column, columns}
                    a.R.work[2 * unz] = make_int4(ee, run, local[j], 0);
                    uidx_s[ee] = unz;
                    a.R.uexp[unz++] = ee;
                }
                run += local[j];
            }
        }
        const int total_u = __shfl_sync(0xffffffffu, inz, 31);
        const int nu_max = (C < E) ? C : E;
        for (int uu = total_u + lane; uu < nu_max; uu += 32) a.R.work[2 * uu] = make_int4(-1, 0, 0, 0);
        if (lane == 31) {
            bounds_s[E] = isum;
            a.R.expert_bounds[E] = isum;
            *a.R.n_uexp = inz;
        }
    }
    __syncthreads();
    if (warp < npw) {
        const int p = warp * 32 + lane;
        if (p < C) {
            int before = my_rank;  // same expert, lower pair index
            for (int w = 0; w < warp; ++w) before += cntw_s[w][my_e];
            const int col = bounds_s[my_e] + before;
            a.R.col_expert[col] = my_e;
            a.R.col_src_tok[col] = p / K;
            a.R.dst_to_col[p] = col;
            // source tokens of the expert's first four columns ride in its work record
            if (before < 4) reinterpret_cast<int*>(a.R.work)[8 * uidx_s[my_e] + 4 + before] = p / K;
        }
    }
    if (tid == 0) *a.R.ticket = 0u;
}

// ---------------------------------------------------------------------------
// gate/up + SwiGLU
// ---------------------------------------------------------------------------
constexpr int GU_THREADS = 256;
constexpr int GU_WARPS = GU_THREADS / 32;

// NG: column groups the code covers (1 or 4). The groups' bodies are predicated, not branched
// around, so a caller that knows there is one group uses NG = 1 and issues a quarter of the code.
template <int Q, int NG = 4>
__device__ __forceinline__ void tile_mma_pair(const WTile<Q>& wg, const WTile<Q>& wu,
                                              const uint4* (&bptr)[4], int ngroups,
                                              float (&acc_g)[4][4], float (&acc_u)[4][4]) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        uint32_t g_lo[4], g_hi[4], u_lo[4], u_hi[4];
        unpack_block<Q>(wg, b, g_lo, g_hi);
        unpack_block<Q>(wu, b, u_lo, u_hi);
        const float2 sg = block_scales<Q>(wg, b);
        const float2 su = block_scales<Q>(wu, b);
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            if (g < ngroups) {
                uint4 bf = make_uint4(0u, 0u, 0u, 0u);
                if (bptr[g] != nullptr) bf = ldg_cached(bptr[g] + b * 4);
                float cg[4] = {0.f, 0.f, 0.f, 0.f}, cu[4] = {0.f, 0.f, 0.f, 0.f};
                if (Q == BF16) {
                    mma_bf16(cg, g_lo, bf.x, bf.y);
                    mma_bf16(cg, g_hi, bf.z, bf.w);
                    mma_bf16(cu, u_lo, bf.x, bf.y);
                    mma_bf16(cu, u_hi, bf.z, bf.w);
                } else {
                    mma_f16(cg, g_lo, bf.x, bf.y);
                    mma_f16(cg, g_hi, bf.z, bf.w);
                    mma_f16(cu, u_lo, bf.x, bf.y);
                    mma_f16(cu, u_hi, bf.z, bf.w);
                }
                acc_g[g][0] = fmaf(sg.x, cg[0], acc_g[g][0]);
                acc_g[g][1] = fmaf(sg.x, cg[1], acc_g[g][1]);
                acc_g[g][2] = fmaf(sg.y, cg[2], acc_g[g][2]);
                acc_g[g][3] = fmaf(sg.y, cg[3], acc_g[g][3]);
                acc_u[g][0] = fmaf(su.x, cu[0], acc_u[g][0]);
                acc_u[g][1] = fmaf(su.x, cu[1], acc_u[g][1]);
                acc_u[g][2] = fmaf(su.y, cu[2], acc_u[g][2]);
                acc_u[g][3] = fmaf(su.y, cu[3], acc_u[g][3]);
            }
        }
    }
}

// Position of element r (0..15 within a half block) inside the 8-half fragment
// vector: quad t = r/4, order within the quad (v0, v2, v1, v3).
__device__ __forceinline__ int frag_pos(int r) {
    const int m = r & 3;
    return (m == 0) ? 0 : (m == 2) ? 1 : (m == 1) ? 2 : 3;
}

template <int Q>
__global__ void __launch_bounds__(GU_THREADS)
gate_up_kernel(const __grid_constant__ DecodeArgs a) {
    __shared__ float red[GU_WARPS][4][16][4][2];  // [warp][group][row][token in group][gate,up]
    // wait first, then release the down kernel: it reads the router's tables before its own wait
    pdl_wait();
    pdl_trigger();
    const int u = blockIdx.y;
    if (u >= *a.R.n_uexp) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const int rt = blockIdx.x;
    const int e = a.R.uexp[u];
    const int c0 = a.R.expert_bounds[e], c1 = a.R.expert_bounds[e + 1];
    const int kg_h = a.L.kg_h, I = a.L.I;
    const int nblk_pad = kg_h * 4, nblk_i_pad = a.L.kg_i * 4;
    const uint4* gq_base = a.L.gate_q(e);
    const uint4* uq_base = a.L.up_q(e);
    const uint4* gs_base = a.L.gate_s(e);
    const uint4* us_base = a.L.up_s(e);

    for (int chunk = c0; chunk < c1; chunk += 16) {
        const int ncol = min(16, c1 - chunk);
        const int ng = (ncol + 3) >> 2;
        const uint4* bbase[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const int col = chunk + 4 * g + (gq >> 1);
            bbase[g] = nullptr;
            if (g < ng && col < c1) {
                const int tok = a.R.col_src_tok[col];
                bbase[g] = a.xf + ((size_t)(tok * 2 + (gq & 1)) * nblk_pad) * 4 + t4;
            }
        }
        float acc_g[4][4], acc_u[4][4];
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc_g[g][i] = acc_u[g][i] = 0.0f;

        WTile<Q> wg, wu, ng_t, nu_t;
        int kg = warp;
        if (kg < kg_h) {
            load_wtile<Q>(wg, gq_base, gs_base, rt * kg_h + kg, lane);
            load_wtile<Q>(wu, uq_base, us_base, rt * kg_h + kg, lane);
        }
        for (; kg < kg_h; kg += GU_WARPS) {
            const bool more = (kg + GU_WARPS) < kg_h;
            if (more) {
                load_wtile<Q>(ng_t, gq_base, gs_base, rt * kg_h + kg + GU_WARPS, lane);
                load_wtile<Q>(nu_t, uq_base, us_base, rt * kg_h + kg + GU_WARPS, lane);
            }
            const uint4* bp[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) bp[g] = bbase[g] ? bbase[g] + (size_t)kg * 16 : nullptr;
            if (ng <= 1) tile_mma_pair<Q, 1>(wg, wu, bp, ng, acc_g, acc_u);
            else tile_mma_pair<Q, 4>(wg, wu, bp, ng, acc_g, acc_u);
            if (more) {
                wg = ng_t;
                wu = nu_t;
            }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            red[warp][g][gq][t4][0] = acc_g[g][0] + acc_g[g][1];
            red[warp][g][gq][t4][1] = acc_u[g][0] + acc_u[g][1];
            red[warp][g][gq + 8][t4][0] = acc_g[g][2] + acc_g[g][3];
            red[warp][g][gq + 8][t4][1] = acc_u[g][2] + acc_u[g][3];
        }
        __syncthreads();
        {
            const int row = tid & 15, tokc = tid >> 4;
            if (tokc < ncol) {
                float gate = 0.0f, up = 0.0f;
#pragma unroll
                for (int w = 0; w < GU_WARPS; ++w) {
                    gate += red[w][tokc >> 2][row][tokc & 3][0];
                    up += red[w][tokc >> 2][row][tokc & 3][1];
                }
                const float sv = (gate / (1.0f + expf(-gate))) * up;
                const int col = chunk + tokc;
                const int irow = rt * 16 + row;
                if (a.s_f32 != nullptr) a.s_f32[(size_t)col * I + irow] = sv;
                const bool bf16_mode = (Q == BF16);
                const int blk = irow >> 5, within = irow & 31, j = within >> 4, r16 = within & 15;
                unsigned short hi_bits, lo_bits;
                if (!bf16_mode) {
                    const __half h = __float2half_rn(sv);
                    const __half l = __float2half_rn(sv - __half2float(h));
                    hi_bits = __half_as_ushort(h);
                    lo_bits = __half_as_ushort(l);
                } else {
                    const __nv_bfloat16 h = __float2bfloat16_rn(sv);
                    const __nv_bfloat16 l = __float2bfloat16_rn(sv - __bfloat162float(h));
                    hi_bits = __bfloat16_as_ushort(h);
                    lo_bits = __bfloat16_as_ushort(l);
                }
                unsigned short* sf16 = reinterpret_cast<unsigned short*>(a.sf);
                const size_t in_vec = (size_t)j * 4 + frag_pos(r16);
                const size_t v_hi = (((size_t)(col * 2 + 0) * nblk_i_pad + blk) * 4 + (r16 >> 2)) * 8 + in_vec;
                const size_t v_lo = (((size_t)(col * 2 + 1) * nblk_i_pad + blk) * 4 + (r16 >> 2)) * 8 + in_vec;
                sf16[v_hi] = hi_bits;
                sf16[v_lo] = lo_bits;
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// down + weighted combine (decode: every expert has at most 16 columns)
// ---------------------------------------------------------------------------
constexpr int DC_THREADS = 512;
constexpr int DC_WARPS = DC_THREADS / 32;
constexpr int DC_MAX_COLS = DECODE_MAX_TOKENS * MAX_TOP_K;

template <int Q>
struct DcRing {  // weight tiles in flight per warp
    static constexpr int value = (Q == Q4_0) ? 6 : (Q == Q8_0) ? 4 : 3;
};

__device__ __forceinline__ void cp_async16_dc(void* smem_dst, const void* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}

// I8 (Q4_0 only): the SwiGLU outputs arrive as two-term int8 blocks (a.sq, written by
// gate_up_stream_kernel) and the products run on the integer tensor cores, raw nibbles against
// int8, as in the gate/up kernels: ~20 instead of ~33 instructions per 32-input block.
template <int Q, bool I8 = false>
__global__ void __launch_bounds__(DC_THREADS)
down_combine_kernel(const __grid_constant__ DecodeArgs a) {
    __shared__ float dsm[DC_MAX_COLS][16];
    __shared__ int exp_s[MAX_EXPERTS], c0_s[MAX_EXPERTS], nc_s[MAX_EXPERTS];
    // The routing tables come from the router kernel, which had completed before the gate/up kernel
    // (the immediate predecessor) released this launch: they are read, and the first weight tiles
    // they determine requested, before waiting for gate/up.
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const int rt = blockIdx.x;
    const int U = *a.R.n_uexp;
    const int kg_i = a.L.kg_i, H = a.L.H, K = a.K, T = a.T;
    const int nblk_i_pad = kg_i * 4;
    // expert id, first column and column count of every expert with work, once per CTA: the
    // per-item lookups below then stay out of the chain of dependent global loads
    for (int u = tid; u < U; u += DC_THREADS) {
        const int ee = a.R.uexp[u];
        const int b0 = a.R.expert_bounds[ee];
        exp_s[u] = ee;
        c0_s[u] = b0;
        nc_s[u] = min(16, a.R.expert_bounds[ee + 1] - b0);
    }
    __syncthreads();

    // flattened (expert, k-group) items of this warp; a ring of DC_RING tiles per warp is kept
    // in flight with cp.async (one commit group per item, empty past the end), so that the
    // bytes in flight per SM cover the HBM latency
    extern __shared__ uint4 dc_ring[];  // [DC_WARPS][DC_RING][NQ * 32 + 8]
    constexpr int NQ32 = QTraits<Q>::NQ * 32, TU4 = NQ32 + 8;
    uint4* my_ring = dc_ring + (size_t)warp * DcRing<Q>::value * TU4;
    const int n_exp_w = (U > warp) ? (U - warp + DC_WARPS - 1) / DC_WARPS : 0;
    const int nitems = n_exp_w * kg_i;
    // (expert slot, k-group) of the next item to request / to prefetch activations for / to multiply:
    // three cursors stepped by one item, no division in the loop
    int is_u = warp, is_kg = 0, is_slot = 0;
    const uint4 *is_q = nullptr, *is_s = nullptr;  // this lane's source words of the next item
    auto issue = [&]() {
        if (is_u < U) {
            if (is_kg == 0) {
                const int ee = exp_s[is_u];
                is_q = a.L.down_q(ee) + (size_t)rt * kg_i * NQ32 + lane;
                is_s = a.L.down_s(ee) + (size_t)rt * kg_i * 8 + lane;
            }
            uint4* slot = my_ring + (size_t)is_slot * TU4;
#pragma unroll
            for (int j = 0; j < QTraits<Q>::NQ; ++j) cp_async16_dc(slot + j * 32 + lane, is_q + j * 32);
            if (Q != BF16 && lane < 8) cp_async16_dc(slot + NQ32 + lane, is_s);
            is_q += NQ32;
            is_s += 8;
            if (++is_kg == kg_i) {
                is_kg = 0;
                is_u += DC_WARPS;
            }
        }
        if (++is_slot == DcRing<Q>::value) is_slot = 0;
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll 1
    for (int i = 0; i < DcRing<Q>::value; ++i) issue();
    pdl_wait();  // the SwiGLU outputs are final from here on
    float acc[4][4];
    int c0 = 0, ncol = 0, ng = 0;
    // activation fragments of the first column group (an expert rarely has more than four columns
    // here) are fetched one item ahead, so that their L2 latency is not paid tile by tile
    const int sq_term = dcommon::xq_term_words(nblk_i_pad), sq_tok = dcommon::xq_tok_words(nblk_i_pad);
    // B operand of block b of item (expert slot u_slot, k-group kgx), column group g. f16 form: the
    // lane's fragment of the hi / lo plane of its column. Int8 form: {word pair of the lane's
    // column and term, {sx, 8 sx sum q} of the column of the lane's accumulators}.
    auto load_b = [&](int u_slot, int kgx, int g, int b) -> uint4 {
        const int ncu = nc_s[u_slot], c0u = c0_s[u_slot];
        const int colr = 4 * g + (gq >> 1);
        if (I8) {
            const int cols = 4 * g + t4;
            uint2 w = make_uint2(0u, 0u);
            if (colr < ncu)
                w = __ldg(reinterpret_cast<const uint2*>(a.sq + (size_t)(c0u + colr) * sq_tok + (gq & 1) * sq_term +
                                                         (size_t)(kgx * 4 + b) * 8 + t4 * 2));
            const float2 sc = __ldg(reinterpret_cast<const float2*>(a.sq + (size_t)(c0u + (cols < ncu ? cols : 0)) * sq_tok +
                                                                    2 * sq_term) + kgx * 4 + b);
            return make_uint4(w.x, w.y, __float_as_uint(sc.x), __float_as_uint(sc.y));
        }
        if (colr >= ncu) return make_uint4(0u, 0u, 0u, 0u);
        return ldg_cached(a.sf + ((size_t)((c0u + colr) * 2 + (gq & 1)) * nblk_i_pad) * 4 + t4 + (size_t)kgx * 16 + b * 4);
    };
    // group 0 of the next item: running pointers, recomputed when the expert changes (null = no column)
    int pb_u = warp, pb_kg = 0;
    const unsigned* pb_w = nullptr;  // int8 form: word pairs of the lane's column and term | f16 form: fragments
    const float2* pb_s = nullptr;    // int8 form: scales of the column of the lane's accumulators
    uint4 bnx[4];
    auto b0_next = [&]() {
        if (pb_u < U) {
            if (pb_kg == 0) {
                const int ncu = nc_s[pb_u], c0u = c0_s[pb_u];
                const int colr = gq >> 1;
                if (I8) {
                    pb_w = (colr < ncu) ? a.sq + (size_t)(c0u + colr) * sq_tok + (gq & 1) * sq_term + t4 * 2 : nullptr;
                    pb_s = reinterpret_cast<const float2*>(a.sq + (size_t)(c0u + (t4 < ncu ? t4 : 0)) * sq_tok + 2 * sq_term);
                } else {
                    pb_w = (colr < ncu) ? reinterpret_cast<const unsigned*>(
                                              a.sf + ((size_t)((c0u + colr) * 2 + (gq & 1)) * nblk_i_pad) * 4 + t4)
                                        : nullptr;
                }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (I8) {
                    const uint2 w = pb_w ? __ldg(reinterpret_cast<const uint2*>(pb_w) + b * 4) : make_uint2(0u, 0u);
                    const float2 sc = __ldg(pb_s + b);
                    bnx[b] = make_uint4(w.x, w.y, __float_as_uint(sc.x), __float_as_uint(sc.y));
                } else {
                    bnx[b] = pb_w ? ldg_cached(reinterpret_cast<const uint4*>(pb_w) + b * 4) : make_uint4(0u, 0u, 0u, 0u);
                }
            }
            if (pb_w) pb_w += I8 ? 32 : 64;  // one k-group on: 4 blocks x 8 words | 16 uint4
            pb_s += 4;
            if (++pb_kg == kg_i) {
                pb_kg = 0;
                pb_u += DC_WARPS;
            }
        } else {
#pragma unroll
            for (int b = 0; b < 4; ++b) bnx[b] = make_uint4(0u, 0u, 0u, 0u);
        }
    };
    b0_next();
    int uu = warp - DC_WARPS, kg = kg_i - 1, rslot = 0;
#pragma unroll 1
    for (int n = 0; n < nitems; ++n) {
        asm volatile("cp.async.wait_group %0;" ::"n"(DcRing<Q>::value - 1) : "memory");
        __syncwarp();
        WTile<Q> cur;
        {
            const uint4* slot = my_ring + (size_t)rslot * TU4;
#pragma unroll
            for (int j = 0; j < QTraits<Q>::NQ; ++j) cur.q[j] = slot[j * 32 + lane];
            if (Q != BF16) cur.s = slot[NQ32 + (lane >> 2)];
            if (++rslot == DcRing<Q>::value) rslot = 0;
        }
        __syncwarp();
        issue();  // refill the slot just read
        uint4 bcur[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) bcur[b] = bnx[b];
        b0_next();
        if (++kg == kg_i) {
            kg = 0;
            uu += DC_WARPS;
        }
        if (kg == 0) {
            c0 = c0_s[uu];
            ncol = nc_s[uu];
            ng = (ncol + 3) >> 2;
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[g][i] = 0.0f;
        }
        // Group 0 from the prefetched registers, further groups fetched in place. An expert with more
        // than four columns is rare in a decode batch, so the one-group case gets code of its own:
        // in the four-group form the compiler predicates the other groups' bodies instead of
        // branching around them, and a tile then costs ~400 issued instructions instead of ~150.
        auto tile_blocks = [&](auto ng_tag) {
            constexpr int NG = decltype(ng_tag)::value;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float2 sc = block_scales<Q>(cur, b);
                if (I8) {
                    const uint4 qv = cur.q[(b >> 1) % QTraits<Q>::NQ];
                    const unsigned w0 = (b & 1) ? qv.z : qv.x, w8 = (b & 1) ? qv.w : qv.y;
                    const unsigned a0 = w0 & 0x0F0F0F0Fu, a1 = w8 & 0x0F0F0F0Fu;
                    const unsigned a2 = (w0 >> 4) & 0x0F0F0F0Fu, a3 = (w8 >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                    for (int g = 0; g < NG; ++g) {
                        if (g == 0 || g < ng) {
                            const uint4 bf = (g == 0) ? bcur[b] : load_b(uu, kg, g, b);
                            int c[4] = {0, 0, 0, 0};
                            dcommon::mma_u8s8(c, a0, a1, a2, a3, bf.x, bf.y);
                            const float sx = __uint_as_float(bf.z), off = __uint_as_float(bf.w);
                            const float k1 = 1.0f / 254.0f;
                            acc[g][0] = fmaf(sc.x, fmaf(sx, fmaf((float)c[1], k1, (float)c[0]), -off), acc[g][0]);
                            acc[g][2] = fmaf(sc.y, fmaf(sx, fmaf((float)c[3], k1, (float)c[2]), -off), acc[g][2]);
                        }
                    }
                } else {
                    uint32_t a_lo[4], a_hi[4];
                    unpack_block<Q>(cur, b, a_lo, a_hi);
#pragma unroll
                    for (int g = 0; g < NG; ++g) {
                        if (g == 0 || g < ng) {
                            const uint4 bf = (g == 0) ? bcur[b] : load_b(uu, kg, g, b);
                            float c[4] = {0.f, 0.f, 0.f, 0.f};
                            if (Q == BF16) {
                                mma_bf16(c, a_lo, bf.x, bf.y);
                                mma_bf16(c, a_hi, bf.z, bf.w);
                            } else {
                                mma_f16(c, a_lo, bf.x, bf.y);
                                mma_f16(c, a_hi, bf.z, bf.w);
                            }
                            acc[g][0] = fmaf(sc.x, c[0], acc[g][0]);
                            acc[g][1] = fmaf(sc.x, c[1], acc[g][1]);
                            acc[g][2] = fmaf(sc.y, c[2], acc[g][2]);
                            acc[g][3] = fmaf(sc.y, c[3], acc[g][3]);
                        }
                    }
                }
            }
        };
        if (ng <= 1) tile_blocks(std::integral_constant<int, 1>{});
        else tile_blocks(std::integral_constant<int, 4>{});
        if (kg == kg_i - 1) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int tokc = 4 * g + t4;
                if (tokc < ncol) {
                    dsm[c0 + tokc][gq] = acc[g][0] + acc[g][1];
                    dsm[c0 + tokc][gq + 8] = acc[g][2] + acc[g][3];
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    {
        const int row = tid & 15, t = tid >> 4;
        if (t < T) {
            const size_t o = (size_t)t * H + rt * 16 + row;
            float accv = a.residual[o];
            for (int slot = 0; slot < K; ++slot) {
                const int col = a.R.dst_to_col[t * K + slot];
                const float w = a.R.weights[t * K + slot];
                accv = __fadd_rn(accv, __fmul_rn(w, dsm[col][row]));
            }
            a.out[o] = accv;
        }
    }
}

// ---------------------------------------------------------------------------
// down projection for any number of columns per expert (mma.sync grouped path of
// the prefill entry point): one CTA per (16 rows of H, expert), k-groups split
// across warps, output f16 by compact column for the scatter-accumulate.
// ---------------------------------------------------------------------------
template <int Q>
__global__ void __launch_bounds__(GU_THREADS)
down_general_kernel(const __grid_constant__ DecodeArgs a, __half* __restrict__ d16) {
    __shared__ float red[GU_WARPS][4][16][4];
    const int u = blockIdx.y;
    if (u >= *a.R.n_uexp) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const int rt = blockIdx.x;
    const int e = a.R.uexp[u];
    const int c0 = a.R.expert_bounds[e], c1 = a.R.expert_bounds[e + 1];
    const int kg_i = a.L.kg_i, H = a.L.H;
    const int nblk_i_pad = kg_i * 4;
    const uint4* q_base = a.L.down_q(e);
    const uint4* s_base = a.L.down_s(e);
    for (int chunk = c0; chunk < c1; chunk += 16) {
        const int ncol = min(16, c1 - chunk);
        const int ng = (ncol + 3) >> 2;
        const uint4* bbase[4];
        float acc[4][4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const int colr = 4 * g + (gq >> 1);
            bbase[g] = (colr < ncol)
                           ? a.sf + ((size_t)((chunk + colr) * 2 + (gq & 1)) * nblk_i_pad) * 4 + t4
                           : nullptr;
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[g][i] = 0.0f;
        }
        for (int kg = warp; kg < kg_i; kg += GU_WARPS) {
            WTile<Q> w;
            load_wtile<Q>(w, q_base, s_base, rt * kg_i + kg, lane);
            const uint4* bp[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) bp[g] = bbase[g] ? bbase[g] + (size_t)kg * 16 : nullptr;
            tile_mma<Q, 4>(w, bp, ng, acc);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            red[warp][g][gq][t4] = acc[g][0] + acc[g][1];
            red[warp][g][gq + 8][t4] = acc[g][2] + acc[g][3];
        }
        __syncthreads();
        {
            const int row = tid & 15, tokc = tid >> 4;
            if (tokc < ncol) {
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < GU_WARPS; ++w) v += red[w][tokc >> 2][row][tokc & 3];
                d16[(size_t)(chunk + tokc) * H + rt * 16 + row] = __float2half_rn(v);
            }
        }
        __syncthreads();
    }
}

cudaError_t launch_grouped_mma(const DecodeArgs& a, __half* d16, cudaStream_t st) {
    const dim3 g_gu(a.L.rt_i, a.L.E), g_dn(a.L.rt_h, a.L.E);
    count_launch(2);
    switch (a.L.quant) {
        case Q4_0:
            gate_up_kernel<Q4_0><<<g_gu, GU_THREADS, 0, st>>>(a);
            down_general_kernel<Q4_0><<<g_dn, GU_THREADS, 0, st>>>(a, d16);
            break;
        case Q8_0:
            gate_up_kernel<Q8_0><<<g_gu, GU_THREADS, 0, st>>>(a);
            down_general_kernel<Q8_0><<<g_dn, GU_THREADS, 0, st>>>(a, d16);
            break;
        default:
            gate_up_kernel<BF16><<<g_gu, GU_THREADS, 0, st>>>(a);
            down_general_kernel<BF16><<<g_dn, GU_THREADS, 0, st>>>(a, d16);
            break;
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// launch
// ---------------------------------------------------------------------------
template <typename Kern>
static cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, cudaStream_t st, const DecodeArgs& a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    count_launch();
    return cudaLaunchKernelEx(&cfg, kern, a);
}

template <int Q, bool I8 = false>
static cudaError_t launch_down_combine(const DecodeArgs& a, dim3 grid, cudaStream_t st) {
    const size_t smem = (size_t)DC_WARPS * DcRing<Q>::value * (QTraits<Q>::NQ * 32 + 8) * 16;
    static SmemOptIn optin;
    {
        cudaError_t e = ensure_dyn_smem(down_combine_kernel<Q, I8>, smem, optin);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    count_launch();
    return cudaLaunchKernelEx(&cfg, down_combine_kernel<Q, I8>, a);
}

cudaError_t launch_route_small(const DecodeArgs& a, cudaStream_t st) {
    return launch_pdl(router_small_kernel, dim3(a.L.E), dim3(RS_THREADS), st, a);
}

bool decode_small_applicable(const DecodeArgs& a, int phase);
bool decode_stream_applicable(const DecodeArgs& a);
cudaError_t launch_decode_small_phase(const DecodeArgs& a, int phase, cudaStream_t st);

cudaError_t launch_decode_phase(const DecodeArgs& a_in, int phase, cudaStream_t st) {
    // the int8 activation form belongs to the Q4_0 gate/up kernel that walks columns four at a time
    DecodeArgs a = a_in;
    if (!(a.xq != nullptr && a.xf != nullptr && a.L.quant == Q4_0 && decode_small_applicable(a, 1))) a.xq = nullptr;
    // 5..16 tokens, Q4_0: streaming gate/up that hands the down product int8 activations
    const bool stream = decode_stream_applicable(a);
    if (!stream) a.sq = nullptr;
    if (phase == 0) return launch_route_small(a, st);
    if (stream && phase == 2) return launch_down_combine<Q4_0, true>(a, dim3(a.L.rt_h), st);  // consumes the int8 SwiGLU values
    if (decode_small_applicable(a, phase)) return launch_decode_small_phase(a, phase, st);
    const int C = a.T * a.K;
    const int nu = C < a.L.E ? C : a.L.E;
    const dim3 g_gu(a.L.rt_i, nu), g_dc(a.L.rt_h);
    if (phase == 1) {
        switch (a.L.quant) {
            case Q4_0: return launch_pdl(gate_up_kernel<Q4_0>, g_gu, dim3(GU_THREADS), st, a);
            case Q8_0: return launch_pdl(gate_up_kernel<Q8_0>, g_gu, dim3(GU_THREADS), st, a);
            default: return launch_pdl(gate_up_kernel<BF16>, g_gu, dim3(GU_THREADS), st, a);
        }
    }
    switch (a.L.quant) {
        case Q4_0: return launch_down_combine<Q4_0>(a, g_dc, st);
        case Q8_0: return launch_down_combine<Q8_0>(a, g_dc, st);
        default: return launch_down_combine<BF16>(a, g_dc, st);
    }
}

bool decode_fused_applicable(const DecodeArgs& a);
cudaError_t launch_decode_fused(const DecodeArgs& a, cudaStream_t st);

// Which form a decode call takes. The persistent fused kernel wins up to three tokens; at four
// tokens on a Q4_0 layer the chain with the streaming gate/up kernel and the int8 down product is
// faster (35.5 against 38.1 us per layer call; 31.9 / 30.6 at three, 26.1 / 23.9 at two).
bool decode_uses_fused(const DecodeArgs& a) {
    if (!decode_fused_applicable(a)) return false;
    return !(a.T >= 4 && decode_stream_applicable(a));
}

cudaError_t launch_decode(const DecodeArgs& a, cudaStream_t st) {
    if (decode_uses_fused(a)) return launch_decode_fused(a, st);
    for (int phase = 0; phase < 3; ++phase) {
        const cudaError_t err = launch_decode_phase(a, phase, st);
        if (err != cudaSuccess) return err;
    }
    return cudaSuccess;
}

}  // namespace lumen
