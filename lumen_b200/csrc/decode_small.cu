// Latency-optimised expert kernels for decode batches of 1..4 tokens (every
// expert then has at most 4 columns = one MMA column group).
//
// The general kernels in decode.cu stream a few weight tiles per warp; at batch 1
// the whole layer is only 22 MB, so what counts is to have EVERY byte of a
// kernel's weights requested before the first one is consumed, in a single wave
// of CTAs, and to keep the chain of dependent loads in front of that as short as
// possible. Each CTA reads ONE 32-byte work descriptor written by the router
// (expert, first column, column count, source tokens), each warp then issues all
// of its 128-bit weight loads (registers are the staging buffer), the activation
// fragments of the expert's tokens are staged in shared memory with cp.async
// while the weights are in flight, and only then does the tensor-core loop start.
//
//   gate_up_small_kernel   CTA = (16 rows of I, distinct expert); WARPS warps split
//                          the H/128 input groups, ITERS groups each
//                          (cuda/shaders/moe_expert_q4_0.cu:58-108; moe_expert.cu:62-97)
//   down_small_kernel      CTA = 16 rows of H; warp w walks experts w, w+8, ... with a
//                          ring of RB weight tiles in flight. Its weight loads depend
//                          only on the routing, so they are issued BEFORE the kernel
//                          waits for the gate/up kernel (programmatic dependent launch):
//                          the down weights stream while gate/up is still computing.
//                          Weighted combine in slot order at the end
//                          (moe_expert_q4_0.cu:118-151; cuda/shaders/moe_accum.cu:22-46)
#include "decode_common.cuh"

namespace lumen {

namespace {

using namespace dcommon;

template <int Q>
struct SmallCfg;
template <>
struct SmallCfg<Q4_0> {
    static constexpr int GU_WARPS = 8, GU_ITERS = 2, DN_RING = 6;
};
template <>
struct SmallCfg<Q8_0> {
    static constexpr int GU_WARPS = 8, GU_ITERS = 2, DN_RING = 3;
};
template <>
struct SmallCfg<BF16> {
    static constexpr int GU_WARPS = 16, GU_ITERS = 1, DN_RING = 2;
};

}  // namespace

template <int Q>
__global__ void __launch_bounds__(SmallCfg<Q>::GU_WARPS * 32)
gate_up_small_kernel(const __grid_constant__ DecodeArgs a) {
    constexpr int WARPS = SmallCfg<Q>::GU_WARPS, ITERS = SmallCfg<Q>::GU_ITERS;
    extern __shared__ uint4 xs[];  // [4 columns][2][nblk_pad][4]
    __shared__ float red[WARPS][16][4][2];
    pdl_wait();
    // the router has completed: everything the next kernel reads before ITS wait is final
    pdl_trigger();
    const int u = blockIdx.y;
    const int4 wd = a.R.work[2 * u];
    if (wd.x < 0) return;
    const int4 wt = a.R.work[2 * u + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const int rt = blockIdx.x;
    const int e = wd.x, c0 = wd.y;
    const int kg_h = a.L.kg_h, I = a.L.I;
    const int nblk_pad = kg_h * 4, nblk_i_pad = a.L.kg_i * 4;

    // every weight byte of this warp is requested now
    WTile<Q> wg[ITERS], wu[ITERS];
    {
        const uint4* gq_base = a.L.gate_q(e);
        const uint4* uq_base = a.L.up_q(e);
        const uint4* gs_base = a.L.gate_s(e);
        const uint4* us_base = a.L.up_s(e);
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int kg = warp + it * WARPS;
            if (kg < kg_h) {
                load_wtile<Q>(wg[it], gq_base, gs_base, rt * kg_h + kg, lane);
                load_wtile<Q>(wu[it], uq_base, us_base, rt * kg_h + kg, lane);
            }
        }
    }
    // The expert's columns are taken four at a time (one MMA column group: an expert has at
    // most four columns at batches up to 4, rarely more at batches up to 16); the weights stay
    // in registers across the chunks.
    const int per_col = 2 * nblk_pad * 4;
    const bool int8_act = (Q == Q4_0) && (a.xq != nullptr);
    const int xq_term = xq_term_words(nblk_pad), xq_tok = xq_tok_words(nblk_pad);  // 32-bit words
    for (int cb = 0; cb < wd.z; cb += 4) {
        const int ncol = min(4, wd.z - cb);
        // stage the activation fragments of these columns' tokens (first chunk: while the weights are in flight)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j < ncol) {
                const int tok = (cb == 0) ? (j == 0 ? wt.x : j == 1 ? wt.y : j == 2 ? wt.z : wt.w)
                                          : a.R.col_src_tok[c0 + cb + j];
                if (int8_act) {
                    const uint4* src = reinterpret_cast<const uint4*>(a.xq + (size_t)tok * xq_tok);
                    for (int i = tid; i < xq_tok / 4; i += WARPS * 32) cp_async16(&xs[j * (xq_tok / 4) + i], src + i);
                } else {
                    const uint4* src = a.xf + (size_t)tok * per_col;
                    for (int i = tid; i < per_col; i += WARPS * 32) cp_async16(&xs[j * per_col + i], src + i);
                }
            }
        }
        cp_async_wait_all();
        __syncthreads();

        const int jcol = gq >> 1;
        const bool bvalid = jcol < ncol;
        const uint4* bbase = xs + ((size_t)(jcol * 2 + (gq & 1)) * nblk_pad) * 4 + t4;
        float acc_g[4] = {0.f, 0.f, 0.f, 0.f}, acc_u[4] = {0.f, 0.f, 0.f, 0.f};
        if (Q == Q4_0 && int8_act) {
            // raw nibbles (u8) times the two int8 terms of the activations; n index = 2 * column + term,
            // so acc[0] / acc[2] are rows gq / gq + 8 of the lane's column t4 (acc[1], acc[3] stay zero)
            const unsigned* xqs = reinterpret_cast<const unsigned*>(xs);
            const unsigned* bq0 = xqs + (size_t)jcol * xq_tok + (gq & 1) * xq_term + t4 * 2;
            const float2* sc0 = reinterpret_cast<const float2*>(xqs + (size_t)(t4 < ncol ? t4 : 0) * xq_tok + 2 * xq_term);
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                const int kg = warp + it * WARPS;
                if (kg < kg_h) {
                    const unsigned* bq = bq0 + (kg * 4) * 8;
                    const float2* sc = sc0 + kg * 4;
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        uint2 bb = make_uint2(0u, 0u);
                        if (bvalid) bb = *reinterpret_cast<const uint2*>(bq + b * 8);
                        const uint4 qg = wg[it].q[b >> 1], qu = wu[it].q[b >> 1];
                        const unsigned g0 = (b & 1) ? qg.z : qg.x, g8 = (b & 1) ? qg.w : qg.y;
                        const unsigned u0 = (b & 1) ? qu.z : qu.x, u8 = (b & 1) ? qu.w : qu.y;
                        int cg[4] = {0, 0, 0, 0}, cu[4] = {0, 0, 0, 0};
                        mma_u8s8(cg, g0 & 0x0F0F0F0Fu, g8 & 0x0F0F0F0Fu, (g0 >> 4) & 0x0F0F0F0Fu, (g8 >> 4) & 0x0F0F0F0Fu,
                                 bb.x, bb.y);
                        mma_u8s8(cu, u0 & 0x0F0F0F0Fu, u8 & 0x0F0F0F0Fu, (u0 >> 4) & 0x0F0F0F0Fu, (u8 >> 4) & 0x0F0F0F0Fu,
                                 bb.x, bb.y);
                        const float2 sxo = sc[b];  // {sx, 8 * sx * sum(q)}
                        const float2 sg = block_scales<Q>(wg[it], b), su = block_scales<Q>(wu[it], b);
                        const float k1 = 1.0f / 254.0f;
                        acc_g[0] = fmaf(sg.x, fmaf(sxo.x, fmaf((float)cg[1], k1, (float)cg[0]), -sxo.y), acc_g[0]);
                        acc_g[2] = fmaf(sg.y, fmaf(sxo.x, fmaf((float)cg[3], k1, (float)cg[2]), -sxo.y), acc_g[2]);
                        acc_u[0] = fmaf(su.x, fmaf(sxo.x, fmaf((float)cu[1], k1, (float)cu[0]), -sxo.y), acc_u[0]);
                        acc_u[2] = fmaf(su.y, fmaf(sxo.x, fmaf((float)cu[3], k1, (float)cu[2]), -sxo.y), acc_u[2]);
                    }
                }
            }
        } else {
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                const int kg = warp + it * WARPS;
                if (kg < kg_h) {
                    const uint4* bp = bbase + (size_t)kg * 16;
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        block_mma_smem<Q>(wg[it], b, bp, bvalid, acc_g);
                        block_mma_smem<Q>(wu[it], b, bp, bvalid, acc_u);
                    }
                }
            }
        }
        red[warp][gq][t4][0] = acc_g[0] + acc_g[1];
        red[warp][gq][t4][1] = acc_u[0] + acc_u[1];
        red[warp][gq + 8][t4][0] = acc_g[2] + acc_g[3];
        red[warp][gq + 8][t4][1] = acc_u[2] + acc_u[3];
        __syncthreads();
        if (tid < 64) {
            const int row = tid & 15, tokc = tid >> 4;
            if (tokc < ncol) {
                float gate = 0.0f, up = 0.0f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    gate += red[w][row][tokc][0];
                    up += red[w][row][tokc][1];
                }
                const float sv = (gate / (1.0f + expf(-gate))) * up;
                const int col = c0 + cb + tokc;
                const int irow = rt * 16 + row;
                if (a.s_f32 != nullptr) a.s_f32[(size_t)col * I + irow] = sv;
                store_swiglu_frag<Q>(a.sf, col, irow, nblk_i_pad, sv);
            }
        }
        __syncthreads();  // red and xs are reused by the next chunk
    }
}

constexpr int DS_WARPS = 8;

template <int Q>
__global__ void __launch_bounds__(DS_WARPS * 32)
down_small_kernel(const __grid_constant__ DecodeArgs a) {
    constexpr int RB = SmallCfg<Q>::DN_RING;
    extern __shared__ uint4 ss[];  // [C columns][2][nblk_i_pad][4], then float dsm[C][16]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const int rt = blockIdx.x;
    const int kg_i = a.L.kg_i, H = a.L.H, K = a.K, T = a.T;
    const int nblk_i_pad = kg_i * 4;
    const int C = T * K;
    const int per_col = 2 * nblk_i_pad * 4;
    float* dsm = reinterpret_cast<float*>(ss + (size_t)C * per_col);

    // Routing tables come from the router kernel, which had completed before the
    // gate/up kernel (the immediate predecessor) released this launch; they are
    // read, and the weight loads they determine issued, before waiting for gate/up.
    const int U = *a.R.n_uexp;
    const int n_exp_w = (U > warp) ? (U - warp + DS_WARPS - 1) / DS_WARPS : 0;
    const int nitems = n_exp_w * kg_i;
    auto load_item = [&](int n, WTile<Q>& dst) {
        const int uu = warp + DS_WARPS * (n / kg_i), kg = n % kg_i;
        const int ee = a.R.work[2 * uu].x;
        load_wtile<Q>(dst, a.L.down_q(ee), a.L.down_s(ee), rt * kg_i + kg, lane);
    };
    WTile<Q> ring[RB];
#pragma unroll
    for (int i = 0; i < RB; ++i)
        if (i < nitems) load_item(i, ring[i]);

    pdl_wait();
    pdl_trigger();
    // stage all SwiGLU fragments (written by the gate/up kernel)
    for (int i = tid; i < C * per_col; i += DS_WARPS * 32) cp_async16(&ss[i], a.sf + i);
    cp_async_wait_all();
    __syncthreads();

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int c0 = 0, ncol = 0;
    const uint4* bbase = ss;
    bool bvalid = false;
    for (int n0 = 0; n0 < nitems; n0 += RB) {
#pragma unroll
        for (int i = 0; i < RB; ++i) {
            const int n = n0 + i;
            if (n < nitems) {
                const int kg = n % kg_i;
                if (kg == 0) {
                    const int uu = warp + DS_WARPS * (n / kg_i);
                    const int4 wd = a.R.work[2 * uu];
                    c0 = wd.y;
                    ncol = min(4, wd.z);
                    const int jcol = gq >> 1;
                    bvalid = jcol < ncol;
                    bbase = ss + ((size_t)((c0 + jcol) * 2 + (gq & 1)) * nblk_i_pad) * 4 + t4;
                    acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
                }
                const uint4* bp = bbase + (size_t)kg * 16;
#pragma unroll
                for (int b = 0; b < 4; ++b) block_mma_smem<Q>(ring[i], b, bp, bvalid, acc);
                if (n + RB < nitems) load_item(n + RB, ring[i]);
                if (kg == kg_i - 1 && t4 < ncol) {
                    dsm[(c0 + t4) * 16 + gq] = acc[0] + acc[1];
                    dsm[(c0 + t4) * 16 + gq + 8] = acc[2] + acc[3];
                }
            }
        }
    }
    __syncthreads();
    if (tid < 16 * T) {
        const int row = tid & 15, t = tid >> 4;
        const size_t o = (size_t)t * H + rt * 16 + row;
        float accv = a.residual[o];
        for (int slot = 0; slot < K; ++slot) {
            const int col = a.R.dst_to_col[t * K + slot];
            const float w = a.R.weights[t * K + slot];
            accv = __fadd_rn(accv, __fmul_rn(w, dsm[col * 16 + row]));
        }
        a.out[o] = accv;
    }
}

// ---------------------------------------------------------------------------
// gate/up + SwiGLU for decode batches of 5..16 tokens, Q4_0 with int8 activations: streaming form.
//
// gate_up_small_kernel above is one CTA per (16 rows of I, expert): descriptor, weights,
// products, a reduction across its warps, SwiGLU, a chain of a few microseconds per CTA and 13
// waves of them at 16 tokens. Here a WARP owns a whole item (16 rows of I of one expert with
// work, every input group): it streams the item's gate and up tiles through a ring of its own
// in shared memory (cp.async, GS_RING tile pairs in flight), multiplies them with the int8
// activations of the expert's tokens (the whole batch's, 16 x 4.7 KB, is staged in shared memory
// once per CTA) and finishes the 16 rows itself: no reduction between warps. One CTA of 16 warps per SM;
// items are dealt so that every SM gets the same number of them (+-1).
// (cuda/shaders/moe_expert_q4_0.cu:58-108; SwiGLU cuda/shaders/moe_expert.cu:47-50)
// ---------------------------------------------------------------------------
constexpr int GS_WARPS = 16, GS_RING = 3;
constexpr int GS_TU4 = QTraits<Q4_0>::NQ * 32 + 8;  // uint4 of one raw tile: quant words, then 8 scale words

__global__ void __launch_bounds__(GS_WARPS * 32, 1)
gate_up_stream_kernel(const __grid_constant__ DecodeArgs a) {
    extern __shared__ uint4 gs_ring[];  // [GS_WARPS][GS_RING][gate | up][GS_TU4]
    __shared__ float pair_s[GS_WARPS][4][2];  // [warp][column][absmax | sum] for the partner warp
    pdl_wait();
    pdl_trigger();
    constexpr int NQ32 = QTraits<Q4_0>::NQ * 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const int kg_h = a.L.kg_h, rt_i = a.L.rt_i, I = a.L.I;
    const int nblk_pad = kg_h * 4, nblk_i_pad = a.L.kg_i * 4;
    const int xq_term = xq_term_words(nblk_pad), xq_tok = xq_tok_words(nblk_pad);  // 32-bit words
    const int nitems = *a.R.n_uexp * rt_i;
    uint4* ring = gs_ring + (size_t)warp * GS_RING * 2 * GS_TU4;
    // the batch's int8 activations, staged once (16-byte copies: xq_tok is a multiple of four words)
    unsigned* xq_s = reinterpret_cast<unsigned*>(gs_ring + (size_t)GS_WARPS * GS_RING * 2 * GS_TU4);
    {
        const uint4* src = reinterpret_cast<const uint4*>(a.xq);
        uint4* dst = reinterpret_cast<uint4*>(xq_s);
        const int n16 = a.T * xq_tok / 4;
        for (int i = tid; i < n16; i += GS_WARPS * 32) cp_async16(dst + i, src + i);
        cp_async_wait_all();
        __syncthreads();
    }
    // Warps 2p and 2p+1 of a CTA take the two 16-row halves of the same 32-row block of I, so that
    // together they hold the block an int8 activation scale belongs to (see the epilogue).
    // Pair-major numbering over the grid: consecutive blocks go to different SMs.
    const int sq_term = xq_term_words(nblk_i_pad), sq_tok = xq_tok_words(nblk_i_pad);
    const int half = warp & 1, pair_bar = 1 + (warp >> 1);
    for (int pitem = (warp >> 1) * gridDim.x + blockIdx.x; pitem < nitems / 2; pitem += (GS_WARPS / 2) * gridDim.x) {
        const int u = pitem / (rt_i / 2), blk_i = pitem - u * (rt_i / 2);
        const int rt = blk_i * 2 + half;
        const int4 wd = a.R.work[2 * u];      // {expert, first column, columns}
        const int4 wt = a.R.work[2 * u + 1];  // source tokens of the first four columns
        const int e = wd.x, c0 = wd.y;
        if (e < 0) continue;
        const uint4* gqb = a.L.gate_q(e) + (size_t)rt * kg_h * NQ32 + lane;
        const uint4* uqb = a.L.up_q(e) + (size_t)rt * kg_h * NQ32 + lane;
        const uint4* gsb = a.L.gate_s(e) + (size_t)rt * kg_h * 8;
        const uint4* usb = a.L.up_s(e) + (size_t)rt * kg_h * 8;
        // the expert's columns four at a time (one MMA column group; rarely more than one round)
        for (int cb = 0; cb < wd.z; cb += 4) {
            const int ncol = min(4, wd.z - cb);
            auto tok_of = [&](int j) -> int {
                return (cb == 0) ? (j == 0 ? wt.x : j == 1 ? wt.y : j == 2 ? wt.z : wt.w) : a.R.col_src_tok[c0 + cb + j];
            };
            const int jcol = gq >> 1;          // column of this lane's B fragment (n index = 2 * column + term)
            const bool bvalid = jcol < ncol;
            const int tok_b = tok_of(bvalid ? jcol : 0);
            const int tok_s = tok_of(t4 < ncol ? t4 : 0);  // column of this lane's accumulators
            const unsigned* bq0 = xq_s + (size_t)tok_b * xq_tok + (gq & 1) * xq_term + t4 * 2;
            const float2* sc0 = reinterpret_cast<const float2*>(xq_s + (size_t)tok_s * xq_tok + 2 * xq_term);
            auto issue = [&](int kg) {
                if (kg < kg_h) {
                    uint4* slot = ring + (size_t)(kg % GS_RING) * 2 * GS_TU4;
                    cp_async16(slot + lane, gqb + (size_t)kg * NQ32);
                    cp_async16(slot + 32 + lane, gqb + (size_t)kg * NQ32 + 32);
                    cp_async16(slot + GS_TU4 + lane, uqb + (size_t)kg * NQ32);
                    cp_async16(slot + GS_TU4 + 32 + lane, uqb + (size_t)kg * NQ32 + 32);
                    if (lane < 8) cp_async16(slot + NQ32 + lane, gsb + (size_t)kg * 8 + lane);
                    else if (lane < 16) cp_async16(slot + GS_TU4 + NQ32 + lane - 8, usb + (size_t)kg * 8 + lane - 8);
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            };
#pragma unroll 1
            for (int i = 0; i < GS_RING; ++i) issue(i);
            float acc_g0 = 0.f, acc_g8 = 0.f, acc_u0 = 0.f, acc_u8 = 0.f;  // rows gq, gq + 8 of column t4
#pragma unroll 1
            for (int kg = 0; kg < kg_h; ++kg) {
                asm volatile("cp.async.wait_group %0;" ::"n"(GS_RING - 1) : "memory");
                __syncwarp();  // the scale words of a slot are copied by lanes 0..15 for the whole warp
                const uint4* slot = ring + (size_t)(kg % GS_RING) * 2 * GS_TU4;
                WTile<Q4_0> wg, wu;
                wg.q[0] = slot[lane];
                wg.q[1] = slot[32 + lane];
                wg.s = slot[NQ32 + (lane >> 2)];
                wu.q[0] = slot[GS_TU4 + lane];
                wu.q[1] = slot[GS_TU4 + 32 + lane];
                wu.s = slot[GS_TU4 + NQ32 + (lane >> 2)];
                __syncwarp();  // every lane has its words before the slot is requested again
                issue(kg + GS_RING);
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    // raw nibbles (u8) times the two int8 terms of the activations
                    const uint4 qg = wg.q[b >> 1], qu = wu.q[b >> 1];
                    const unsigned g0 = (b & 1) ? qg.z : qg.x, g8 = (b & 1) ? qg.w : qg.y;
                    const unsigned u0 = (b & 1) ? qu.z : qu.x, u8 = (b & 1) ? qu.w : qu.y;
                    int cg[4] = {0, 0, 0, 0}, cu[4] = {0, 0, 0, 0};
                    uint2 bb = make_uint2(0u, 0u);
                    if (bvalid) bb = *reinterpret_cast<const uint2*>(bq0 + (size_t)(kg * 4 + b) * 8);
                    mma_u8s8(cg, g0 & 0x0F0F0F0Fu, g8 & 0x0F0F0F0Fu, (g0 >> 4) & 0x0F0F0F0Fu, (g8 >> 4) & 0x0F0F0F0Fu,
                             bb.x, bb.y);
                    mma_u8s8(cu, u0 & 0x0F0F0F0Fu, u8 & 0x0F0F0F0Fu, (u0 >> 4) & 0x0F0F0F0Fu, (u8 >> 4) & 0x0F0F0F0Fu,
                             bb.x, bb.y);
                    const float2 sxo = sc0[kg * 4 + b];  // {sx, 8 * sx * sum(q)}
                    const float2 sg = block_scales<Q4_0>(wg, b), su = block_scales<Q4_0>(wu, b);
                    const float k1 = 1.0f / 254.0f;
                    acc_g0 = fmaf(sg.x, fmaf(sxo.x, fmaf((float)cg[1], k1, (float)cg[0]), -sxo.y), acc_g0);
                    acc_g8 = fmaf(sg.y, fmaf(sxo.x, fmaf((float)cg[3], k1, (float)cg[2]), -sxo.y), acc_g8);
                    acc_u0 = fmaf(su.x, fmaf(sxo.x, fmaf((float)cu[1], k1, (float)cu[0]), -sxo.y), acc_u0);
                    acc_u8 = fmaf(su.y, fmaf(sxo.x, fmaf((float)cu[3], k1, (float)cu[2]), -sxo.y), acc_u8);
                }
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            // SwiGLU of rows gq, gq + 8 of column t4, then the block's two-term int8 form for the down
            // product (x ~ sx (q0 + q1 / 254), sx = absmax / 127 over the 32 rows of the block): the
            // absmax and the sum of the quantised values need the partner warp's half, exchanged
            // through shared memory behind a named barrier of the pair.
            const bool cvalid = t4 < ncol;
            const float sv0 = cvalid ? (acc_g0 / (1.0f + expf(-acc_g0))) * acc_u0 : 0.0f;
            const float sv8 = cvalid ? (acc_g8 / (1.0f + expf(-acc_g8))) * acc_u8 : 0.0f;
            const int col = c0 + cb + (cvalid ? t4 : 0);
            if (cvalid && a.s_f32 != nullptr) {
                a.s_f32[(size_t)col * I + rt * 16 + gq] = sv0;
                a.s_f32[(size_t)col * I + rt * 16 + gq + 8] = sv8;
            }
            float am = fmaxf(fabsf(sv0), fabsf(sv8));
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            if (gq == 0) pair_s[warp][t4][0] = am;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            am = fmaxf(am, pair_s[warp ^ 1][t4][0]);
            const float inv = (am > 0.0f) ? 127.0f / am : 0.0f;
            const float sx = am * (1.0f / 127.0f);
            const float r0 = sv0 * inv, r8 = sv8 * inv;
            const float q00 = rintf(r0), q08 = rintf(r8);
            const float q10 = rintf((r0 - q00) * 254.0f), q18 = rintf((r8 - q08) * 254.0f);
            float sum = (q00 + q08) + (q10 + q18) * (1.0f / 254.0f);
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (gq == 0) pair_s[warp][t4][1] = sum;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            if (cvalid) {
                // input i of the block (0..31) is byte i % 4 of word (i % 16) / 4 * 2 + i / 16
                unsigned* sqc = a.sq + (size_t)col * sq_tok;
                signed char* w0 = reinterpret_cast<signed char*>(sqc + blk_i * 8 + (gq >> 2) * 2 + half) + (gq & 3);
                signed char* w8 = reinterpret_cast<signed char*>(sqc + blk_i * 8 + (2 + (gq >> 2)) * 2 + half) + (gq & 3);
                w0[0] = (signed char)(int)q00;
                w8[0] = (signed char)(int)q08;
                w0[(size_t)sq_term * 4] = (signed char)(int)q10;
                w8[(size_t)sq_term * 4] = (signed char)(int)q18;
                if (half == 0 && gq == 0) {
                    const float total = sum + pair_s[warp ^ 1][t4][1];  // first half + second half
                    reinterpret_cast<float2*>(sqc + 2 * sq_term)[blk_i] = make_float2(sx, 8.0f * sx * total);
                }
            }
            __syncwarp();
        }
    }
}

template <typename Kern>
static cudaError_t launch_pdl_smem(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                   const DecodeArgs& a) {
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
    count_launch();
    return cudaLaunchKernelEx(&cfg, kern, a);
}

// Whether the small-batch kernels apply (shape limits of the register staging
// and of shared memory); otherwise the caller uses the general kernels.
bool decode_small_applicable(const DecodeArgs& a, int phase) {
    // gate/up walks an expert's columns four at a time, so it serves every decode batch; the down
    // kernel keeps all SwiGLU fragments in shared memory, which limits it to four tokens
    if (phase != 1 && a.T > 4) return false;
    const int q = a.L.quant;
    const int warps = (q == BF16) ? 16 : 8;
    const int iters = (q == BF16) ? 1 : 2;
    if (a.L.kg_h > warps * iters) return false;
    const size_t gu_smem = (size_t)4 * 2 * a.L.kg_h * 4 * 4 * 16;
    const size_t dn_smem = (size_t)a.T * a.K * (2 * a.L.kg_i * 4 * 4 * 16 + 64);
    return (phase == 1) ? gu_smem <= 160 * 1024 : dn_smem <= 200 * 1024;
}

static size_t gate_up_stream_smem(const DecodeArgs& a) {
    return (size_t)GS_WARPS * GS_RING * 2 * GS_TU4 * 16 + (size_t)a.T * xq_tok_words(a.L.kg_h * 4) * 4;
}

// The streaming gate/up kernel and the int8 down product that consumes its output: Q4_0 layers,
// 2..16 tokens (whenever the three-kernel chain runs; from four tokens on it is also faster than the
// fused kernel), batch activations + rings within shared memory.
bool decode_stream_applicable(const DecodeArgs& a) {
    return a.L.quant == Q4_0 && a.xq != nullptr && a.sq != nullptr && a.T >= 2 && a.T <= DECODE_MAX_TOKENS &&
           a.L.kg_h <= 16 && (a.L.rt_i & 1) == 0 && gate_up_stream_smem(a) <= 220 * 1024;
}

template <int Q>
static cudaError_t launch_small_t(const DecodeArgs& a, int phase, cudaStream_t st) {
    const int C = a.T * a.K;
    const int nu = C < a.L.E ? C : a.L.E;
    if (phase == 1 && decode_stream_applicable(a)) {
        const size_t smem = gate_up_stream_smem(a);
        static SmemOptIn optin_gs;
        cudaError_t e = ensure_dyn_smem(gate_up_stream_kernel, smem, optin_gs);
        if (e != cudaSuccess) return e;
        int device = 0, sms = 0;
        if ((e = cudaGetDevice(&device)) != cudaSuccess) return e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return e;
        return launch_pdl_smem(gate_up_stream_kernel, dim3(sms), dim3(GS_WARPS * 32), smem, st, a);
    }
    if (phase == 1) {
        const size_t smem = (size_t)min(a.T, 4) * 2 * a.L.kg_h * 4 * 4 * 16;
        static SmemOptIn optin_gu;
        cudaError_t e = ensure_dyn_smem(gate_up_small_kernel<Q>, smem, optin_gu);
        if (e != cudaSuccess) return e;
        return launch_pdl_smem(gate_up_small_kernel<Q>, dim3(a.L.rt_i, nu), dim3(SmallCfg<Q>::GU_WARPS * 32), smem, st, a);
    }
    const size_t smem = (size_t)C * (2 * a.L.kg_i * 4 * 4 * 16 + 64);
    static SmemOptIn optin_dn;
    cudaError_t e = ensure_dyn_smem(down_small_kernel<Q>, smem, optin_dn);
    if (e != cudaSuccess) return e;
    return launch_pdl_smem(down_small_kernel<Q>, dim3(a.L.rt_h), dim3(DS_WARPS * 32), smem, st, a);
}

cudaError_t launch_decode_small_phase(const DecodeArgs& a, int phase, cudaStream_t st) {
    switch (a.L.quant) {
        case Q4_0: return launch_small_t<Q4_0>(a, phase, st);
        case Q8_0: return launch_small_t<Q8_0>(a, phase, st);
        default: return launch_small_t<BF16>(a, phase, st);
    }
}

}  // namespace lumen
