// One persistent kernel for a whole MoE layer call at decode batches of 1..4 tokens.
//
// The three-kernel chain (router -> gate/up -> down) pays a kernel boundary twice;
// at batch 1 a layer is only ~22 MB of weights, so those boundaries cost more than
// the streaming itself. Here one CTA per SM stays resident and the two boundaries
// become grid barriers:
//
//   phase A  router logit of expert row(s) e = CTA, CTA + G, ... (cuda/moe.rs:1119-1140);
//            every CTA also builds the activation fragments of all tokens in its own
//            shared memory (and the fused FFN RMSNorm scale when asked)
//   barrier 1
//   phase B  every CTA redoes the (tiny) top-k and counting sort from the logits, so the
//            routing never makes a second trip through memory; CTA 0 publishes the tables.
//            gate/up + SwiGLU work items (expert with work, 16 inter rows), dealt
//            round-robin from the last CTA downwards; each warp owns one 128-input
//            group; an item's weight tiles arrive by bulk copies (cp.async.bulk on
//            mbarriers) through a ring of up to three items, requested for the expert set
//            predicted from the raw logits while the exact gating still runs. The
//            down-projection weights of this CTA's 16 output rows are requested the same way.
//            (cuda/shaders/moe_expert_q4_0.cu:58-108; moe_expert.cu:62-97)
//   barrier 2
//   phase C  down product for output rows 16*CTA.., all experts with work; weighted
//            combine in slot order + residual
//            (moe_expert_q4_0.cu:118-151; cuda/shaders/moe_accum.cu:22-46)
//
// The barrier is an arrival counter that only grows, so nothing is reset between
// launches; every wait is bounded (one second), after which the kernel raises the
// context's status word and every CTA returns.
#include "decode_common.cuh"
#include "router.cuh"

namespace lumen {

namespace {

using namespace dcommon;

constexpr int FW = 16;        // warps per CTA
constexpr int FT = FW * 32;   // threads per CTA
constexpr int FMAX_T = 4;     // tokens
constexpr int FMAX_C = 32;    // (token, slot) pairs

// n / d for 0 <= n < 2^20 and a divisor known when the kernel starts: one multiply by the
// float reciprocal and a fix-up instead of the ~25-instruction integer division sequence
// (these quotients sit in dependency chains that run once per launch).
struct SmallDiv {
    int d;
    float inv;
    __device__ __forceinline__ explicit SmallDiv(int dd) : d(dd), inv(1.0f / (float)dd) {}
    __device__ __forceinline__ int div(int n) const {
        int q = (int)(((float)n + 0.5f) * inv);
        const int r = n - q * d;
        q += (r >= d) - (r < 0);
        return q;
    }
};

template <int Q>
struct TileU4 {  // uint4 words of one weight tile staged in shared memory: lane-major q words, then 8 scale words
    static constexpr int value = QTraits<Q>::NQ * 32 + 8;
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add_u32(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Barrier 1 carries its payload: each logit travels as one 8-byte word {value, launch tag},
// written with a single store and polled by one thread per (token, expert) until the tag is
// this launch's: when the wait is over the logits are already in hand (one L2 round trip
// instead of flag + data).
__device__ __forceinline__ void st_tagged(float* slot, float v, unsigned tag) {
    asm volatile("st.relaxed.gpu.global.v2.b32 [%0], {%1, %2};" ::"l"(slot), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_tagged(const float* slot) {
    uint2 r;
    asm volatile("ld.relaxed.gpu.global.v2.b32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(slot) : "memory");
    return r;
}

// Grid barrier: one arrival counter that only grows (bar[0]); barrier number `epoch`
// (counted per CTA in bar[1 + cta], written by that CTA alone) is passed when the
// counter reaches epoch * G, compared modulo 2^32, so nothing is reset between
// launches. Arriving is one fire-and-forget reduction by thread 0 (call it after a
// __syncthreads that follows the CTA's last store); one thread per CTA polls.
__device__ __forceinline__ void grid_arrive(unsigned* bar) {
    if (threadIdx.x == 0) red_release_add_u32(bar, 1u);
}

// Returns false when the wait expired (one second) or another CTA already raised the
// status word.
struct WaitCtl {
    int* status;
    int* status_host;
    unsigned long long limit_ns;
};

__device__ __forceinline__ bool grid_wait(unsigned* bar, const WaitCtl& wc, int G, unsigned epoch, int extra,
                                          int* fail_s) {
    if (threadIdx.x == 0) {
        const unsigned target = epoch * (unsigned)G + (unsigned)extra;
        unsigned long long t0 = 0;
        unsigned spins = 0;
        bool ok = true;
        while ((int)(ld_relaxed_u32(bar) - target) < 0) {
            if ((++spins & 63u) == 0) {
                if (t0 == 0) t0 = global_ns();
                if (global_ns() - t0 > wc.limit_ns || *reinterpret_cast<volatile int*>(wc.status) != 0) {
                    ok = false;
                    break;
                }
            }
        }
        __threadfence();
        if (!ok) {
            raise_status(wc.status, wc.status_host, 4);  // LUMEN_MOE_TIMEOUT
            *fail_s = 1;
        }
    }
    __syncthreads();
    return *fail_s == 0;
}

// mbarrier + bulk-copy helpers: a weight tile range is contiguous in the fragment planes, so
// one cp.async.bulk moves all input groups of a work item's matrix at once.
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, unsigned bytes, void* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ bool mbar_try(void* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait (one second unless the launch says otherwise); false when it expired or the
// status word is already raised.
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, const WaitCtl& wc) {
    if (mbar_try(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (unsigned i = 0;; ++i) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 63u) == 63u) {
            if (global_ns() - t0 > wc.limit_ns || *reinterpret_cast<volatile int*>(wc.status) != 0) {
                raise_status(wc.status, wc.status_host, 4);  // LUMEN_MOE_TIMEOUT
                return false;
            }
        }
    }
}

// One lane's share of a staged tile: q words of the tile at qp (lane-major), scale words at sp.
template <int Q>
__device__ __forceinline__ void read_staged(WTile<Q>& w, const uint4* qp, const uint4* sp, int lane) {
#pragma unroll
    for (int j = 0; j < QTraits<Q>::NQ; ++j) w.q[j] = qp[j * 32 + lane];
    if (Q != BF16) w.s = sp[lane >> 2];
}

struct RouteSm {
    int ids[FMAX_C];
    float w[FMAX_C];
    int d2c[FMAX_C];      // pair -> column
    int col_u[FMAX_C];    // column -> index of its expert in the list of experts with work
    int col_tok[FMAX_C];  // column -> source token
    int ue[FMAX_C];       // experts with work, ascending
    int uc0[FMAX_C];      // first column of the expert
    int uncol[FMAX_C];    // columns of the expert
    int U;
    int pr_ue[FMAX_C];    // experts with work as predicted from the raw logits, ascending
    int pr_U;
    unsigned pr_mask[MAX_EXPERTS / 32];
};

// Q4_0 gate/up at decode runs on the integer tensor-core path: the nibbles go in as
// they are (unsigned, two AND/shift pairs per 32 weights instead of the sixteen
// instructions of the exact-f16 unpack), the activations as a two-term int8 split
// x ~ sx * (q0 + q1 / 254) with one f32 scale per 32-block (|error| <= amax_block * 1.6e-5),
// q0 and q1 in adjacent MMA columns; the -8 offset of the nibbles is taken out with the
// block's precomputed 8 * sx * sum(q0 + q1 / 254).
constexpr bool kInt8GateUp = true;

struct TopkSm {
    float lg[FMAX_T][MAX_EXPERTS];
    float p[FMAX_T][MAX_EXPERTS];
    unsigned long long tab[32];  // copy of the exp table: lanes index it divergently
};

}  // namespace

template <int Q>
__global__ void __launch_bounds__(FT, 1)
decode_fused_kernel(const __grid_constant__ DecodeArgs a, const int pf_experts, const int gs_slots, const int gs_alias) {
    extern __shared__ uint4 dyn[];
    __shared__ __align__(16) TopkSm ts;
    __shared__ float red_a[FW][FMAX_T];
    __shared__ float scale_s[FMAX_T];
    __shared__ float red[FW][16][4][2];
    __shared__ RouteSm rs;
    __shared__ int fail_s;
    __shared__ __align__(8) unsigned long long mbar[8];  // 0..6: staged gate/up items, 7: staged down tiles

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    auto stamp = [&](int i) {
        if (a.trace != nullptr && tid == 0) a.trace[(size_t)blockIdx.x * 12 + i] = global_ns();
    };
    stamp(0);
    if (tid < 32) ts.tab[tid] = lumen_exact::exp2_tab_entry(tid);
    if (tid == 0) {
        fail_s = 0;
        for (int i = 0; i < 8; ++i) mbar_init(&mbar[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int gq = lane >> 2, t4 = lane & 3;
    const int cta = blockIdx.x, G = gridDim.x;
    const int H = a.L.H, I = a.L.I, E = a.L.E, T = a.T, K = a.K;
    const int C = T * K;
    const int H4 = H >> 2;
    const int kg_h = a.L.kg_h, kg_i = a.L.kg_i;
    const int nblk = H >> 5, nblk_pad = kg_h * 4, nblk_i_pad = kg_i * 4;
    const int per_col = 2 * nblk_pad * 4, per_col_i = 2 * nblk_i_pad * 4;
    const bool want_logits = (a.logits_override == nullptr);
    constexpr int TU4 = TileU4<Q>::value;
    const WaitCtl wc{a.status, a.status_host, a.wait_limit_us ? (unsigned long long)a.wait_limit_us * 1000ull : 1000000000ull};

    // dynamic shared memory: activation fragments | SwiGLU fragments | down partial sums | staged down tiles
    uint4* xs = dyn;                                  // [T][per_col]
    uint4* ss = xs + (size_t)T * per_col;             // [C][per_col_i]
    float* part = reinterpret_cast<float*>(ss + (size_t)C * per_col_i);  // [C * kg_i][4 cols][16 rows]
    float* wd = part + (size_t)C * kg_i * 64;         // [C][16] weighted expert outputs
    // the f32 activations of phase A share the ss/part/wd region, whichever is larger
    const size_t mid_bytes = max((size_t)C * per_col_i * 16 + (size_t)C * kg_i * 256 + (size_t)C * 64, (size_t)T * H * 4);
    // staged down tiles of this CTA's 16 output rows: [pf_experts][q of kg_i tiles | scales of kg_i tiles]
    uint4* pf = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(ss) + mid_bytes);
    // staged gate/up tiles: a ring of gs_slots work items, each [gate | up][q of kg_h tiles | scales
    // of kg_h tiles]. The first gs_alias slots lie over the ss/part/wd region, which is only
    // written after every gate/up item has been consumed (phase C); the rest follow the down tiles.
    uint4* gs = pf + (size_t)pf_experts * kg_i * TU4;
    constexpr int NQ32 = QTraits<Q>::NQ * 32;
    const size_t item_u4 = (size_t)2 * kg_h * TU4;
    auto gs_slot = [&](int sl) -> uint4* {
        return sl < gs_alias ? ss + (size_t)sl * item_u4 : gs + (size_t)(sl - gs_alias) * item_u4;
    };
    const SmallDiv div_kgi(kg_i), div_rti(a.L.rt_i), div_g(G);

    // ---------------- phase A ----------------
    // first router row in registers before waiting on the previous kernel (weights are static)
    float4 wv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (want_logits && cta < E && tid < H4)
        wv = __ldg(reinterpret_cast<const float4*>(a.L.router_w + (size_t)cta * H) + tid);
    pdl_wait();
    stamp(1);
    // Thread i holds inputs 4i..4i+3 of every token (H <= 4 * FT): they feed the router
    // dot products straight from registers; the status word and this CTA's barrier count
    // are requested in the same round trip.
    float4 xv[FMAX_T];
#pragma unroll
    for (int t = 0; t < FMAX_T; ++t)
        xv[t] = (t < T && tid < H4) ? reinterpret_cast<const float4*>(a.x)[t * H4 + tid] : make_float4(0.f, 0.f, 0.f, 0.f);
    const int status_now = *reinterpret_cast<volatile int*>(a.status);
    unsigned epoch = *reinterpret_cast<volatile unsigned*>(a.bar + 1 + cta);  // barriers this CTA has passed so far
    if (status_now != 0) return;  // an earlier launch gave up: do not touch the barrier

    // normalised activations of all tokens, f32, in shared memory for the fragment build (the
    // region is reused for the SwiGLU fragments and partial sums, written only after the routing)
    float4* xn4 = reinterpret_cast<float4*>(ss);
    if (a.gamma != nullptr) {
#pragma unroll
        for (int t = 0; t < FMAX_T; ++t) {
            if (t < T) {
                float sq = xv[t].x * xv[t].x + xv[t].y * xv[t].y + xv[t].z * xv[t].z + xv[t].w * xv[t].w;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (lane == 0) red_a[warp][t] = sq;
            }
        }
        __syncthreads();
        if (tid < T) {
            float sq = 0.0f;
#pragma unroll
            for (int w = 0; w < FW; ++w) sq += red_a[w][tid];
            scale_s[tid] = 1.0f / sqrtf(sq / (float)H + a.eps);
        }
        __syncthreads();
        if (tid < H4) {
            const float4 g = __ldg(reinterpret_cast<const float4*>(a.gamma) + tid);
#pragma unroll
            for (int t = 0; t < FMAX_T; ++t) {
                if (t < T) {
                    const float sc = scale_s[t];
                    xv[t].x = xv[t].x * sc * g.x;
                    xv[t].y = xv[t].y * sc * g.y;
                    xv[t].z = xv[t].z * sc * g.z;
                    xv[t].w = xv[t].w * sc * g.w;
                    if (a.normed_out != nullptr && (tid % G) == cta)
                        reinterpret_cast<float4*>(a.normed_out)[t * H4 + tid] = xv[t];
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < FMAX_T; ++t)
        if (t < T && tid < H4) xn4[t * H4 + tid] = xv[t];

    if (want_logits) {
#pragma unroll 1
        for (int e = cta; e < E; e += G) {
            float4 w4 = wv;
            if (e != cta && tid < H4) w4 = __ldg(reinterpret_cast<const float4*>(a.L.router_w + (size_t)e * H) + tid);
#pragma unroll
            for (int t = 0; t < FMAX_T; ++t) {
                if (t < T) {
                    float acc = w4.x * xv[t].x + w4.y * xv[t].y + w4.z * xv[t].z + w4.w * xv[t].w;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    if (lane == 0) red_a[warp][t] = acc;
                }
            }
            __syncthreads();
            if (tid < T) {
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < FW; ++w) v += red_a[w][tid];
                st_tagged(a.R.logits + 2 * ((size_t)tid * E + e), v, epoch + 1u);  // tag = this launch's barrier number
            }
            __syncthreads();
        }
    }
    // logits are out: build the activation operand while the other CTAs catch up
    __syncthreads();
    // activation operand of every token, private to this CTA
    // int8 form: per token [2 terms][nblk_pad * 8 + 8 words] then [nblk_pad] {sx, 8 * sx * sum}; inside a block
    // the word pair of lane quad t is adjacent: {inputs 4t..4t+3, inputs 16+4t..16+4t+3}
    const int xq_term = xq_term_words(nblk_pad), xq_tok = xq_tok_words(nblk_pad);  // in 32-bit words
    unsigned* xq = reinterpret_cast<unsigned*>(xs);
    if (Q == Q4_0 && kInt8GateUp) {
        const int sub = tid & 7;
#pragma unroll 1
        for (int item = tid >> 3; item < T * nblk; item += FT / 8) {
            const int t = item / nblk, b = item - t * nblk;
            build_xq_block(xn4[t * H4 + b * 8 + sub], sub, lane, xq + (size_t)t * xq_tok, nblk_pad, b);
        }
        // padding blocks (kg_h * 4 > H / 32) must read as zero
        const int padw = (nblk_pad - nblk) * 8;
#pragma unroll 1
        for (int i = tid; i < T * 2 * padw; i += FT) {
            const int tt = i / padw, r = i - tt * padw;
            xq[(size_t)(tt >> 1) * xq_tok + (tt & 1) * xq_term + nblk * 8 + r] = 0u;
        }
#pragma unroll 1
        for (int i = tid; i < T * (nblk_pad - nblk); i += FT) {
            const int t = i / (nblk_pad - nblk), b = nblk + i - t * (nblk_pad - nblk);
            reinterpret_cast<float2*>(xq + (size_t)t * xq_tok + 2 * xq_term)[b] = make_float2(0.0f, 0.0f);
        }
    } else {
        const bool bf16_mode = (Q == BF16);
        const int sub = tid & 7, hl = sub >> 2, s4 = sub & 3;
#pragma unroll 1
        for (int item = tid >> 3; item < T * nblk; item += FT / 8) {
            const int t = item / nblk, b = item - t * nblk;
            const float4 lo4 = xn4[t * H4 + b * 8 + s4];
            const float4 hi4 = xn4[t * H4 + b * 8 + 4 + s4];
            xs[(size_t)t * per_col + ((size_t)hl * nblk_pad + b) * 4 + s4] = make_act_frag(lo4, hi4, hl, bf16_mode);
        }
        // padding blocks (kg_h * 4 > H / 32) must read as zero
        const int per = (nblk_pad - nblk) * 4;
#pragma unroll 1
        for (int i = tid; i < T * 2 * per; i += FT) {
            const int th = i / per, r = i - th * per;
            xs[(size_t)(th >> 1) * per_col + ((size_t)(th & 1) * nblk_pad + nblk) * 4 + r] = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    stamp(2);
    // barrier 1: wait for (and fetch) every logit of this launch
    {
        const float* lg = a.logits_override;
        bool ok = true;
#pragma unroll 1
        for (int i = tid; i < T * E; i += FT) {
            const int t = i / E, e = i - t * E;
            float v;
            if (want_logits) {
                const float* slot = a.R.logits + 2 * (size_t)i;
                uint2 r = ld_tagged(slot);
                unsigned long long t0 = 0;
                unsigned spins = 0;
                while (r.y != epoch + 1u) {
                    if ((++spins & 63u) == 0) {
                        if (t0 == 0) t0 = global_ns();
                        if (global_ns() - t0 > wc.limit_ns || *reinterpret_cast<volatile int*>(a.status) != 0) {
                            ok = false;
                            break;
                        }
                    }
                    r = ld_tagged(slot);
                }
                v = __uint_as_float(r.x);
            } else {
                v = __ldcg(lg + i);
            }
            ts.lg[t][e] = v;
        }
        if (!ok) {
            raise_status(a.status, a.status_host, 4);  // LUMEN_MOE_TIMEOUT
            fail_s = 1;
        }
        __syncthreads();
        if (fail_s) return;
    }
    stamp(3);

    // ---------------- phase B: routing (redundantly per CTA) ----------------
    // The exact gating below takes a few microseconds in which HBM would sit idle. The SET
    // of selected experts almost always equals the top-K by raw logit (the exp and the
    // division are monotonic; only probabilities that round to the same value with the
    // higher logit at the higher index can differ), and the set is all the weight staging
    // needs. So: rank the raw logits, request every tile for the predicted set, run the
    // exact gating while the tiles stream, then check the prediction and, if it was wrong,
    // drain and request again.
    const int rt_i = a.L.rt_i;
    const int it0 = G - 1 - cta;  // work items of this CTA: G-1-cta, then every G-th (CTAs without down rows first)
    const bool has_down = cta < a.L.rt_h;
    // Requests every byte this CTA needs for the experts ue[0..nu), called by ONE warp: the
    // tiles of its first gs_slots gate/up items (all input groups of a matrix are contiguous:
    // one bulk copy for the quants, one for the scales; barrier j counts item j's bytes), then
    // the down tiles of its 16 output rows for the first pf_experts experts (barrier 7).
    // copy r of work item j (its j-th for this CTA) into ring slot sl: r = matrix * PER + {quants, scales}
    auto copy_gu = [&](int j, int sl, int r, const int* ue) {
        constexpr int PER_ = (Q != BF16) ? 2 : 1;
        const int mat = r / PER_, is_s = r - mat * PER_;
        const int it = it0 + j * G;
        const int u = div_rti.div(it), rt = it - u * rt_i;
        const int e = ue[u];
        uint4* dst = gs_slot(sl) + (size_t)mat * kg_h * TU4 + (is_s ? kg_h * NQ32 : 0);
        const uint4* src = is_s ? (mat ? a.L.up_s(e) : a.L.gate_s(e)) + (size_t)rt * kg_h * 8
                                : (mat ? a.L.up_q(e) : a.L.gate_q(e)) + (size_t)rt * kg_h * NQ32;
        bulk_copy(dst, src, is_s ? (unsigned)kg_h * 128 : (unsigned)kg_h * NQ32 * 16, &mbar[sl]);
    };
    auto stage_all = [&](const int* ue, int nu) {
        const int n_items_ = nu * rt_i;
        const int n_my_ = (it0 < n_items_) ? div_g.div(n_items_ - it0 + G - 1) : 0;
        const int n_st_ = min(n_my_, gs_slots);
        const int n_pf_ = has_down ? min(nu, pf_experts) : 0;
        const unsigned q_gu = (unsigned)kg_h * NQ32 * 16, s_gu = (Q != BF16) ? (unsigned)kg_h * 128 : 0u;
        const unsigned q_dn = (unsigned)kg_i * NQ32 * 16, s_dn = (Q != BF16) ? (unsigned)kg_i * 128 : 0u;
        if (lane < n_st_) mbar_expect_tx(&mbar[lane], 2u * (q_gu + s_gu));
        if (lane == 7) mbar_expect_tx(&mbar[7], (unsigned)n_pf_ * (q_dn + s_dn));
        __syncwarp();
        constexpr int PER = (Q != BF16) ? 2 : 1;  // copies per matrix: quants, scales
#pragma unroll 1
        for (int c = lane; c < n_st_ * 2 * PER; c += 32) copy_gu(c / (2 * PER), c / (2 * PER), c % (2 * PER), ue);
#pragma unroll 1
        for (int c = lane; c < n_pf_ * PER; c += 32) {
            const int uu = c / PER, is_s = c - uu * PER;
            const int ee = ue[uu];
            uint4* dst = pf + ((size_t)uu * kg_i) * TU4 + (is_s ? kg_i * NQ32 : 0);
            const uint4* src = is_s ? a.L.down_s(ee) + (size_t)cta * kg_i * 8 : a.L.down_q(ee) + (size_t)cta * kg_i * NQ32;
            bulk_copy(dst, src, is_s ? s_dn : q_dn, &mbar[7]);
        }
    };
    {
        // Four warps per token share the exps; then warp 0 of the four finishes the token
        // exactly while another warp ranks the raw logits and requests the tiles.
        const int tok = warp >> 2, sub = warp & 3;
        const bool selects = (tok < T) && (sub == 0);
        // predictor of token t: an idle warp when there is one (T <= 3; it does not wait for
        // the exps), else warp 1 of the token's four
        const bool idle_pred = (T < FMAX_T);
        const bool predicts = idle_pred ? (warp >= 4 * T && warp < 5 * T) : (sub == 1);
        const int pred_tok = idle_pred ? warp - 4 * T : tok;
        if (tid < MAX_EXPERTS / 32) rs.pr_mask[tid] = 0u;
        __syncthreads();
        if (tok < T) {
            warp_gate_probs(ts.lg[tok], E, a.gating, ts.p[tok], ts.tab, sub, 4);
            asm volatile("bar.sync %0, 128;" ::"r"(1 + tok) : "memory");
        }
        if (predicts) {
            // rank the raw logits, merge the tokens' masks, and let the first predictor turn the
            // mask into the ascending expert list and request the tiles: no other warp is involved
            warp_predict_mask(ts.lg[pred_tok], E, K, rs.pr_mask);
            if (T > 1) asm volatile("bar.sync 6, %0;" ::"r"(T * 32) : "memory");
            else __syncwarp();
            if (pred_tok == 0) {
                int below = 0;  // set bits in lower words
#pragma unroll
                for (int wi = 0; wi < MAX_EXPERTS / 32; ++wi) {
                    const unsigned word = rs.pr_mask[wi];
                    if ((word >> lane) & 1u) rs.pr_ue[below + __popc(word & ((1u << lane) - 1u))] = wi * 32 + lane;
                    below += __popc(word);
                }
                if (lane == 0) rs.pr_U = below;
                __syncwarp();
                stage_all(rs.pr_ue, below);
                if (a.trace != nullptr && lane == 0) a.trace[(size_t)blockIdx.x * 12 + 10] = global_ns();
            }
        }
        if (selects) {
            warp_select(ts.p[tok], E, K, a.gating, reinterpret_cast<uint32_t*>(rs.ids) + tok * K, rs.w + tok * K);
            // the sort only needs the finishing warps: it does not wait for the warps that request tiles
            if (T > 1) asm volatile("bar.sync 11, %0;" ::"r"(T * 32) : "memory");
            if (warp == 0) {
                // stable counting sort of the C <= 32 pairs by expert, one pair per lane
                const int my = (lane < C) ? rs.ids[lane] : 0x7fffffff;
                unsigned lt = 0u;  // pairs with a smaller expert
#pragma unroll 4
                for (int q = 0; q < C; ++q) lt |= (__shfl_sync(0xffffffffu, my, q) < my ? 1u : 0u) << q;
                const unsigned same = __match_any_sync(0xffffffffu, my);
                const int less = __popc(lt), cnt = __popc(same), eqb = __popc(same & ((1u << lane) - 1u));
                const bool first = (lane < C) && (eqb == 0);
                const unsigned fmask = __ballot_sync(0xffffffffu, first);
                const int u = __popc(lt & fmask);  // distinct smaller experts
                if (lane < C) {
                    const int col = less + eqb;
                    rs.d2c[lane] = col;
                    rs.col_u[col] = u;
                    rs.col_tok[col] = lane / K;
                    if (first) {
                        rs.ue[u] = my;
                        rs.uc0[u] = col;
                        rs.uncol[u] = cnt;
                    }
                    if (cta == 0) {
                        a.R.ids[lane] = (uint32_t)my;
                        a.R.weights[lane] = rs.w[lane];
                        a.R.dst_to_col[lane] = col;
                        a.R.col_expert[col] = my;
                        a.R.col_src_tok[col] = lane / K;
                        if (first) a.R.uexp[u] = my;
                    }
                }
                if (lane == 0) {
                    rs.U = __popc(fmask);
                    if (cta == 0) *a.R.n_uexp = __popc(fmask);
                }
                if (cta == 0) {
                    for (int e = lane; e <= E; e += 32) {
                        int below = 0;
                        for (int q = 0; q < C; ++q) below += (rs.ids[q] < e);
                        a.R.expert_bounds[e] = below;
                    }
                }
            }
        }
        __syncthreads();
    }
    stamp(4);
    const int U = rs.U;
    const int n_items = U * rt_i;
    const int n_down = U * kg_i;
    {
        bool same = (U == rs.pr_U);
        if (same && tid < U) same = (rs.ue[tid] == rs.pr_ue[tid]);
        if (__syncthreads_or(same ? 0 : 1)) {
            // wrong prediction: let its copies land (they target the same slots), start the
            // barriers afresh and request the right tiles
            const int n_items_p = rs.pr_U * rt_i;
            const int n_my_p = (it0 < n_items_p) ? div_g.div(n_items_p - it0 + G - 1) : 0;
            bool ok = true;
            for (int j = 0; j < min(n_my_p, gs_slots) && ok; ++j) ok = mbar_wait(&mbar[j], 0, wc);
            ok = ok && mbar_wait(&mbar[7], 0, wc);
            if (__syncthreads_or(ok ? 0 : 1)) return;
            if (tid == 0) {
                for (int i = 0; i < 8; ++i) {
                    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_addr(&mbar[i])) : "memory");
                    mbar_init(&mbar[i], 1);
                }
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            }
            __syncthreads();
            if (warp == 0) stage_all(rs.ue, U);
        }
    }
    auto load_gu = [&](int it, WTile<Q>& g, WTile<Q>& up) {
        const int u = div_rti.div(it), rt = it - u * rt_i;
        const int e = rs.ue[u];
        if (warp < kg_h) {
            load_wtile<Q>(g, a.L.gate_q(e), a.L.gate_s(e), rt * kg_h + warp, lane);
            load_wtile<Q>(up, a.L.up_q(e), a.L.up_s(e), rt * kg_h + warp, lane);
        }
    };
    const int n_my = (it0 < n_items) ? div_g.div(n_items - it0 + G - 1) : 0;
    WTile<Q> wg0, wu0, wg1, wu1;
    if (gs_slots == 0 && n_my > 0) load_gu(it0, wg1, wu1);  // no ring: tiles go through registers, one item ahead

    // gate/up + SwiGLU
    auto compute_gu = [&](int it, const WTile<Q>& g, const WTile<Q>& up) {
        const int u = div_rti.div(it), rt = it - u * rt_i;
        const int c0 = rs.uc0[u];
        const int ncol = min(4, rs.uncol[u]);
        const int jcol = gq >> 1;
        const bool bvalid = jcol < ncol;
        const int tok = bvalid ? rs.col_tok[c0 + jcol] : 0;
        float acc_g[4] = {0.f, 0.f, 0.f, 0.f}, acc_u[4] = {0.f, 0.f, 0.f, 0.f};
        if (Q == Q4_0 && kInt8GateUp) {
            // acc[0] / acc[2]: rows gq / gq + 8 of the lane's token column t4 (acc[1], acc[3] stay zero)
            if (warp < kg_h) {
                const unsigned* bq = xq + (size_t)tok * xq_tok + (gq & 1) * xq_term + (warp * 4) * 8 + t4 * 2;
                const int tok_d = (t4 < ncol) ? rs.col_tok[c0 + t4] : 0;
                const float2* sc = reinterpret_cast<const float2*>(xq + (size_t)tok_d * xq_tok + 2 * xq_term) + warp * 4;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    uint2 bb = make_uint2(0u, 0u);
                    if (bvalid) bb = *reinterpret_cast<const uint2*>(bq + b * 8);
                    const uint4 qg = g.q[b >> 1], qu = up.q[b >> 1];
                    const unsigned g0 = (b & 1) ? qg.z : qg.x, g8 = (b & 1) ? qg.w : qg.y;
                    const unsigned u0 = (b & 1) ? qu.z : qu.x, u8 = (b & 1) ? qu.w : qu.y;
                    int cg[4] = {0, 0, 0, 0}, cu[4] = {0, 0, 0, 0};
                    mma_u8s8(cg, g0 & 0x0F0F0F0Fu, g8 & 0x0F0F0F0Fu, (g0 >> 4) & 0x0F0F0F0Fu, (g8 >> 4) & 0x0F0F0F0Fu,
                             bb.x, bb.y);
                    mma_u8s8(cu, u0 & 0x0F0F0F0Fu, u8 & 0x0F0F0F0Fu, (u0 >> 4) & 0x0F0F0F0Fu, (u8 >> 4) & 0x0F0F0F0Fu,
                             bb.x, bb.y);
                    const float2 sxo = sc[b];  // {sx, 8 * sx * sum(q)}
                    const float2 sg = block_scales<Q>(g, b), su = block_scales<Q>(up, b);
                    const float k1 = 1.0f / 254.0f;
                    acc_g[0] = fmaf(sg.x, fmaf(sxo.x, fmaf((float)cg[1], k1, (float)cg[0]), -sxo.y), acc_g[0]);
                    acc_g[2] = fmaf(sg.y, fmaf(sxo.x, fmaf((float)cg[3], k1, (float)cg[2]), -sxo.y), acc_g[2]);
                    acc_u[0] = fmaf(su.x, fmaf(sxo.x, fmaf((float)cu[1], k1, (float)cu[0]), -sxo.y), acc_u[0]);
                    acc_u[2] = fmaf(su.y, fmaf(sxo.x, fmaf((float)cu[3], k1, (float)cu[2]), -sxo.y), acc_u[2]);
                }
            }
        } else if (warp < kg_h) {
            const uint4* bp = xs + (size_t)tok * per_col + ((size_t)(gq & 1) * nblk_pad) * 4 + t4 + (size_t)warp * 16;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                block_mma_smem<Q>(g, b, bp, bvalid, acc_g);
                block_mma_smem<Q>(up, b, bp, bvalid, acc_u);
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
                float gate = 0.0f, upv = 0.0f;
#pragma unroll
                for (int w = 0; w < FW; ++w) {
                    gate += red[w][row][tokc][0];
                    upv += red[w][row][tokc][1];
                }
                const float sv = (gate / (1.0f + expf(-gate))) * upv;
                const int col = c0 + tokc;
                const int irow = rt * 16 + row;
                if (a.s_f32 != nullptr) a.s_f32[(size_t)col * I + irow] = sv;
                store_swiglu_frag<Q>(a.sf, col, irow, nblk_i_pad, sv);
            }
        }
        __syncthreads();
    };
    int sl = 0;          // ring slot of item j: j % gs_slots
    unsigned ring_ph = 0;  // parity of (j / gs_slots): how often the slot has been filled
#pragma unroll 1
    for (int j = 0; j < n_my; ++j) {
        if (gs_slots > 0) {
            if (!mbar_wait(&mbar[sl], ring_ph, wc)) return;  // all threads give up together
            if (a.trace != nullptr && tid == 0 && j == n_my - 1) a.trace[(size_t)blockIdx.x * 12 + 11] = global_ns();
            if (warp < kg_h) {
                const uint4* gq_ = gs_slot(sl);
                const uint4* uq_ = gq_ + (size_t)kg_h * TU4;
                read_staged<Q>(wg0, gq_ + warp * NQ32, gq_ + kg_h * NQ32 + warp * 8, lane);
                read_staged<Q>(wu0, uq_ + warp * NQ32, uq_ + kg_h * NQ32 + warp * 8, lane);
            }
        } else {
            wg0 = wg1;
            wu0 = wu1;
            if (j + 1 < n_my) load_gu(it0 + (j + 1) * G, wg1, wu1);
        }
        compute_gu(it0 + j * G, wg0, wu0);
        // every warp has its tiles of slot j % gs_slots in registers (compute_gu ends on CTA barriers):
        // refill the slot with the item gs_slots further on
        if (gs_slots > 0 && tid == 0 && j + gs_slots < n_my) {
            constexpr int PER_ = (Q != BF16) ? 2 : 1;
            mbar_expect_tx(&mbar[sl], 2u * ((unsigned)kg_h * NQ32 * 16 + ((Q != BF16) ? (unsigned)kg_h * 128 : 0u)));
            for (int r = 0; r < 2 * PER_; ++r) copy_gu(j + gs_slots, sl, r, rs.ue);
        }
        if (++sl == gs_slots) {
            sl = 0;
            ring_ph ^= 1u;
        }
    }
    // residual of this CTA's output rows, requested before the barrier
    float resid = 0.0f;
    if (has_down && tid < 16 * T) resid = a.residual[(size_t)(tid >> 4) * H + cta * 16 + (tid & 15)];
    stamp(5);
    __syncthreads();
    grid_arrive(a.bar);
    if (!grid_wait(a.bar, wc, G, ++epoch, a.debug_extra_arrivals, &fail_s)) {
        mbar_wait(&mbar[7], 0, wc);  // bounded: do not leave with the down copies in flight
        return;
    }
    if (tid == 0) a.bar[1 + cta] = epoch;
    stamp(6);

    // ---------------- phase C: down + combine ----------------
    if (!has_down) return;  // (no down tiles were requested for this CTA)
    for (int i = tid; i < C * per_col_i; i += FT) cp_async16(&ss[i], a.sf + i);
    cp_async_wait_all();
    if (!mbar_wait(&mbar[7], 0, wc)) return;
    __syncthreads();
    stamp(7);
    {
        // DG tiles of a warp are worked on together: their dependent chains (shared load ->
        // unpack -> two MMAs -> scale) overlap instead of running one after the other
        constexpr int DG = (Q == Q4_0) ? 3 : (Q == Q8_0) ? 2 : 1;
        const int rt = cta;
#pragma unroll 1
        for (int i0 = 0; warp + FW * i0 < n_down; i0 += DG) {
            WTile<Q> w[DG];
            int nn[DG];
#pragma unroll
            for (int j = 0; j < DG; ++j) {
                const int i = i0 + j;
                nn[j] = min(warp + FW * i, n_down - 1);
                const int uu = div_kgi.div(nn[j]), kg = nn[j] - uu * kg_i;
                if (uu < pf_experts) {
                    const uint4* base = pf + ((size_t)uu * kg_i) * TU4;
                    read_staged<Q>(w[j], base + kg * NQ32, base + kg_i * NQ32 + kg * 8, lane);
                } else {
                    const int ee = rs.ue[uu];
                    load_wtile<Q>(w[j], a.L.down_q(ee), a.L.down_s(ee), rt * kg_i + kg, lane);
                }
            }
#pragma unroll
            for (int j = 0; j < DG; ++j) {
                const int uu = div_kgi.div(nn[j]), kg = nn[j] - uu * kg_i;
                const int c0 = rs.uc0[uu];
                const int ncol = min(4, rs.uncol[uu]);
                const int jcol = gq >> 1;
                const bool bvalid = jcol < ncol;
                const uint4* bp = ss + ((size_t)((c0 + (bvalid ? jcol : 0)) * 2 + (gq & 1)) * nblk_i_pad) * 4 + t4 +
                                  (size_t)kg * 16;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int b = 0; b < 4; ++b) block_mma_smem<Q>(w[j], b, bp, bvalid, acc);
                if (warp + FW * (i0 + j) < n_down) {
                    float* pp = part + (size_t)nn[j] * 64 + t4 * 16;
                    pp[gq] = acc[0] + acc[1];
                    pp[gq + 8] = acc[2] + acc[3];
                }
            }
        }
        __syncthreads();
        stamp(8);
        // weighted expert outputs of every (token, slot) pair, one (pair, row) per thread ...
#pragma unroll 1
        for (int idx = tid; idx < C * 16; idx += FT) {
            const int pair = idx >> 4, row = idx & 15;
            const int col = rs.d2c[pair];
            const int uu = rs.col_u[col];
            const int j = min(col - rs.uc0[uu], 3);
            const float* pp = part + (size_t)uu * kg_i * 64 + j * 16 + row;
            float d = 0.0f;
#pragma unroll 2
            for (int kg = 0; kg < kg_i; ++kg) d += pp[kg * 64];
            wd[idx] = __fmul_rn(rs.w[pair], d);
        }
        __syncthreads();
        // ... then the sum in slot order on top of the residual (cuda/shaders/moe_accum.cu:22-46)
        if (tid < 16 * T) {
            const int row = tid & 15, t = tid >> 4;
            float accv = resid;
#pragma unroll 1
            for (int slot = 0; slot < K; ++slot) accv = __fadd_rn(accv, wd[(t * K + slot) * 16 + row]);
            a.out[(size_t)t * H + rt * 16 + row] = accv;
        }
    }
    stamp(9);
}

// Shared memory the fused kernel needs besides its static arrays; pf_experts = experts whose
// down tiles are staged, gs_slots = staged gate/up work items.
// gs_slots counts only the ring slots with storage of their own (see fused_mid_bytes).
static size_t fused_mid_bytes(const DecodeArgs& a) {
    const size_t C = (size_t)a.T * a.K;
    const size_t mid = C * 2 * a.L.kg_i * 16 * 16 + C * a.L.kg_i * 256 + C * 64;
    const size_t xn = (size_t)a.T * a.L.H * 4;
    return mid > xn ? mid : xn;
}
static size_t fused_smem_bytes(const DecodeArgs& a, int tile_u4, int pf_experts, int gs_slots = 0) {
    return (size_t)a.T * 2 * a.L.kg_h * 16 * 16 + fused_mid_bytes(a) +
           (size_t)pf_experts * a.L.kg_i * tile_u4 * 16 + (size_t)gs_slots * 2 * a.L.kg_h * tile_u4 * 16;
}

static int tile_u4_of(int quant) {
    return quant == Q4_0 ? TileU4<Q4_0>::value : quant == Q8_0 ? TileU4<Q8_0>::value : TileU4<BF16>::value;
}

struct FusedDeviceInfo {
    int sms = 0;
    int smem_optin = 0;
};

static const FusedDeviceInfo& fused_device_info(int device) {
    static FusedDeviceInfo info[64];
    FusedDeviceInfo& d = info[device & 63];
    if (d.sms == 0) {
        int sms = 0, smem = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
        d.smem_optin = smem;
        d.sms = sms;
    }
    return d;
}

// Shape limits of the fused kernel: one 128-input group per warp, one pair per lane in
// the sort, one CTA per 16 output rows, and the shared-memory budget.
bool decode_fused_applicable(const DecodeArgs& a) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return false;
    if (a.bar == nullptr || a.status == nullptr) return false;
    if (a.T < 1 || a.T > FMAX_T || a.T * a.K > FMAX_C) return false;
    if (a.L.kg_h > FW || a.L.H > FT * 4) return false;
    const FusedDeviceInfo& d = fused_device_info(device);
    if (d.sms <= 0 || d.sms > 1023 || a.L.rt_h > d.sms) return false;
    const size_t static_smem = 20 * 1024;
    return fused_smem_bytes(a, tile_u4_of(a.L.quant), 0) + static_smem <= (size_t)d.smem_optin;
}

template <int Q>
static cudaError_t launch_fused_t(const DecodeArgs& a, int device, cudaStream_t st) {
    const FusedDeviceInfo& d = fused_device_info(device);
    const size_t static_smem = 20 * 1024;
    const int C = a.T * a.K;
    // shared memory goes to the gate/up items of a CTA first (they are needed first), then to the down tiles
    const int nu_max = C < a.L.E ? C : a.L.E;
    // ring of gate/up work items: as many as a CTA can have, at most 3 (three items in flight cover the
    // HBM latency); slots that fit over the phase C region cost nothing, the others get storage of their own
    int ring = (nu_max * a.L.rt_i + d.sms - 1) / d.sms;
    if (ring > 3) ring = 3;
    const size_t item_bytes = (size_t)2 * a.L.kg_h * TileU4<Q>::value * 16;
    int alias = (int)(fused_mid_bytes(a) / item_bytes);
    if (alias > ring) alias = ring;
    while (ring > alias && fused_smem_bytes(a, TileU4<Q>::value, 0, ring - alias) + static_smem > (size_t)d.smem_optin) --ring;
    const int gs = ring - alias;  // slots with storage of their own
    int pf = nu_max;  // experts whose down tiles are staged
    while (pf > 0 && fused_smem_bytes(a, TileU4<Q>::value, pf, gs) + static_smem > (size_t)d.smem_optin) --pf;
    const size_t smem = fused_smem_bytes(a, TileU4<Q>::value, pf, gs);
    static size_t attr_smem[64] = {};
    if (smem > attr_smem[device & 63]) {
        cudaError_t e = cudaFuncSetAttribute(decode_fused_kernel<Q>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
        attr_smem[device & 63] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(d.sms);
    cfg.blockDim = dim3(FT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    // All CTAs must be resident at once (grid barriers): a cooperative launch makes the
    // driver check that; the programmatic attribute lets the prologue overlap the
    // previous kernel's tail.
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    count_launch();
    return cudaLaunchKernelEx(&cfg, decode_fused_kernel<Q>, a, pf, ring, alias);
}

cudaError_t launch_decode_fused(const DecodeArgs& a, cudaStream_t st) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    switch (a.L.quant) {
        case Q4_0: return launch_fused_t<Q4_0>(a, device, st);
        case Q8_0: return launch_fused_t<Q8_0>(a, device, st);
        default: return launch_fused_t<BF16>(a, device, st);
    }
}

}  // namespace lumen
