// Gating + top-k + renormalisation for one token by one warp.
//
// Follows cpu_router_softmax phases 2-3 (crates/lumen-runtime/src/cuda/moe.rs:6464-6504)
// operation for operation where the result depends on it:
//   maxv  = fold(max)                         (exact in any order)
//   p[e]  = exp(logit[e] - maxv)              (libm-identical exp, exact_expf.h)
//   sum   = p[0] + p[1] + ...                 (sequential f32, e ascending)
//   p[e] /= sum                               (IEEE division)
//   K rounds of argmax with strict '>' (the lowest index wins a tie), the winner
//          masked: done here as two warp reductions per round (largest value, then the
//          lowest index holding it: the tie-break of cuda/shaders/topk_moe_fused.cu:251)
//   renorm = sel[0] + sel[1] + ...            (sequential f32, k ascending)
//   w[k]  = sel[k] / renorm  if renorm > 0
// SIGMOID_RENORM (cuda/shaders/topk_moe_fused.cu:118-129) replaces the first four
// lines by p[e] = 1 / (1 + exp(-logit[e])). Gating 2 is the same without the last two
// lines (the shared expert's gate, cuda/shaders/moe_shared_accum.cu:1-12), gating 3
// sets w[k] = 1.
// Logits are assumed finite (NaN logits give in-range but unspecified ids).
#pragma once
#include "moe_internal.cuh"
#include "exact_expf.h"

namespace lumen {

// smem_p: E floats (E <= 256), 16-byte aligned, private to the calling warp. `tab` is
// a copy of the 32-entry exp table in shared memory, or null for the library's own
// copy (lanes index the table divergently, which a generic load handles better than
// the constant cache). out_ids / out_w may point to global or shared memory.
//
// The chain of dependent operations is what costs here, so: the sequential sum runs
// on every lane redundantly from shared memory, sixteen values per step with the next
// sixteen already loading; each selection round is two warp reductions (redux.sync):
// the largest key, then the lowest index holding it. Keys are the probability's bit
// pattern + 1 (probabilities are >= 0, so unsigned order is value order); 0 marks
// padding and already selected experts.
//
// Double-precision instructions issue slowly on this part, and the exp is the only
// place that needs them, so the exps of one token can be shared by `nsub` warps
// (warp_gate_probs with sub = 0..nsub-1, the caller synchronises them) before one
// warp finishes the token (warp_select). warp_topk is the one-warp form.

// One body for all call sites: the exp is ~60 double-precision instructions and the code of
// these routines runs once per launch, so its size is paid in instruction fetches.
static __device__ __noinline__ float expf_exact_call(float x, const uint64_t* tab) {
    return lumen_exact::expf_libm_tab(x, lumen_exact::Exp2TabPtr{tab});
}

// Unnormalised gate values into smem_p[e] for the experts of this warp's share:
// 32-expert group (e >> 5) belongs to sub-warp (e >> 5) % nsub. Softmax: exp(logit - max);
// sigmoid: the final 1 / (1 + exp(-logit)). `logits` may be shared or global memory.
__device__ __forceinline__ void warp_gate_probs(const float* __restrict__ logits, int E, int gating, float* smem_p,
                                                const unsigned long long* tab, int sub, int nsub) {
    const int lane = threadIdx.x & 31;
    const lumen_exact::Exp2TabPtr et{tab != nullptr ? reinterpret_cast<const uint64_t*>(tab)
                                                    : lumen_exact::exp2_tab_dev};
    float lg[8];  // expert e = lane + 32*i
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        lg[i] = (e < E) ? logits[e] : -INFINITY;
    }
    float m = 0.0f;
    if (gating == 0) {
        m = lg[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) m = fmaxf(m, lg[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        if (e < E && (i % nsub) == sub) {
            const float ex = expf_exact_call((gating == 0) ? lg[i] - m : -lg[i], et.p);
            smem_p[e] = (gating == 0) ? ex : __fdiv_rn(1.0f, __fadd_rn(1.0f, ex));
        }
    }
}

// Normalisation (softmax), K selection rounds and renormalised weights from the gate
// values in smem_p (all E of them visible to this warp).
template <int NS>  // NS * 32 >= E: slots (experts) per lane
__device__ __forceinline__ void warp_select_n(const float* smem_p, int E, int K, int gating, uint32_t* out_ids,
                                              float* out_w) {
    const int lane = threadIdx.x & 31;
    float pe[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) pe[i] = (lane + 32 * i < E) ? smem_p[lane + 32 * i] : 0.0f;
    if (gating == 0) {
        float sum = 0.0f;
        const int E16 = E & ~15;
        int e = 0;
        if (E16 > 0) {
            const float4* p4 = reinterpret_cast<const float4*>(smem_p);
            float4 c0 = p4[0], c1 = p4[1], c2 = p4[2], c3 = p4[3];
#pragma unroll 1
            for (; e < E16; e += 16) {
                float4 n0 = c0, n1 = c1, n2 = c2, n3 = c3;
                if (e + 16 < E16) {
                    const float4* q4 = p4 + ((e + 16) >> 2);
                    n0 = q4[0];
                    n1 = q4[1];
                    n2 = q4[2];
                    n3 = q4[3];
                }
                sum = __fadd_rn(sum, c0.x); sum = __fadd_rn(sum, c0.y); sum = __fadd_rn(sum, c0.z); sum = __fadd_rn(sum, c0.w);
                sum = __fadd_rn(sum, c1.x); sum = __fadd_rn(sum, c1.y); sum = __fadd_rn(sum, c1.z); sum = __fadd_rn(sum, c1.w);
                sum = __fadd_rn(sum, c2.x); sum = __fadd_rn(sum, c2.y); sum = __fadd_rn(sum, c2.z); sum = __fadd_rn(sum, c2.w);
                sum = __fadd_rn(sum, c3.x); sum = __fadd_rn(sum, c3.y); sum = __fadd_rn(sum, c3.z); sum = __fadd_rn(sum, c3.w);
                c0 = n0; c1 = n1; c2 = n2; c3 = n3;
            }
        }
#pragma unroll 1
        for (; e < E; ++e) sum = __fadd_rn(sum, smem_p[e]);
#pragma unroll
        for (int i = 0; i < NS; ++i)
            if (lane + 32 * i < E) pe[i] = __fdiv_rn(pe[i], sum);
    }
    unsigned key[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) key[i] = (lane + 32 * i < E) ? __float_as_uint(pe[i]) + 1u : 0u;
    float my_sel = 0.0f, renorm = 0.0f;
    int my_id = 0;
#pragma unroll 1
    for (int k = 0; k < K; ++k) {
        // own best: ascending scan with strict '>' keeps the lowest index among equals
        unsigned hk = key[0];
        int hi = 0;
#pragma unroll
        for (int i = 1; i < NS; ++i) {
            if (key[i] > hk) {
                hk = key[i];
                hi = i;
            }
        }
        const unsigned mk = __reduce_max_sync(0xffffffffu, hk);
        int win = __reduce_min_sync(0xffffffffu, (hk == mk) ? lane + 32 * hi : 0x7fffffff);
        float sel = __uint_as_float(mk - 1u);
        if (mk == 0u) {  // nothing left: the reference's fold starts at (index 0, -1.0)
            win = 0;
            sel = -1.0f;
        }
        renorm = __fadd_rn(renorm, sel);  // sel[0] + sel[1] + ... in order, on every lane
        if (lane == k) {
            my_sel = sel;
            my_id = win;
        }
#pragma unroll
        for (int i = 0; i < NS; ++i)
            if (lane + 32 * i == win) key[i] = 0u;
    }
    if (lane < K) {
        out_ids[lane] = (uint32_t)my_id;
        // gating 2: the sigmoid value itself (shared-expert gate); 3: unit weight
        out_w[lane] = (gating == 3) ? 1.0f
                      : (gating != 2 && renorm > 0.0f) ? __fdiv_rn(my_sel, renorm) : my_sel;
    }
    __syncwarp();
}

__device__ __forceinline__ void warp_select(const float* smem_p, int E, int K, int gating, uint32_t* out_ids,
                                            float* out_w) {
    if (E <= 128) warp_select_n<4>(smem_p, E, K, gating, out_ids, out_w);
    else warp_select_n<8>(smem_p, E, K, gating, out_ids, out_w);
}

// Sets, in mask (one bit per expert, shared memory, zeroed by the caller), the K experts
// with the largest raw logits, lowest index first among equals: a prediction of the
// selected SET that needs no exp (the gate functions are monotonic), used to start weight
// traffic early; the caller verifies it against warp_select's result.
template <int NS>  // NS * 32 >= E
__device__ __forceinline__ void warp_predict_mask_n(const float* logits, int E, int K, unsigned* mask) {
    const int lane = threadIdx.x & 31;
    unsigned key[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int e = lane + 32 * i;
        const unsigned b = (e < E) ? __float_as_uint(logits[e]) : 0u;
        // order-preserving map of finite floats to unsigned, shifted so that 0 stays free for "taken / padding"
        const unsigned k = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
        key[i] = (e < E) ? max(k, 1u) : 0u;
    }
    int my_win = -1;  // lane k keeps the k-th winner
#pragma unroll 1
    for (int k = 0; k < K; ++k) {
        unsigned hk = key[0];
        int hi = 0;
#pragma unroll
        for (int i = 1; i < NS; ++i) {
            if (key[i] > hk) {
                hk = key[i];
                hi = i;
            }
        }
        const unsigned mk = __reduce_max_sync(0xffffffffu, hk);
        const int win = __reduce_min_sync(0xffffffffu, (hk == mk) ? lane + 32 * hi : 0x7fffffff);
        if (mk == 0u) break;
        if (lane == k) my_win = win;
#pragma unroll
        for (int i = 0; i < NS; ++i)
            if (lane + 32 * i == win) key[i] = 0u;
    }
    if (my_win >= 0) atomicOr(&mask[my_win >> 5], 1u << (my_win & 31));
}

__device__ __forceinline__ void warp_predict_mask(const float* logits, int E, int K, unsigned* mask) {
    if (E <= 128) warp_predict_mask_n<4>(logits, E, K, mask);
    else warp_predict_mask_n<8>(logits, E, K, mask);
}

__device__ __forceinline__ void warp_topk(const float* __restrict__ logits, int E, int K, int gating,
                                          float* smem_p, const unsigned long long* tab, uint32_t* out_ids,
                                          float* out_w) {
    warp_gate_probs(logits, E, gating, smem_p, tab, 0, 1);
    __syncwarp();
    warp_select(smem_p, E, K, gating, out_ids, out_w);
}

}  // namespace lumen
