// Gating + top-k + renormalisation for one token by one warp.
//
// Follows cpu_router_softmax phases 2-3 (crates/lumen-runtime/src/cuda/moe.rs:6464-6504)
// operation for operation where the result depends on it:
//   maxv  = fold(max)                         (exact in any order)
//   p[e]  = exp(logit[e] - maxv)              (libm-identical exp, exact_expf.h)
//   sum   = p[0] + p[1] + ...                 (sequential f32, e ascending)
//   p[e] /= sum                               (IEEE division)
//   K rounds of argmax with strict '>' (the lowest index wins a tie), the winner
//          masked to -1: done here as a warp-shuffle argmax on (value, index) with
//          the explicit lower-index tie-break of cuda/shaders/topk_moe_fused.cu:251
//   renorm = sel[0] + sel[1] + ...            (sequential f32, k ascending)
//   w[k]  = sel[k] / renorm  if renorm > 0
// SIGMOID_RENORM (cuda/shaders/topk_moe_fused.cu:118-129) replaces the first four
// lines by p[e] = 1 / (1 + exp(-logit[e])).
// Logits are assumed finite (NaN logits give in-range but unspecified ids).
#pragma once
#include "moe_internal.cuh"
#include "exact_expf.h"

namespace lumen {

// smem_p: E floats (E <= 256), private to the calling warp. out_ids / out_w may
// point to global or shared memory; lane k (< K) also returns ids[k] in *my_id.
__device__ __forceinline__ void warp_topk(const float* __restrict__ logits, int E, int K, int gating,
                                          float* smem_p, float* /*unused*/, uint32_t* out_ids,
                                          float* out_w) {
    const int lane = threadIdx.x & 31;
    float pe[8];  // expert e = lane + 32*i
    if (gating == 0) {
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            pe[i] = (e < E) ? logits[e] : -INFINITY;
            m = fmaxf(m, pe[i]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            if (e < E) {
                pe[i] = lumen_exact::expf_libm(pe[i] - m);
                smem_p[e] = pe[i];
            }
        }
        __syncwarp();
        float sum = 0.0f;
        if (lane == 0) {
            int e = 0;
            for (; e + 4 <= E; e += 4) {
                const float4 v = *reinterpret_cast<const float4*>(smem_p + e);
                sum = __fadd_rn(sum, v.x);
                sum = __fadd_rn(sum, v.y);
                sum = __fadd_rn(sum, v.z);
                sum = __fadd_rn(sum, v.w);
            }
            for (; e < E; ++e) sum = __fadd_rn(sum, smem_p[e]);
        }
        sum = __shfl_sync(0xffffffffu, sum, 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) pe[i] = (lane + 32 * i < E) ? __fdiv_rn(pe[i], sum) : -2.0f;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            pe[i] = (e < E) ? __fdiv_rn(1.0f, __fadd_rn(1.0f, lumen_exact::expf_libm(-logits[e]))) : -2.0f;
        }
    }
    float my_sel = 0.0f;  // lane k keeps the k-th selected probability
    int my_id = 0;
    for (int k = 0; k < K; ++k) {
        // local best: strict '>' in ascending index order keeps the lowest index among equals
        float bv = -1.0f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (pe[i] > bv) {
                bv = pe[i];
                bi = lane + 32 * i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        if (bi == 0x7fffffff) bi = 0;  // nothing above -1: the reference's fold starts at (0, -1.0)
        if (lane == k) {
            my_sel = bv;
            my_id = bi;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (lane + 32 * i == bi) pe[i] = -1.0f;  // mask the winner
    }
    // renorm = sel[0] + sel[1] + ... in order, on lane 0
    float renorm = 0.0f;
    for (int k = 0; k < K; ++k) {
        const float s = __shfl_sync(0xffffffffu, my_sel, k);
        renorm = __fadd_rn(renorm, s);
    }
    if (lane < K) {
        out_ids[lane] = (uint32_t)my_id;
        out_w[lane] = (renorm > 0.0f) ? __fdiv_rn(my_sel, renorm) : my_sel;
    }
    __syncwarp();
}

}  // namespace lumen
