// Gating + top-k + renormalisation for one token by one warp, and the stable
// counting sort of (token, slot) pairs by expert for small batches.
//
// Follows cpu_router_softmax phases 2-3 (crates/lumen-runtime/src/cuda/moe.rs:6464-6504)
// operation for operation where the result depends on it:
//   maxv  = fold(max)                         (exact in any order)
//   p[e]  = exp(logit[e] - maxv)              (libm-identical exp, exact_expf.h)
//   sum   = p[0] + p[1] + ...                 (sequential f32, e ascending)
//   p[e] /= sum                               (IEEE division)
//   K rounds of argmax with strict '>' from (index 0, value -1), winner masked to -1
//          == rank of e under (p descending, index ascending); ranks < K are the ids
//   renorm = sel[0] + sel[1] + ...            (sequential f32, k ascending)
//   w[k]  = sel[k] / renorm  if renorm > 0
// SIGMOID_RENORM (cuda/shaders/topk_moe_fused.cu:118-129) replaces the first four
// lines by p[e] = 1 / (1 + exp(-logit[e])).
// Logits are assumed finite (NaN logits give in-range but unspecified ids).
#pragma once
#include "moe_internal.cuh"
#include "exact_expf.h"

namespace lumen {

// smem_p: E floats, smem_sel: K floats, private to the calling warp.
__device__ __forceinline__ void warp_topk(const float* __restrict__ logits, int E, int K, int gating,
                                          float* smem_p, float* smem_sel, uint32_t* out_ids,
                                          float* out_w) {
    const int lane = threadIdx.x & 31;
    if (gating == 0) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, logits[e]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        for (int e = lane; e < E; e += 32) smem_p[e] = lumen_exact::expf_libm(logits[e] - m);
        __syncwarp();
        float sum = 0.0f;
        if (lane == 0) {
            for (int e = 0; e < E; ++e) sum = __fadd_rn(sum, smem_p[e]);
        }
        sum = __shfl_sync(0xffffffffu, sum, 0);
        for (int e = lane; e < E; e += 32) smem_p[e] = __fdiv_rn(smem_p[e], sum);
    } else {
        for (int e = lane; e < E; e += 32)
            smem_p[e] = __fdiv_rn(1.0f, __fadd_rn(1.0f, lumen_exact::expf_libm(-logits[e])));
    }
    if (lane < K) {
        out_ids[lane] = 0u;
        smem_sel[lane] = -1.0f;
    }
    __syncwarp();
    {
        // rank of every expert under (p descending, index ascending); each lane
        // ranks up to 8 experts (E <= 256) in one pass over the probabilities
        float pe[8];
        int rank[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            pe[i] = (e < E) ? smem_p[e] : 0.0f;
            rank[i] = 0;
        }
        for (int j = 0; j < E; ++j) {
            const float pj = smem_p[j];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int e = lane + 32 * i;
                rank[i] += (pj > pe[i]) || (pj == pe[i] && j < e);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            if (e < E && rank[i] < K && pe[i] > -1.0f) {
                out_ids[rank[i]] = (uint32_t)e;
                smem_sel[rank[i]] = pe[i];
            }
        }
    }
    __syncwarp();
    if (lane == 0) {
        float renorm = 0.0f;
        for (int k = 0; k < K; ++k) renorm = __fadd_rn(renorm, smem_sel[k]);
        for (int k = 0; k < K; ++k)
            out_w[k] = (renorm > 0.0f) ? __fdiv_rn(smem_sel[k], renorm) : smem_sel[k];
    }
    __syncwarp();
}

}  // namespace lumen
