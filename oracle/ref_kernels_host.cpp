// Host build of the reference project's own scalar MoE kernels, used as a second
// oracle next to the restatement in lumen_moe_oracle.cpp.
//
// TEST INFRASTRUCTURE ONLY. The kernel sources are NOT copied: they are included
// from where they lie in the reference tree (-I<reference>/crates/lumen-runtime/
// src/cuda/shaders, see oracle/Makefile) and compiled by g++ with the handful of
// CUDA keywords they use defined away. These kernels are "one thread per output
// row" (cuda/shaders/moe_expert.cu:62-136, moe_expert_q4_0.cu:58-151,
// moe_accum.cu:22-81), so running them on the host is a loop over
// (blockIdx.x, threadIdx.x). Their only inline PTX is "cvt.f32.f16", replaced
// here by an exact software conversion.
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>

struct RefDim3 {
    unsigned int x, y, z;
};
static thread_local RefDim3 blockIdx, threadIdx;

static inline float ref_f16_to_f32(unsigned short h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31;
    const uint32_t exp = (h >> 10) & 0x1F, frac = h & 0x3FF;
    uint32_t out;
    if (exp == 0) {
        if (frac == 0) {
            out = sign;
        } else {
            int e = -1;
            uint32_t f = frac;
            do {
                ++e;
                f <<= 1;
            } while ((f & 0x400) == 0);
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((f & 0x3FF) << 13);
        }
    } else if (exp == 31) {
        out = sign | 0x7F800000u | (frac << 13);
    } else {
        out = sign | ((exp - 15 + 127) << 23) | (frac << 13);
    }
    float v;
    std::memcpy(&v, &out, 4);
    return v;
}

#define __global__
#define __device__
#define __forceinline__ inline
#define __restrict__
// the two helpers that use inline PTX name their operands `result` and `bits`
#define asm(...) (result = ref_f16_to_f32(bits))

#include "moe_expert.cu"
#include "moe_expert_q4_0.cu"
#include "moe_accum.cu"

#undef asm

#define REF_API extern "C" __attribute__((visibility("default")))

template <typename F>
static void run_grid(unsigned rows, unsigned block, F&& body) {
    const unsigned nblocks = (rows + block - 1) / block;
    for (unsigned b = 0; b < nblocks; ++b)
        for (unsigned t = 0; t < block; ++t) {
            blockIdx = {b, 0, 0};
            threadIdx = {t, 0, 0};
            body();
        }
}

// quant: 0 = Q8_0, 1 = Q4_0
REF_API void ref_gate_up_swiglu(const float* normed_x, const unsigned char* layer_buf, unsigned long long gate_off,
                                unsigned long long up_off, float* swiglu_out, unsigned hidden_dim, unsigned inter_dim,
                                int quant) {
    if (quant == 0)
        run_grid(inter_dim, 128, [&] {
            moe_expert_gate_up_swiglu_q8_0(normed_x, layer_buf, gate_off, up_off, swiglu_out, hidden_dim, inter_dim);
        });
    else
        run_grid(inter_dim, 128, [&] {
            moe_expert_gate_up_swiglu_q4_0(normed_x, layer_buf, gate_off, up_off, swiglu_out, hidden_dim, inter_dim);
        });
}

REF_API void ref_down(const float* swiglu_in, const unsigned char* layer_buf, unsigned long long down_off,
                      float* expert_out, unsigned hidden_dim, unsigned inter_dim, int quant) {
    if (quant == 0)
        run_grid(hidden_dim, 128,
                 [&] { moe_expert_down_q8_0(swiglu_in, layer_buf, down_off, expert_out, hidden_dim, inter_dim); });
    else
        run_grid(hidden_dim, 128,
                 [&] { moe_expert_down_q4_0(swiglu_in, layer_buf, down_off, expert_out, hidden_dim, inter_dim); });
}

REF_API void ref_accum_option_a(float* x, const float* residual, const float* expert_outputs,
                                const float* expert_weights, unsigned hidden_dim, unsigned top_k) {
    run_grid(hidden_dim, 128,
             [&] { moe_expert_accum_option_a(x, residual, expert_outputs, expert_weights, hidden_dim, top_k); });
}
