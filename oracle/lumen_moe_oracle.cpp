// CPU oracle for the MoE feed-forward path of lumen-runtime's CUDA backend.
//
// TEST INFRASTRUCTURE ONLY. This file restates, in plain scalar C++, the CPU
// reference arithmetic that the reference project itself uses to check its MoE
// kernels. It is the checker for the CUDA library and the timed "CPU baseline";
// nothing in the product path may call it. Every function cites the reference
// file:line it follows (paths relative to the reference project's root).
//
// Parity status: PINNED against the reference's own known-answer tests (router
// analytic / tie / epsilon KATs, counting-sort KAT, Q4_0 / Q8_0 block KATs,
// accumulate closed forms, LCG property sweeps) in tests/test_oracle_kat.py, and
// cross-checked against the reference's scalar expert kernels compiled for the
// host (oracle/_ref, see oracle/Makefile).
//
// Third-party arithmetic on the path: the reference's softmax and SwiGLU call
// Rust's f32::exp, which on x86_64-unknown-linux-gnu lowers to the platform
// libm's expf (glibc 2.39 in this image). The oracle calls the same libm expf.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>
#include <algorithm>
#include <atomic>
#include <functional>

#define ORC_API extern "C" __attribute__((visibility("default")))

enum { ORC_Q8_0 = 0, ORC_Q4_0 = 1, ORC_BF16 = 2 };

// ---------------------------------------------------------------------------
// Scalar formats
// ---------------------------------------------------------------------------

// f16 bits -> f32. crates/lumen-runtime/src/compute/cpu_naive.rs:177-208
// (subnormals decoded as frac/1024 * 2^-14; inf/nan preserved).
ORC_API float orc_f16_bits_to_f32(uint16_t bits) {
    const uint32_t sign = (bits >> 15) & 1u;
    const uint32_t exp = (bits >> 10) & 0x1fu;
    const uint32_t frac = bits & 0x3ffu;
    if (exp == 0) {
        if (frac == 0) return sign ? -0.0f : 0.0f;
        const float f = (float)frac / 1024.0f;
        const float v = f * 6.103515625e-05f;  // 2^-14
        return sign ? -v : v;
    }
    if (exp == 31) {
        if (frac == 0) return sign ? -INFINITY : INFINITY;
        return NAN;
    }
    const uint32_t out = ((exp - 15u + 127u) << 23) | (frac << 13);
    float v;
    std::memcpy(&v, &out, 4);
    return sign ? -v : v;
}

// f32 -> f16 bits by TRUNCATION of the significand (no rounding), subnormals
// kept. crates/lumen-convert/src/dequant.rs:741-785.
ORC_API uint16_t orc_f32_to_f16_bits(float val) {
    uint32_t bits;
    std::memcpy(&bits, &val, 4);
    const uint32_t sign = (bits >> 31) & 1u;
    const int32_t exp = (int32_t)((bits >> 23) & 0xFFu);
    const uint32_t frac = bits & 0x7FFFFFu;
    if (exp == 255) {
        const uint32_t f16_frac = frac != 0 ? 0x200u : 0u;
        return (uint16_t)((sign << 15) | (0x1Fu << 10) | f16_frac);
    }
    const int32_t new_exp = exp - 127 + 15;
    if (new_exp >= 31) return (uint16_t)((sign << 15) | (0x1Fu << 10));
    if (new_exp <= 0) {
        if (new_exp < -10) return (uint16_t)(sign << 15);
        const uint32_t mantissa = frac | 0x00800000u;
        const uint32_t shift = (uint32_t)(14 - new_exp);
        const uint32_t f16_frac = mantissa >> shift;
        return (uint16_t)((sign << 15) | (f16_frac & 0x3FFu));
    }
    return (uint16_t)((sign << 15) | ((uint32_t)new_exp << 10) | (frac >> 13));
}

// bf16 bits -> f32: bits << 16.
// crates/lumen-runtime/src/cuda/shaders/moe_batched_bf16.cu:31-34
static inline float bf16_bits_to_f32(uint16_t b) {
    const uint32_t x = ((uint32_t)b) << 16;
    float v;
    std::memcpy(&v, &x, 4);
    return v;
}

// f32 -> bf16 bits, round to nearest even. Used only to synthesise BF16 test
// weights (the benchmark configuration states "round-to-nearest-even of the
// f32 draws"); the reference path itself only ever reads bf16.
ORC_API uint16_t orc_f32_to_bf16_bits(float v) {
    uint32_t x;
    std::memcpy(&x, &v, 4);
    if ((x & 0x7F800000u) == 0x7F800000u && (x & 0x7FFFFFu)) return (uint16_t)((x >> 16) | 0x40u);
    const uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

// ---------------------------------------------------------------------------
// Quantisers / dequantisers (define "quantised to Q4_0 / Q8_0")
// ---------------------------------------------------------------------------

// crates/lumen-convert/src/dequant.rs:791-849. roundf == Rust f32::round (half
// away from zero). The block stores the f16-truncated scale; quantisation divides
// by the full-precision f32 scale.
ORC_API void orc_quantize_q4_0(const float* src, int64_t n_elements, uint8_t* dst) {
    const int64_t nb = n_elements / 32;
    for (int64_t b = 0; b < nb; ++b) {
        const float* v = src + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(v[i]));
        const float scale = (amax == 0.0f) ? 1.0f : std::fmin(amax / 7.0f, 65504.0f);
        const float inv = (scale == 0.0f) ? 0.0f : 1.0f / scale;
        const uint16_t s16 = orc_f32_to_f16_bits(scale);
        uint8_t* o = dst + b * 18;
        o[0] = (uint8_t)(s16 & 0xFF);
        o[1] = (uint8_t)(s16 >> 8);
        for (int i = 0; i < 16; ++i) {
            int lo = (int)std::roundf(v[i] * inv) + 8;
            int hi = (int)std::roundf(v[i + 16] * inv) + 8;
            lo = std::min(15, std::max(0, lo));
            hi = std::min(15, std::max(0, hi));
            o[2 + i] = (uint8_t)(lo | (hi << 4));
        }
    }
}

// crates/lumen-convert/src/dequant.rs:854-906.
ORC_API void orc_quantize_q8_0(const float* src, int64_t n_elements, uint8_t* dst) {
    const int64_t nb = n_elements / 32;
    for (int64_t b = 0; b < nb; ++b) {
        const float* v = src + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(v[i]));
        const float scale = amax / 127.0f;
        const float inv = (scale != 0.0f) ? 1.0f / scale : 0.0f;
        const uint16_t s16 = orc_f32_to_f16_bits(scale);
        uint8_t* o = dst + b * 34;
        o[0] = (uint8_t)(s16 & 0xFF);
        o[1] = (uint8_t)(s16 >> 8);
        for (int i = 0; i < 32; ++i) {
            float q = std::roundf(v[i] * inv);
            q = std::fmin(127.0f, std::fmax(-128.0f, q));
            o[2 + i] = (uint8_t)(int8_t)q;
        }
    }
}

ORC_API void orc_quantize_bf16(const float* src, int64_t n_elements, uint8_t* dst) {
    for (int64_t i = 0; i < n_elements; ++i) {
        const uint16_t b = orc_f32_to_bf16_bits(src[i]);
        dst[2 * i] = (uint8_t)(b & 0xFF);
        dst[2 * i + 1] = (uint8_t)(b >> 8);
    }
}

// crates/lumen-convert/src/dequant.rs:108-127 (Q8_0), :133-165 (Q4_0).
ORC_API void orc_dequantize(const uint8_t* src, int64_t n_elements, int quant, float* dst) {
    if (quant == ORC_Q8_0) {
        for (int64_t b = 0; b < n_elements / 32; ++b) {
            const uint8_t* blk = src + b * 34;
            const float s = orc_f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            for (int i = 0; i < 32; ++i) dst[b * 32 + i] = s * (float)(int8_t)blk[2 + i];
        }
    } else if (quant == ORC_Q4_0) {
        for (int64_t b = 0; b < n_elements / 32; ++b) {
            const uint8_t* blk = src + b * 18;
            const float s = orc_f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            for (int i = 0; i < 16; ++i) {
                dst[b * 32 + i] = s * (float)((int)(blk[2 + i] & 0x0F) - 8);
                dst[b * 32 + 16 + i] = s * (float)((int)((blk[2 + i] >> 4) & 0x0F) - 8);
            }
        }
    } else {
        for (int64_t i = 0; i < n_elements; ++i)
            dst[i] = bf16_bits_to_f32((uint16_t)(src[2 * i] | (src[2 * i + 1] << 8)));
    }
}

ORC_API int64_t orc_row_bytes(int in_dim, int quant) {
    if (quant == ORC_Q8_0) return (int64_t)(in_dim / 32) * 34;
    if (quant == ORC_Q4_0) return (int64_t)(in_dim / 32) * 18;
    return (int64_t)in_dim * 2;
}

// ---------------------------------------------------------------------------
// Scalar matvec rows. crates/lumen-runtime/src/compute/cpu_naive.rs:230-254
// (Q8_0: sum += (scale*q)*x[j], j ascending) and :256-283 (Q4_0: the 16 low
// nibbles then the 16 high nibbles of each block). BF16 follows
// cuda/shaders/moe_batched_bf16.cu:52-84 (sequential f32 multiply-add).
// ---------------------------------------------------------------------------
static inline float row_dot(const uint8_t* row, const float* x, int in_dim, int quant) {
    float sum = 0.0f;
    if (quant == ORC_Q8_0) {
        const int nb = in_dim / 32;
        int xi = 0;
        for (int b = 0; b < nb; ++b) {
            const uint8_t* blk = row + (size_t)b * 34;
            const float s = orc_f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            for (int k = 0; k < 32; ++k) {
                const float q = (float)(int8_t)blk[2 + k];
                sum += (s * q) * x[xi++];
            }
        }
    } else if (quant == ORC_Q4_0) {
        const int nb = in_dim / 32;
        int xi = 0;
        for (int b = 0; b < nb; ++b) {
            const uint8_t* blk = row + (size_t)b * 18;
            const float s = orc_f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            for (int k = 0; k < 16; ++k) {
                const int lo = (int)(blk[2 + k] & 0x0F) - 8;
                sum += (s * (float)lo) * x[xi++];
            }
            for (int k = 0; k < 16; ++k) {
                const int hi = (int)((blk[2 + k] >> 4) & 0x0F) - 8;
                sum += (s * (float)hi) * x[xi++];
            }
        }
    } else {
        for (int j = 0; j < in_dim; ++j) {
            const float w = bf16_bits_to_f32((uint16_t)(row[2 * j] | (row[2 * j + 1] << 8)));
            sum += w * x[j];
        }
    }
    return sum;
}

ORC_API void orc_matvec(const uint8_t* w, const float* x, float* out, int out_dim, int in_dim, int quant) {
    const int64_t rb = orc_row_bytes(in_dim, quant);
    for (int i = 0; i < out_dim; ++i) out[i] = row_dot(w + (size_t)i * rb, x, in_dim, quant);
}

// cpu_naive.rs:319-324: (g / (1 + exp(-g))) * u.
static inline float swiglu1(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

ORC_API void orc_swiglu(float* gate, const float* up, int n) {
    for (int i = 0; i < n; ++i) gate[i] = swiglu1(gate[i], up[i]);
}

// cpu_naive.rs:142-150: ms = sum(x^2)/n (sequential f32), scale = 1/sqrt(ms+eps).
ORC_API void orc_rmsnorm(float* out, const float* x, const float* weight, int n, float eps) {
    float ss = 0.0f;
    for (int i = 0; i < n; ++i) ss += x[i] * x[i];
    const float ms = ss / (float)n;
    const float scale = 1.0f / std::sqrt(ms + eps);
    for (int i = 0; i < n; ++i) out[i] = x[i] * scale * weight[i];
}

// ---------------------------------------------------------------------------
// Router. crates/lumen-runtime/src/cuda/moe.rs:6448-6505 (cpu_router_softmax).
// ---------------------------------------------------------------------------

// Phase 1 (:6456-6463): sequential dot per expert.
ORC_API void orc_router_logits(const float* x, const float* w, int H, int E, float* logits) {
    for (int e = 0; e < E; ++e) {
        float acc = 0.0f;
        for (int j = 0; j < H; ++j) acc += w[(size_t)e * H + j] * x[j];
        logits[e] = acc;
    }
}

// Phases 2+3 (:6464-6504). gating: 0 = softmax then renormalise (the CPU
// reference); 1 = sigmoid then renormalise (cuda/shaders/topk_moe_fused.cu:118-129,
// the CUDA backend's production default; same ids, different weights);
// 2 = sigmoid, weights NOT renormalised: with E = K = 1 this is the gate of the
// always-on shared expert, sigmoid(dot(ffn_gate_inp_shexp, x))
// (cuda/moe.rs:5455-5470, cuda/shaders/moe_shared_accum.cu:1-12);
// 3 = unit weights (shared expert without a gate vector, cuda/moe.rs:5483-5485).
// probs_scratch: E floats (clobbered).
ORC_API void orc_topk_from_logits(const float* logits_in, int E, int K, int gating,
                                  uint32_t* ids, float* weights, float* probs_scratch) {
    float* p = probs_scratch;
    if (gating == 0) {
        float maxv = -INFINITY;
        for (int e = 0; e < E; ++e) maxv = std::fmax(maxv, logits_in[e]);
        float sum = 0.0f;
        for (int e = 0; e < E; ++e) {
            p[e] = expf(logits_in[e] - maxv);
            sum += p[e];
        }
        for (int e = 0; e < E; ++e) p[e] /= sum;
    } else {
        for (int e = 0; e < E; ++e) p[e] = 1.0f / (1.0f + expf(-logits_in[e]));
    }
    float renorm = 0.0f;
    for (int k = 0; k < K; ++k) {
        int best_e = 0;
        float best = -1.0f;
        for (int e = 0; e < E; ++e) {
            if (p[e] > best) {
                best = p[e];
                best_e = e;
            }
        }
        ids[k] = (uint32_t)best_e;
        weights[k] = best;
        renorm += best;
        p[best_e] = -1.0f;
    }
    if (gating == 3) {
        for (int k = 0; k < K; ++k) weights[k] = 1.0f;
    } else if (gating != 2 && renorm > 0.0f) {
        for (int k = 0; k < K; ++k) weights[k] /= renorm;
    }
}

ORC_API void orc_router_softmax(const float* x, const float* w, int H, int E, int K,
                                uint32_t* ids, float* weights, float* logits_out) {
    std::vector<float> logits(E), scratch(E);
    orc_router_logits(x, w, H, E, logits.data());
    if (logits_out) std::memcpy(logits_out, logits.data(), sizeof(float) * E);
    orc_topk_from_logits(logits.data(), E, K, 0, ids, weights, scratch.data());
}

// ---------------------------------------------------------------------------
// Combine. cuda/moe.rs:6508-6524 (dense slots) and :6527-6545 (sparse slots).
// ---------------------------------------------------------------------------
ORC_API void orc_accum_option_a(const float* residual, const float* expert_outputs,
                                const float* expert_weights, int H, int K, float* out) {
    for (int i = 0; i < H; ++i) {
        float acc = residual[i];
        for (int k = 0; k < K; ++k) acc += expert_weights[k] * expert_outputs[(size_t)k * H + i];
        out[i] = acc;
    }
}

ORC_API void orc_accum_batched_b(const float* residual, const float* expert_outputs,
                                 const float* expert_weights, const uint32_t* expert_ids,
                                 int H, int K, float* out) {
    for (int i = 0; i < H; ++i) {
        float acc = residual[i];
        for (int k = 0; k < K; ++k)
            acc += expert_weights[k] * expert_outputs[(size_t)expert_ids[k] * H + i];
        out[i] = acc;
    }
}

// ---------------------------------------------------------------------------
// Permutation. cuda/moe.rs:2115-2147: stable counting sort of (token, slot)
// pairs by expert, tokens ascending then slots ascending. ids has row stride
// ids_stride (the reference's batched buffer uses stride E; ours uses K).
// ---------------------------------------------------------------------------
ORC_API void orc_counting_sort(const uint32_t* ids, int T, int K, int E, int ids_stride,
                               int32_t* col_expert, int32_t* col_src_tok, int32_t* dst_to_col,
                               int32_t* expert_bounds) {
    std::vector<int32_t> counts(E, 0);
    for (int t = 0; t < T; ++t)
        for (int s = 0; s < K; ++s) counts[ids[(size_t)t * ids_stride + s]]++;
    expert_bounds[0] = 0;
    for (int e = 0; e < E; ++e) expert_bounds[e + 1] = expert_bounds[e] + counts[e];
    std::vector<int32_t> cursor(expert_bounds, expert_bounds + E);
    for (int t = 0; t < T; ++t) {
        for (int s = 0; s < K; ++s) {
            const int e = (int)ids[(size_t)t * ids_stride + s];
            const int c = cursor[e]++;
            col_expert[c] = e;
            col_src_tok[c] = t;
            dst_to_col[(size_t)t * K + s] = c;
        }
    }
}

// ---------------------------------------------------------------------------
// Whole layer: composition as in crates/lumen-runtime/src/metal/tests/moe.rs:884-909
// (per token, per selected expert: gate/up rows -> SwiGLU -> down rows), with the
// in-place quantised row arithmetic of cpu_naive.rs and the combine order of
// cuda/moe.rs:6508-6524 (acc = residual; slots ascending).
//
// blob layout as produced by crates/lumen-convert/src/arch/qwen35_moe.rs:512-551:
// router f32 [E,H] at router_off; expert e gate [I,H] at gate_offs[e], up [I,H]
// at up_offs[e], down [H,I] at down_offs[e]; rows are runs of blocks along the
// input dimension.
//
// routing_mode: 0 = route from x with the router weight; 1 = take logits_in
// [T,E] as given (identical-logits parity tests); 2 = take ids_in/weights_in.
// ---------------------------------------------------------------------------
struct LayerArgs {
    const uint8_t* blob;
    uint64_t router_off;
    const uint64_t *gate_offs, *up_offs, *down_offs;
    int quant, H, I, E, K, T, gating;
};

static void parallel_for(int64_t n, int threads, const std::function<void(int64_t, int64_t)>& fn) {
    if (threads <= 1 || n <= 1) {
        fn(0, n);
        return;
    }
    const int nt = (int)std::min<int64_t>(threads, n);
    std::vector<std::thread> th;
    th.reserve(nt);
    for (int i = 0; i < nt; ++i) {
        const int64_t lo = n * i / nt, hi = n * (i + 1) / nt;
        th.emplace_back([=, &fn] { fn(lo, hi); });
    }
    for (auto& t : th) t.join();
}

ORC_API int orc_moe_layer(const uint8_t* blob, uint64_t router_off, const uint64_t* gate_offs,
                          const uint64_t* up_offs, const uint64_t* down_offs, int quant, int H,
                          int I, int E, int K, int T, int gating, int routing_mode,
                          const float* normed, const float* residual, const float* logits_in,
                          uint32_t* ids_io, float* weights_io, float* out, int threads) {
    if (quant < 0 || quant > 2 || H % 32 || I % 32 || K > E) return 1;
    const float* wr = reinterpret_cast<const float*>(blob + router_off);
    // routing (parallel over tokens; per-token arithmetic is sequential)
    if (routing_mode != 2) {
        parallel_for(T, threads, [&](int64_t lo, int64_t hi) {
            std::vector<float> logits(E), scratch(E);
            for (int64_t t = lo; t < hi; ++t) {
                const float* lg;
                if (routing_mode == 0) {
                    orc_router_logits(normed + t * H, wr, H, E, logits.data());
                    lg = logits.data();
                } else {
                    lg = logits_in + t * E;
                }
                orc_topk_from_logits(lg, E, K, gating, ids_io + t * K, weights_io + t * K, scratch.data());
            }
        });
    }
    const int64_t rb_h = orc_row_bytes(H, quant), rb_i = orc_row_bytes(I, quant);
    std::vector<float> sw((size_t)T * K * I), dn((size_t)T * K * H);
    // gate/up + SwiGLU: parallel over (token, slot, row)
    parallel_for((int64_t)T * K * I, threads, [&](int64_t lo, int64_t hi) {
        for (int64_t idx = lo; idx < hi; ++idx) {
            const int64_t p = idx / I;
            const int r = (int)(idx % I);
            const int64_t t = p / K;
            const uint32_t e = ids_io[p];
            const float g = row_dot(blob + gate_offs[e] + (size_t)r * rb_h, normed + t * H, H, quant);
            const float u = row_dot(blob + up_offs[e] + (size_t)r * rb_h, normed + t * H, H, quant);
            sw[idx] = swiglu1(g, u);
        }
    });
    parallel_for((int64_t)T * K * H, threads, [&](int64_t lo, int64_t hi) {
        for (int64_t idx = lo; idx < hi; ++idx) {
            const int64_t p = idx / H;
            const int r = (int)(idx % H);
            const uint32_t e = ids_io[p];
            dn[idx] = row_dot(blob + down_offs[e] + (size_t)r * rb_i, sw.data() + p * I, I, quant);
        }
    });
    parallel_for(T, threads, [&](int64_t lo, int64_t hi) {
        for (int64_t t = lo; t < hi; ++t)
            orc_accum_option_a(residual + t * H, dn.data() + t * K * H, weights_io + t * K, H, K, out + t * H);
    });
    return 0;
}

// 48-layer style stack: x <- x + MoE(rmsnorm(x; gamma_l, eps)) per layer, the
// attention / GDN mixers replaced by identity. Wrapper semantics follow
// cuda/moe.rs:3214-3291 (standalone rmsnorm, MoE input = normed, residual = x).
// blobs[l] / offs tables are per layer. x is updated in place; [T,H].
ORC_API int orc_moe_stack(int L, const uint8_t* const* blobs, const uint64_t* router_offs,
                          const uint64_t* const* gate_offs, const uint64_t* const* up_offs,
                          const uint64_t* const* down_offs, const float* const* gammas, float eps,
                          int quant, int H, int I, int E, int K, int T, float* x, int threads) {
    std::vector<float> normed((size_t)T * H), out((size_t)T * H), w((size_t)T * K);
    std::vector<uint32_t> ids((size_t)T * K);
    for (int l = 0; l < L; ++l) {
        for (int t = 0; t < T; ++t)
            orc_rmsnorm(normed.data() + (size_t)t * H, x + (size_t)t * H, gammas[l], H, eps);
        int rc = orc_moe_layer(blobs[l], router_offs[l], gate_offs[l], up_offs[l], down_offs[l], quant,
                               H, I, E, K, T, 0, 0, normed.data(), x, nullptr, ids.data(), w.data(),
                               out.data(), threads);
        if (rc) return rc;
        std::memcpy(x, out.data(), sizeof(float) * (size_t)T * H);
    }
    return 0;
}

ORC_API int orc_hardware_threads() { return (int)std::thread::hardware_concurrency(); }
