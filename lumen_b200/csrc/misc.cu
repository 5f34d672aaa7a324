// One-time and auxiliary kernels: repack of the raw layer blob into fragment
// planes, device quantisers for synthetic weights, standalone RMSNorm, and the
// device check of the router's exp.
#include "moe_internal.cuh"
#include "exact_expf.h"

namespace lumen {

// ---------------------------------------------------------------------------
// Repack (the counterpart of build_repacked_down, cuda/moe.rs:337-394, and of
// moe_repack_down_q8_0 / moe_repack_gate_up_q8_0, cuda/shaders/moe_grouped.cu:1772,1831;
// done here for every quant type and for both decode and prefill consumers).
// The raw blob is only read (byte loads: raw blocks are 2-byte aligned at best).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_u32_bytes(const uint8_t* p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

template <int Q>
__device__ __forceinline__ uint32_t raw_word(const uint8_t* mat, int rows, int nblk, int r, int b, int i) {
    // word i of block b of row r; out-of-range blocks decode to zero values
    if (Q == Q4_0) {
        if (b >= nblk || r >= rows) return 0x88888888u;
        return ld_u32_bytes(mat + ((size_t)r * nblk + b) * 18 + 2 + 4 * i);
    } else if (Q == Q8_0) {
        if (b >= nblk || r >= rows) return 0u;
        return ld_u32_bytes(mat + ((size_t)r * nblk + b) * 34 + 2 + 4 * i);
    } else {
        // BF16: word i (0..15) = elements 2i, 2i+1 of the 32-element block
        if (b >= nblk || r >= rows) return 0u;
        return ld_u32_bytes(mat + (((size_t)r * nblk + b) * 32 + 2 * i) * 2);
    }
}

template <int Q>
__global__ void repack_q_kernel(const uint8_t* __restrict__ blob, const uint64_t* __restrict__ offs,
                                int rows, int nblk, int kg_n, int rt_n, uint4* __restrict__ out,
                                size_t mat_off_u4, size_t exp_stride_u4) {
    constexpr int NQ = (Q == Q4_0) ? 2 : (Q == Q8_0) ? 4 : 8;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)rt_n * kg_n * NQ * 32;
    if (idx >= total) return;
    const int e = blockIdx.y;
    const int lane = (int)(idx & 31);
    const int j = (int)((idx >> 5) % NQ);
    const size_t tile = idx / (32 * NQ);
    const int kg = (int)(tile % kg_n), rt = (int)(tile / kg_n);
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* mat = blob + offs[e];
    const int r0 = rt * 16 + g, r1 = r0 + 8;
    uint4 v;
    if (Q == Q4_0) {
        const int b0 = kg * 4 + 2 * j, b1 = b0 + 1;
        v.x = raw_word<Q>(mat, rows, nblk, r0, b0, t);
        v.y = raw_word<Q>(mat, rows, nblk, r1, b0, t);
        v.z = raw_word<Q>(mat, rows, nblk, r0, b1, t);
        v.w = raw_word<Q>(mat, rows, nblk, r1, b1, t);
    } else if (Q == Q8_0) {
        const int b = kg * 4 + j;
        v.x = raw_word<Q>(mat, rows, nblk, r0, b, t);
        v.y = raw_word<Q>(mat, rows, nblk, r0, b, 4 + t);
        v.z = raw_word<Q>(mat, rows, nblk, r1, b, t);
        v.w = raw_word<Q>(mat, rows, nblk, r1, b, 4 + t);
    } else {
        const int b = kg * 4 + (j >> 1);
        const int r = (j & 1) ? r1 : r0;
        v.x = raw_word<Q>(mat, rows, nblk, r, b, 2 * t);
        v.y = raw_word<Q>(mat, rows, nblk, r, b, 2 * t + 1);
        v.z = raw_word<Q>(mat, rows, nblk, r, b, 8 + 2 * t);
        v.w = raw_word<Q>(mat, rows, nblk, r, b, 8 + 2 * t + 1);
    }
    out[(size_t)e * exp_stride_u4 + mat_off_u4 + idx] = v;
}

__global__ void repack_s_kernel(const uint8_t* __restrict__ blob, const uint64_t* __restrict__ offs,
                                int rows, int nblk, int blk_bytes, int kg_n, int rt_n,
                                uint4* __restrict__ out, size_t mat_off_u4, size_t exp_stride_u4) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)rt_n * kg_n * 8;
    if (idx >= total) return;
    const int e = blockIdx.y;
    const int g = (int)(idx & 7);
    const size_t tile = idx >> 3;
    const int kg = (int)(tile % kg_n), rt = (int)(tile / kg_n);
    const uint8_t* mat = blob + offs[e];
    uint32_t h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = rt * 16 + g + ((i >= 4) ? 8 : 0);
        const int b = kg * 4 + (i & 3);
        uint32_t bits = 0u;
        if (b < nblk && r < rows) {
            const uint8_t* p = mat + ((size_t)r * nblk + b) * blk_bytes;
            bits = (uint32_t)p[0] | ((uint32_t)p[1] << 8);
        }
        h[i] = bits;
    }
    uint4 v;
    v.x = h[0] | (h[1] << 16);
    v.y = h[2] | (h[3] << 16);
    v.z = h[4] | (h[5] << 16);
    v.w = h[6] | (h[7] << 16);
    out[(size_t)e * exp_stride_u4 + mat_off_u4 + idx] = v;
}

template <int Q>
static cudaError_t repack_t(const uint8_t* blob, const uint64_t* d_gate, const uint64_t* d_up,
                            const uint64_t* d_down, const LayerDev& L, uint4* q, uint4* s,
                            cudaStream_t st) {
    const int nq = L.nq;
    const int nblk_h = L.H / 32, nblk_i = L.I / 32;
    const int blk_bytes = (Q == Q4_0) ? 18 : 34;
    {
        const size_t total = (size_t)L.rt_i * L.kg_h * nq * 32;
        const dim3 grid((unsigned)((total + 255) / 256), L.E);
        repack_q_kernel<Q><<<grid, 256, 0, st>>>(blob, d_gate, L.I, nblk_h, L.kg_h, L.rt_i, q, 0, L.q_exp);
        repack_q_kernel<Q><<<grid, 256, 0, st>>>(blob, d_up, L.I, nblk_h, L.kg_h, L.rt_i, q, L.q_gu, L.q_exp);
        count_launch(2);
    }
    {
        const size_t total = (size_t)L.rt_h * L.kg_i * nq * 32;
        const dim3 grid((unsigned)((total + 255) / 256), L.E);
        repack_q_kernel<Q><<<grid, 256, 0, st>>>(blob, d_down, L.H, nblk_i, L.kg_i, L.rt_h, q, 2 * L.q_gu, L.q_exp);
        count_launch(1);
    }
    if (Q != BF16) {
        {
            const size_t total = (size_t)L.rt_i * L.kg_h * 8;
            const dim3 grid((unsigned)((total + 255) / 256), L.E);
            repack_s_kernel<<<grid, 256, 0, st>>>(blob, d_gate, L.I, nblk_h, blk_bytes, L.kg_h, L.rt_i, s, 0, L.s_exp);
            repack_s_kernel<<<grid, 256, 0, st>>>(blob, d_up, L.I, nblk_h, blk_bytes, L.kg_h, L.rt_i, s, L.s_gu, L.s_exp);
        }
        {
            const size_t total = (size_t)L.rt_h * L.kg_i * 8;
            const dim3 grid((unsigned)((total + 255) / 256), L.E);
            repack_s_kernel<<<grid, 256, 0, st>>>(blob, d_down, L.H, nblk_i, blk_bytes, L.kg_i, L.rt_h, s, 2 * L.s_gu, L.s_exp);
        }
        count_launch(3);
    }
    return cudaGetLastError();
}

// Expert weights as plain f16 matrices (scale folded in, one rounding: the value the grouped
// GEMM's in-smem dequantiser produces), row-major, for the TMA-fed form of the prefill
// products: gu16 [E][2 I rows: gate then up][H], dn16 [E][H rows][I]. One thread per 32-block.
template <int Q>
__global__ void dequant_rows_f16_kernel(const uint8_t* __restrict__ blob, const uint64_t* __restrict__ offs, int rows,
                                        int nblk, size_t exp_rows, size_t row_off, __half* __restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * nblk) return;
    const int e = blockIdx.y;
    const int r = (int)(idx / nblk), b = (int)(idx % nblk);
    const uint8_t* mat = blob + offs[e];
    __align__(16) __half v[32];
    if (Q == BF16) {
        const uint8_t* p = mat + ((size_t)r * nblk + b) * 64;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const uint32_t bits = ((uint32_t)p[2 * i] | ((uint32_t)p[2 * i + 1] << 8)) << 16;
            v[i] = __float2half_rn(__uint_as_float(bits));
        }
    } else {
        const int bb = (Q == Q4_0) ? 18 : 34;
        const uint8_t* p = mat + ((size_t)r * nblk + b) * bb;
        const float sc = __half2float(__ushort_as_half((unsigned short)((uint32_t)p[0] | ((uint32_t)p[1] << 8))));
        if (Q == Q4_0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                v[i] = __float2half_rn((float)((int)(p[2 + i] & 0xF) - 8) * sc);
                v[16 + i] = __float2half_rn((float)((int)(p[2 + i] >> 4) - 8) * sc);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float2half_rn((float)(int)(int8_t)p[2 + i] * sc);
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + (((size_t)e * exp_rows + row_off + r) * nblk + b) * 32);
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = reinterpret_cast<const uint4*>(v)[i];
}

template <int Q>
static cudaError_t dequant_f16_t(const uint8_t* blob, const uint64_t* d_gate, const uint64_t* d_up, const uint64_t* d_down,
                                 const LayerDev& L, __half* gu16, __half* dn16, cudaStream_t st) {
    const int nblk_h = L.H / 32, nblk_i = L.I / 32;
    const dim3 g_gu((unsigned)(((size_t)L.I * nblk_h + 255) / 256), L.E), g_dn((unsigned)(((size_t)L.H * nblk_i + 255) / 256), L.E);
    count_launch(3);
    dequant_rows_f16_kernel<Q><<<g_gu, 256, 0, st>>>(blob, d_gate, L.I, nblk_h, (size_t)2 * L.I, 0, gu16);
    dequant_rows_f16_kernel<Q><<<g_gu, 256, 0, st>>>(blob, d_up, L.I, nblk_h, (size_t)2 * L.I, (size_t)L.I, gu16);
    dequant_rows_f16_kernel<Q><<<g_dn, 256, 0, st>>>(blob, d_down, L.H, nblk_i, (size_t)L.H, 0, dn16);
    return cudaGetLastError();
}

cudaError_t launch_dequant_f16(const uint8_t* blob, const uint64_t* d_gate_offs, const uint64_t* d_up_offs,
                               const uint64_t* d_down_offs, const LayerDev& L, __half* gu16, __half* dn16,
                               cudaStream_t st) {
    switch (L.quant) {
        case Q4_0: return dequant_f16_t<Q4_0>(blob, d_gate_offs, d_up_offs, d_down_offs, L, gu16, dn16, st);
        case Q8_0: return dequant_f16_t<Q8_0>(blob, d_gate_offs, d_up_offs, d_down_offs, L, gu16, dn16, st);
        default: return dequant_f16_t<BF16>(blob, d_gate_offs, d_up_offs, d_down_offs, L, gu16, dn16, st);
    }
}

cudaError_t launch_repack(const uint8_t* blob, const uint64_t* d_gate_offs, const uint64_t* d_up_offs,
                          const uint64_t* d_down_offs, const LayerDev& L, uint4* q, uint4* s,
                          cudaStream_t st) {
    switch (L.quant) {
        case Q4_0: return repack_t<Q4_0>(blob, d_gate_offs, d_up_offs, d_down_offs, L, q, s, st);
        case Q8_0: return repack_t<Q8_0>(blob, d_gate_offs, d_up_offs, d_down_offs, L, q, s, st);
        default: return repack_t<BF16>(blob, d_gate_offs, d_up_offs, d_down_offs, L, q, s, st);
    }
}

// ---------------------------------------------------------------------------
// Quantisers (crates/lumen-convert/src/dequant.rs:741-906), one thread per block.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint16_t f32_to_f16_bits_trunc(float val) {
    const uint32_t bits = __float_as_uint(val);
    const uint32_t sign = (bits >> 31) & 1u;
    const int exp = (int)((bits >> 23) & 0xFFu);
    const uint32_t frac = bits & 0x7FFFFFu;
    if (exp == 255) return (uint16_t)((sign << 15) | (0x1Fu << 10) | (frac != 0 ? 0x200u : 0u));
    const int new_exp = exp - 127 + 15;
    if (new_exp >= 31) return (uint16_t)((sign << 15) | (0x1Fu << 10));
    if (new_exp <= 0) {
        if (new_exp < -10) return (uint16_t)(sign << 15);
        const uint32_t mant = frac | 0x00800000u;
        return (uint16_t)((sign << 15) | ((mant >> (uint32_t)(14 - new_exp)) & 0x3FFu));
    }
    return (uint16_t)((sign << 15) | ((uint32_t)new_exp << 10) | (frac >> 13));
}

__global__ void quantize_q4_0_kernel(const float* __restrict__ src, int64_t nblocks, uint16_t* __restrict__ dst) {
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const float4* v4 = reinterpret_cast<const float4*>(src + b * 32);
    float v[32];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 t = v4[i];
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float scale = (amax == 0.0f) ? 1.0f : fminf(__fdiv_rn(amax, 7.0f), 65504.0f);
    const float inv = (scale == 0.0f) ? 0.0f : __fdiv_rn(1.0f, scale);
    uint16_t* o = dst + b * 9;
    o[0] = f32_to_f16_bits_trunc(scale);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t w = 0;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int idx = 2 * i + k;
            int lo = (int)roundf(__fmul_rn(v[idx], inv)) + 8;
            int hi = (int)roundf(__fmul_rn(v[idx + 16], inv)) + 8;
            lo = min(15, max(0, lo));
            hi = min(15, max(0, hi));
            w |= (uint32_t)(lo | (hi << 4)) << (8 * k);
        }
        o[1 + i] = (uint16_t)w;
    }
}

__global__ void quantize_q8_0_kernel(const float* __restrict__ src, int64_t nblocks, uint16_t* __restrict__ dst) {
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const float4* v4 = reinterpret_cast<const float4*>(src + b * 32);
    float v[32];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 t = v4[i];
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float scale = __fdiv_rn(amax, 127.0f);
    const float inv = (scale != 0.0f) ? __fdiv_rn(1.0f, scale) : 0.0f;
    uint16_t* o = dst + b * 17;
    o[0] = f32_to_f16_bits_trunc(scale);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float q0 = fminf(127.0f, fmaxf(-128.0f, roundf(__fmul_rn(v[2 * i], inv))));
        float q1 = fminf(127.0f, fmaxf(-128.0f, roundf(__fmul_rn(v[2 * i + 1], inv))));
        const uint32_t b0 = (uint32_t)(uint8_t)(int8_t)(int)q0, b1 = (uint32_t)(uint8_t)(int8_t)(int)q1;
        o[1 + i] = (uint16_t)(b0 | (b1 << 8));
    }
}

__global__ void quantize_bf16_kernel(const float* __restrict__ src, int64_t n, uint16_t* __restrict__ dst) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    dst[i] = __bfloat16_as_ushort(__float2bfloat16_rn(src[i]));
}

cudaError_t launch_quantize(const float* src, int64_t n, int quant, void* dst, cudaStream_t st) {
    count_launch();
    if (quant == Q4_0) {
        const int64_t nb = n / 32;
        quantize_q4_0_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(src, nb, (uint16_t*)dst);
    } else if (quant == Q8_0) {
        const int64_t nb = n / 32;
        quantize_q8_0_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(src, nb, (uint16_t*)dst);
    } else {
        quantize_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(src, n, (uint16_t*)dst);
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Standalone RMSNorm over rows (cuda/shaders/norm.cu:28-76; cpu_naive.rs:142-150).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                      float* __restrict__ out, int H, float eps) {
    __shared__ float red[8];
    __shared__ float scale_s;
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* xr = x + (size_t)t * H;
    float ss = 0.0f;
    for (int i = tid; i < H; i += 256) ss += xr[i] * xr[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
        float s = 0.0f;
        for (int w = 0; w < 8; ++w) s += red[w];
        scale_s = 1.0f / sqrtf(s / (float)H + eps);
    }
    __syncthreads();
    const float sc = scale_s;
    for (int i = tid; i < H; i += 256) out[(size_t)t * H + i] = xr[i] * sc * gamma[i];
}

cudaError_t launch_rmsnorm(const float* x, const float* gamma, float* out, int T, int H, float eps,
                           cudaStream_t st) {
    count_launch();
    rmsnorm_kernel<<<T, 256, 0, st>>>(x, gamma, out, H, eps);
    return cudaGetLastError();
}

__global__ void debug_expf_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = lumen_exact::expf_libm(in[i]);
}

cudaError_t launch_debug_expf(const float* in, float* out, int64_t n, cudaStream_t st) {
    count_launch();
    debug_expf_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(in, out, n);
    return cudaGetLastError();
}

}  // namespace lumen
