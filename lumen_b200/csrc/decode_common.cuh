// Device helpers shared by the small-batch decode kernels (decode_small.cu,
// decode_fused.cu).
#pragma once
#include "mma_frag.cuh"

namespace lumen {
namespace dcommon {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// position of row r (mod 4) inside a fragment word pair: rows 0,2,1,3 -> 0,1,2,3
__device__ __forceinline__ int frag_pos(int r) {
    const int m = r & 3;
    return (m == 0) ? 0 : (m == 2) ? 1 : (m == 1) ? 2 : 3;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// D (s32) += A (u8, 16 x 32) * B (s8, 32 x 8): Q4_0 nibbles go in raw as A.
__device__ __forceinline__ void mma_u8s8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack_s8x4(float a, float b, float c, float d) {
    return ((unsigned)(int)a & 0xffu) | (((unsigned)(int)b & 0xffu) << 8) | (((unsigned)(int)c & 0xffu) << 16) |
           (((unsigned)(int)d & 0xffu) << 24);
}

// Two-term int8 form of the activations for the Q4_0 gate/up product: x ~ sx * (q0 + q1 / 254)
// per 32-input block, sx = absmax / 127. Per token, in 32-bit words:
//   [2 terms][nblk_pad * 8 + 8]   the word pair of lane quad t of a block is adjacent:
//                                 {inputs 4t..4t+3, inputs 16+4t..16+4t+3} (the s8 B fragment)
//   [nblk_pad] float2             {sx, 8 * sx * sum(q0 + q1 / 254)}: the nibbles enter unsigned,
//                                 the second value removes their offset of 8
__host__ __device__ __forceinline__ int xq_term_words(int nblk_pad) { return nblk_pad * 8 + 8; }
__host__ __device__ __forceinline__ int xq_tok_words(int nblk_pad) { return 2 * xq_term_words(nblk_pad) + 2 * nblk_pad; }

// The 8 lanes of a block (sub = 0..7, consecutive lanes of a warp) each bring inputs 4 sub .. 4 sub + 3.
__device__ __forceinline__ void build_xq_block(float4 v, int sub, int lane, unsigned* xq_tok_base, int nblk_pad, int b) {
    const unsigned gmask = 0xFFu << (lane & 24);
    float am = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) am = fmaxf(am, __shfl_xor_sync(gmask, am, o));
    const float inv = (am > 0.0f) ? 127.0f / am : 0.0f;
    const float sx = am * (1.0f / 127.0f);
    const float r0 = v.x * inv, r1 = v.y * inv, r2 = v.z * inv, r3 = v.w * inv;
    const float q00 = rintf(r0), q01 = rintf(r1), q02 = rintf(r2), q03 = rintf(r3);
    const float q10 = rintf((r0 - q00) * 254.0f), q11 = rintf((r1 - q01) * 254.0f);
    const float q12 = rintf((r2 - q02) * 254.0f), q13 = rintf((r3 - q03) * 254.0f);
    float sum = (q00 + q01 + q02 + q03) + (q10 + q11 + q12 + q13) * (1.0f / 254.0f);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(gmask, sum, o);
    const int term = xq_term_words(nblk_pad);
    unsigned* base = xq_tok_base + b * 8 + (sub & 3) * 2 + (sub >> 2);
    base[0] = pack_s8x4(q00, q01, q02, q03);
    base[term] = pack_s8x4(q10, q11, q12, q13);
    if (sub == 0) reinterpret_cast<float2*>(xq_tok_base + 2 * term)[b] = make_float2(sx, 8.0f * sx * sum);
}

// One 32-input block (two MMAs) of one column group; the B fragment comes from shared memory.
template <int Q>
__device__ __forceinline__ void block_mma_smem(const WTile<Q>& w, int b, const uint4* bsm, bool bvalid,
                                               float (&acc)[4]) {
    uint32_t a_lo[4], a_hi[4];
    unpack_block<Q>(w, b, a_lo, a_hi);
    const float2 sc = block_scales<Q>(w, b);
    uint4 bf = make_uint4(0u, 0u, 0u, 0u);
    if (bvalid) bf = bsm[b * 4];
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    if (Q == BF16) {
        mma_bf16(c, a_lo, bf.x, bf.y);
        mma_bf16(c, a_hi, bf.z, bf.w);
    } else {
        mma_f16(c, a_lo, bf.x, bf.y);
        mma_f16(c, a_hi, bf.z, bf.w);
    }
    acc[0] = fmaf(sc.x, c[0], acc[0]);
    acc[1] = fmaf(sc.x, c[1], acc[1]);
    acc[2] = fmaf(sc.y, c[2], acc[2]);
    acc[3] = fmaf(sc.y, c[3], acc[3]);
}

// SwiGLU value -> high/low 16-bit parts in the operand type of the down product,
// stored at the fragment position of (column, inter row) in the sf planes.
template <int Q>
__device__ __forceinline__ void store_swiglu_frag(uint4* sf, int col, int irow, int nblk_i_pad, float sv) {
    unsigned short hi_bits, lo_bits;
    if (Q != BF16) {
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
    const int blk = irow >> 5, within = irow & 31, j = within >> 4, r16 = within & 15;
    unsigned short* sf16 = reinterpret_cast<unsigned short*>(sf);
    const size_t in_vec = (size_t)j * 4 + frag_pos(r16);
    sf16[(((size_t)(col * 2 + 0) * nblk_i_pad + blk) * 4 + (r16 >> 2)) * 8 + in_vec] = hi_bits;
    sf16[(((size_t)(col * 2 + 1) * nblk_i_pad + blk) * 4 + (r16 >> 2)) * 8 + in_vec] = lo_bits;
}

}  // namespace dcommon
}  // namespace lumen
