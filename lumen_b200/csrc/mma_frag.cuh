// Warp-level building blocks of the decode (and small-batch) expert products:
// streaming 128-bit loads of the repacked weight tiles, in-register dequantisation
// to exact integer-valued f16 operands, m16n8k16 tensor-core multiply with f32
// accumulation, and the per-block f32 rescale.
//
// One weight tile = 16 rows x 128 inputs (4 blocks of 32). For block b the warp
// issues two MMAs: the first covers elements 0..15 of the block, the second
// elements 16..31. Within an MMA the k-slot -> element map of lane quad t is
//   slot 2t -> 4t, 2t+1 -> 4t+2, 2t+8 -> 4t+1, 2t+9 -> 4t+3   (+16 for the second MMA),
// which is what unpacking a 32-bit word of Q4_0 nibbles (or Q8_0 bytes) yields
// without any cross-lane traffic. The activation fragments (moe_internal.cuh)
// are stored in the same order, so the permutation cancels.
//
// Arithmetic contract (the reference's, compute/cpu_naive.rs:230-283 and
// cuda/shaders/moe_expert_q4_0.cu:78-104): integer quants times activations
// summed per 32-block in f32, then multiplied by the block's f16 scale and
// accumulated in f32. Activations enter as a two-term f16 split (high + low
// part, 22 significand bits) in adjacent MMA columns, so no precision is lost
// against the f32 activations of the reference.
#pragma once
#include "moe_internal.cuh"

namespace lumen {

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint4 ldg_cached(const uint4* p) { return __ldg(p); }

__device__ __forceinline__ uint32_t lop_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & b) | c
    return r;
}

__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int Q>
struct QTraits;
template <>
struct QTraits<Q4_0> {
    static constexpr int NQ = 2;
};
template <>
struct QTraits<Q8_0> {
    static constexpr int NQ = 4;
};
template <>
struct QTraits<BF16> {
    static constexpr int NQ = 8;
};

// One lane's share of a weight tile.
template <int Q>
struct WTile {
    uint4 q[QTraits<Q>::NQ];
    uint4 s;
};

template <int Q>
__device__ __forceinline__ void load_wtile(WTile<Q>& w, const uint4* qbase, const uint4* sbase, int tile,
                                           int lane) {
    constexpr int NQ = QTraits<Q>::NQ;
    const uint4* qp = qbase + ((size_t)tile * NQ) * 32 + lane;
#pragma unroll
    for (int j = 0; j < NQ; ++j) w.q[j] = ldg_stream(qp + j * 32);
    if (Q != BF16) w.s = ldg_stream(sbase + (size_t)tile * 8 + (lane >> 2));
}

// A fragments of the two MMAs of block b of the tile: a_lo covers elements 0..15,
// a_hi elements 16..31. Values are the exact integers (q - 8) / q as f16, or the
// bf16 weights themselves.
template <int Q>
__device__ __forceinline__ void unpack_block(const WTile<Q>& w, int b, uint32_t (&a_lo)[4],
                                             uint32_t (&a_hi)[4]) {
    if (Q == Q4_0) {
        const uint4 v = w.q[b >> 1];
        const uint32_t wg = (b & 1) ? v.z : v.x;   // row g
        const uint32_t wg8 = (b & 1) ? v.w : v.y;  // row g+8
        const uint32_t sub_lo = 0x64086408u;       // 1032 = 1024 + 8
        const uint32_t sub_hi = 0x54805480u;       // 72   = 64 + 8
        a_lo[0] = hsub2_u32(lop_and_or(wg, 0x000F000Fu, 0x64006400u), sub_lo);
        a_lo[1] = hsub2_u32(lop_and_or(wg8, 0x000F000Fu, 0x64006400u), sub_lo);
        a_lo[2] = hsub2_u32(lop_and_or(wg >> 8, 0x000F000Fu, 0x64006400u), sub_lo);
        a_lo[3] = hsub2_u32(lop_and_or(wg8 >> 8, 0x000F000Fu, 0x64006400u), sub_lo);
        a_hi[0] = hsub2_u32(lop_and_or(wg, 0x00F000F0u, 0x54005400u), sub_hi);
        a_hi[1] = hsub2_u32(lop_and_or(wg8, 0x00F000F0u, 0x54005400u), sub_hi);
        a_hi[2] = hsub2_u32(lop_and_or(wg >> 8, 0x00F000F0u, 0x54005400u), sub_hi);
        a_hi[3] = hsub2_u32(lop_and_or(wg8 >> 8, 0x00F000F0u, 0x54005400u), sub_hi);
    } else if (Q == Q8_0) {
        const uint4 v = w.q[b];
        // bytes biased by 128 -> unsigned; 0x64xx = 1024 + xx; subtract 1152.
        const uint32_t sub = 0x64806480u;
        const uint32_t x0 = v.x ^ 0x80808080u, x1 = v.y ^ 0x80808080u;
        const uint32_t y0 = v.z ^ 0x80808080u, y1 = v.w ^ 0x80808080u;
        a_lo[0] = hsub2_u32(prmt(x0, 0x64646464u, 0x4240u), sub);
        a_lo[1] = hsub2_u32(prmt(y0, 0x64646464u, 0x4240u), sub);
        a_lo[2] = hsub2_u32(prmt(x0, 0x64646464u, 0x4341u), sub);
        a_lo[3] = hsub2_u32(prmt(y0, 0x64646464u, 0x4341u), sub);
        a_hi[0] = hsub2_u32(prmt(x1, 0x64646464u, 0x4240u), sub);
        a_hi[1] = hsub2_u32(prmt(y1, 0x64646464u, 0x4240u), sub);
        a_hi[2] = hsub2_u32(prmt(x1, 0x64646464u, 0x4341u), sub);
        a_hi[3] = hsub2_u32(prmt(y1, 0x64646464u, 0x4341u), sub);
    } else {
        const uint4 r0 = w.q[2 * b];      // row g:   {e0e1, e2e3, e16e17, e18e19} (+4t)
        const uint4 r1 = w.q[2 * b + 1];  // row g+8
        a_lo[0] = prmt(r0.x, r0.y, 0x5410u);
        a_lo[1] = prmt(r1.x, r1.y, 0x5410u);
        a_lo[2] = prmt(r0.x, r0.y, 0x7632u);
        a_lo[3] = prmt(r1.x, r1.y, 0x7632u);
        a_hi[0] = prmt(r0.z, r0.w, 0x5410u);
        a_hi[1] = prmt(r1.z, r1.w, 0x5410u);
        a_hi[2] = prmt(r0.z, r0.w, 0x7632u);
        a_hi[3] = prmt(r1.z, r1.w, 0x7632u);
    }
}

// f32 scales of block b for rows g (first) and g+8 (second).
template <int Q>
__device__ __forceinline__ float2 block_scales(const WTile<Q>& w, int b) {
    if (Q == BF16) return make_float2(1.0f, 1.0f);
    const uint32_t lo = (b < 2) ? w.s.x : w.s.y;
    const uint32_t hi = (b < 2) ? w.s.z : w.s.w;
    const __half2 hl = *reinterpret_cast<const __half2*>(&lo);
    const __half2 hh = *reinterpret_cast<const __half2*>(&hi);
    const float sg = (b & 1) ? __high2float(hl) : __low2float(hl);
    const float sg8 = (b & 1) ? __high2float(hh) : __low2float(hh);
    return make_float2(sg, sg8);
}

// acc[grp] += scale * (A_block x B_block) for NG column groups of 8 columns.
// bptr[grp]: this lane's activation-fragment pointer for the tile's first block
// (already offset by lane t), or nullptr if the lane's column is unused.
template <int Q, int NG>
__device__ __forceinline__ void tile_mma(const WTile<Q>& w, const uint4* (&bptr)[NG], int ngroups,
                                         float (&acc)[NG][4]) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        uint32_t a_lo[4], a_hi[4];
        unpack_block<Q>(w, b, a_lo, a_hi);
        const float2 sc = block_scales<Q>(w, b);
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            if (g < ngroups) {
                uint4 bf = make_uint4(0u, 0u, 0u, 0u);
                if (bptr[g] != nullptr) bf = ldg_cached(bptr[g] + b * 4);
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

// Split 4+4 f32 values of a block (v[4t..4t+3] and v[16+4t..16+4t+3]) into the
// activation fragment of moe_internal.cuh. hl = 0: high parts, 1: low parts.
// bf16_mode: split into bf16 pairs instead (BF16 weights use the bf16 MMA).
__device__ __forceinline__ uint32_t pack_split(float a, float b, int hl, bool bf16_mode) {
    if (!bf16_mode) {
        __half ha = __float2half_rn(a), hb = __float2half_rn(b);
        if (hl) {
            ha = __float2half_rn(a - __half2float(ha));
            hb = __float2half_rn(b - __half2float(hb));
        }
        return (uint32_t)__half_as_ushort(ha) | ((uint32_t)__half_as_ushort(hb) << 16);
    } else {
        __nv_bfloat16 ha = __float2bfloat16_rn(a), hb = __float2bfloat16_rn(b);
        if (hl) {
            ha = __float2bfloat16_rn(a - __bfloat162float(ha));
            hb = __float2bfloat16_rn(b - __bfloat162float(hb));
        }
        return (uint32_t)__bfloat16_as_ushort(ha) | ((uint32_t)__bfloat16_as_ushort(hb) << 16);
    }
}

__device__ __forceinline__ uint4 make_act_frag(const float4 lo4, const float4 hi4, int hl, bool bf16_mode) {
    uint4 r;
    r.x = pack_split(lo4.x, lo4.z, hl, bf16_mode);
    r.y = pack_split(lo4.y, lo4.w, hl, bf16_mode);
    r.z = pack_split(hi4.x, hi4.z, hl, bf16_mode);
    r.w = pack_split(hi4.y, hi4.w, hl, bf16_mode);
    return r;
}

}  // namespace lumen
