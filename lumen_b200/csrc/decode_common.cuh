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
