// Router logits of a multi-token batch on the 5th-generation tensor cores:
//   logit[t, e] = sum_j W_r[e, j] * x[t, j]        (moe_router_logits_batched,
//                                                   cuda/shaders/moe_grouped.cu:79; CPU: cuda/moe.rs:6456-6463)
// with f32-grade accuracy from 16-bit operands: W_r and x are each split into a high and a
// low f16 part (w = w_hi + w_lo to ~2^-22 relative) and the three products w_hi x_hi +
// w_lo x_hi + w_hi x_lo accumulate in ONE f32 accumulator in TMEM (the dropped w_lo x_lo term is
// ~2^-22 relative). The x_lo product is skipped for a batch whose low parts are all zero
// (bf16 activations).
//
// Formulation: the router weight is the M operand (128 expert rows per tile, E <= 256 ->
// one or two row tiles), tokens are the N columns (128 per tile), and the contraction is cut
// into `ksplit` ranges so that a few thousand tokens still fill the machine: CTA (token tile,
// row tile, k range) writes its partial logits, and the top-k kernel adds the ksplit partials
// in a fixed order (deterministic, no atomics). Everything is fed by TMA: the f16 planes of
// W_r are built once per layer, those of x by a pre-pass over the batch.
//
//   thread 0 of warp 0   TMA producer (4 boxes of 64 inputs per stage: W_hi, W_lo, x_hi, x_lo)
//   thread 0 of warp 1   tcgen05.mma issue, tcgen05.commit frees the stages
//   warps 2..5           epilogue: tcgen05.ld, coalesced f32 stores (lane = expert)
// All mbarrier waits are bounded; on expiry the kernel raises the context's status word,
// frees its TMEM and returns.
#include "tc_common.cuh"

namespace lumen {

namespace rtc {

using namespace tc;

constexpr int STAGES = 3;
constexpr int STAGE_BYTES = 4 * SUB_BYTES;  // W_hi | W_lo | x_hi | x_lo, each [128 rows x 64 k] f16
constexpr int THREADS = 6 * 32;
constexpr int BN = 128;  // tokens per tile

struct Args {
    CUtensorMap tmap_w;   // [2 E, H] f16: rows [0, E) high parts, [E, 2 E) low parts
    CUtensorMap tmap_x;   // [2 T, H] f16: rows [0, T) high parts, [T, 2 T) low parts
    float* part;          // [ksplit][T][E] partial logits
    const int32_t* any_lo;  // non-zero when some low part of x is non-zero
    int32_t* status;
    int32_t* status_host;
    uint64_t wait_limit_ns;
    int T, E, H, ksplit, m_tiles;
};

__global__ void __launch_bounds__(THREADS, 1)
router_logits_tc_kernel(const __grid_constant__ Args a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ uint32_t abort_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t stage0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const AbortCtl abort_flag{&abort_s, a.wait_limit_ns};

    // tile of this CTA
    int idx = blockIdx.x;
    const int ks = idx % a.ksplit;
    idx /= a.ksplit;
    const int mt = idx % a.m_tiles;
    const int tt = idx / a.m_tiles;
    const int t0 = tt * BN, e0 = mt * 128;
    const int kh_per = (a.H / 64) / a.ksplit;  // 64-input stages of this CTA's k range
    const int kh0 = ks * kh_per;
    grid_dep_sync();  // (the planes of x and the flag come from the split kernel before this one)
    const bool use_lo = (*a.any_lo != 0);

    if (tid == 0) {
        abort_s = 0u;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&acc_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                     "r"((uint32_t)BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            for (int n = 0; ok && n < kh_per; ++n) {
                const int s = n % STAGES, ph = (n / STAGES) & 1;
                ok = mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag);
                if (!ok) break;
                const uint32_t bar = smem_u32(&full_bar[s]);
                const uint32_t base = stage0 + s * STAGE_BYTES;
                const int k = (kh0 + n) * 64;
                mbar_expect_tx(bar, (use_lo ? 4 : 3) * SUB_BYTES);
                tma_load_2d(base + 0 * SUB_BYTES, &a.tmap_w, k, e0, bar);
                tma_load_2d(base + 1 * SUB_BYTES, &a.tmap_w, k, a.E + e0, bar);
                tma_load_2d(base + 2 * SUB_BYTES, &a.tmap_x, k, t0, bar);
                if (use_lo) tma_load_2d(base + 3 * SUB_BYTES, &a.tmap_x, k, a.T + t0, bar);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(BN, false);
            bool ok = true;
            for (int n = 0; ok && n < kh_per; ++n) {
                const int s = n % STAGES, ph = (n / STAGES) & 1;
                ok = mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t base = stage0 + s * STAGE_BYTES;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint64_t whi = make_desc(base + 0 * SUB_BYTES + j * 32);
                    const uint64_t wlo = make_desc(base + 1 * SUB_BYTES + j * 32);
                    const uint64_t xhi = make_desc(base + 2 * SUB_BYTES + j * 32);
                    umma(tmem_base, whi, xhi, idesc, (n > 0 || j > 0) ? 1u : 0u);
                    umma(tmem_base, wlo, xhi, idesc, 1u);
                    if (use_lo) umma(tmem_base, whi, make_desc(base + 3 * SUB_BYTES + j * 32), idesc, 1u);
                }
                umma_commit(smem_u32(&empty_bar[s]));
            }
            if (ok) umma_commit(smem_u32(&acc_bar));
        }
        __syncwarp();
    } else {
        // epilogue: warp w reads TMEM lanes 32 * (w % 4) ..; lane = expert row of the tile
        const int q = warp & 3;
        const int e = e0 + q * 32 + lane;
        if (mbar_wait(smem_u32(&acc_bar), 0, abort_flag)) {
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
            float* dst = a.part + ((size_t)ks * a.T + t0) * a.E + e;
            for (int n0 = 0; n0 < BN && t0 + n0 < a.T; n0 += 16) {
                uint32_t v[16];
                tmem_ld16(taddr + n0, v);
                tmem_ld_wait();
                if (e < a.E) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (t0 + n0 + j < a.T) dst[(size_t)(n0 + j) * a.E] = __uint_as_float(v[j]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
    if (tid == 0 && abort_s) raise_status(a.status, a.status_host, 4);  // LUMEN_MOE_TIMEOUT
}

// x [T, H] (f32 or bf16) -> f16 planes [2][T][H]: high part, low part; *any_lo |= (some low part != 0)
template <typename XT>
__global__ void __launch_bounds__(256)
split_x16_kernel(const XT* __restrict__ x, size_t n8, size_t plane, __half* __restrict__ out, int32_t* any_lo) {
    grid_dep_sync();
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    unsigned nz = 0u;
    if (i < n8) {
        float f[8];
        if (sizeof(XT) == 4) {
            const float4 p = reinterpret_cast<const float4*>(x)[2 * i], q = reinterpret_cast<const float4*>(x)[2 * i + 1];
            f[0] = p.x; f[1] = p.y; f[2] = p.z; f[3] = p.w;
            f[4] = q.x; f[5] = q.y; f[6] = q.z; f[7] = q.w;
        } else {
            const uint4 v = reinterpret_cast<const uint4*>(x)[i];
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[2 * j] = __uint_as_float(u[j] << 16);
                f[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
            }
        }
        __align__(16) __half hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            hi[j] = __float2half_rn(f[j]);
            lo[j] = __float2half_rn(f[j] - __half2float(hi[j]));
            nz |= (unsigned)(__half_as_ushort(lo[j]) & 0x7fffu);
        }
        reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<const uint4*>(hi);
        reinterpret_cast<uint4*>(out + plane)[i] = *reinterpret_cast<const uint4*>(lo);
    }
    if (__any_sync(0xffffffffu, nz != 0u) && (threadIdx.x & 31) == 0) atomicOr(any_lo, 1);
}

}  // namespace rtc

// W_r [E, H] f32 -> f16 planes [2][E][H] (high, low): once per layer
__global__ void split_router_w16_kernel(const float* __restrict__ w, __half* __restrict__ w16, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = w[i];
    const __half hi = __float2half_rn(v);
    w16[i] = hi;
    w16[n + i] = __float2half_rn(v - __half2float(hi));
}

cudaError_t launch_split_router_w16(const float* w, __half* w16, int E, int H, cudaStream_t st) {
    const size_t n = (size_t)E * H;
    count_launch();
    split_router_w16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(w, w16, n);
    return cudaGetLastError();
}

// k ranges per tile: a function of the shape only, never of the batch size, so that a token's
// logits (the order in which its partial sums are added) do not depend on how many tokens it is
// routed with: an expert-parallel rank routing its shard must get the bits one GPU gets for the
// whole batch. Four ranges of whole 64-input stages when H allows (a few thousand tokens then
// fill the machine), else two, else one.
int router_tc_ksplit(int T, int E, int H, int sms) {
    (void)T;
    (void)E;
    (void)sms;
    const int stages = H / 64;
    return (stages % 4 == 0) ? 4 : (stages % 2 == 0) ? 2 : 1;
}

bool router_tc_applicable(int T, int E, int H, const void* x) {
    return H % 64 == 0 && E >= 1 && E <= 256 && T >= 1 && reinterpret_cast<uintptr_t>(x) % 16 == 0;
}

// logits partials of the whole batch; x16 / any_lo / part are scratch of the context
cudaError_t launch_router_logits_tc(const void* x, int act_dtype, const __half* w16, int T, int E, int H, int ksplit,
                                    __half* x16, int32_t* any_lo, float* part, int32_t* status, int32_t* status_host,
                                    unsigned wait_limit_us, cudaStream_t st) {
    const size_t n8 = (size_t)T * H / 8, plane = (size_t)T * H;
    cudaError_t e = cudaMemsetAsync(any_lo, 0, sizeof(int32_t), st);
    if (e != cudaSuccess) return e;
    count_launch(2);
    const dim3 sgrid((unsigned)((n8 + 255) / 256));
    e = (act_dtype == 0)
            ? launch_dep(rtc::split_x16_kernel<float>, sgrid, dim3(256), 0, st, (const float*)x, n8, plane, x16, any_lo)
            : launch_dep(rtc::split_x16_kernel<__nv_bfloat16>, sgrid, dim3(256), 0, st, (const __nv_bfloat16*)x, n8, plane, x16,
                         any_lo);
    if (e != cudaSuccess) return e;
    rtc::Args a{};
    e = make_tmap_f16(w16, (uint64_t)2 * E, (uint64_t)H, 128, &a.tmap_w);
    if (e != cudaSuccess) return e;
    e = make_tmap_f16(x16, (uint64_t)2 * T, (uint64_t)H, 128, &a.tmap_x);
    if (e != cudaSuccess) return e;
    a.part = part;
    a.any_lo = any_lo;
    a.status = status;
    a.status_host = status_host;
    a.wait_limit_ns = wait_limit_us ? (uint64_t)wait_limit_us * 1000ull : tc::WAIT_LIMIT_NS;
    a.T = T;
    a.E = E;
    a.H = H;
    a.ksplit = ksplit;
    a.m_tiles = (E + 127) / 128;
    const int smem = rtc::STAGES * rtc::STAGE_BYTES + 1024;
    static SmemOptIn optin;
    e = ensure_dyn_smem(rtc::router_logits_tc_kernel, (size_t)smem, optin);
    if (e != cudaSuccess) return e;
    const int grid = ((T + rtc::BN - 1) / rtc::BN) * a.m_tiles * ksplit;
    return launch_dep(rtc::router_logits_tc_kernel, dim3(grid), dim3(rtc::THREADS), (size_t)smem, st, a);
}

}  // namespace lumen
