// Prefill grouped expert products on the 5th-generation tensor cores (tcgen05,
// accumulators in TMEM). Replaces the reference's tiled prefill kernels
// (moe_grouped_gate_up_swiglu_q4_0_tiled_f32act / moe_grouped_down_q4_0_tiled_f32act,
// cuda/shaders/moe_grouped.cu:1202-1510; the Q8_0 dp4a / mma.sync variants :566-1170,
// :2183-2598; the BF16 variants :1523-1760).
//
// Formulation. Gate/up + SwiGLU ("weights are the M operand"): for a tile of up to 256
// compact columns of one expert,  D_g[128 gate rows, N] += G[128, k] X[N, k]^T  and the
// same for the up rows, two tcgen05.mma of shape M=128 x N(16..256) x K=16 per 16 inputs
// sharing the activation operand; N follows the ragged per-expert column counts
// (Zipf-skewed loads) without padding M. Down ("tokens are the M operand"): for up to 128
// columns,  D[128 tokens, 256 output rows] += S[128, k] W[256, k]^T, one MMA per 16 inputs
// whose N operand is the stage's two adjacent 128-row weight tiles, so that an epilogue
// thread owns one token and stores 32 bytes at a time; a tile of up to 256 columns is two
// such products against the same weight stage, into the two accumulator sets.
//
// One CTA per SM, persistent over a device-built tile list, warp-specialised (27 warps):
//   warps 0-7   epilogue: tcgen05.ld of the accumulators, SwiGLU (gate/up), f16 stores
//               (into another rank's return buffer for an expert-parallel down product)
//   warps 8-23  weight producers, one 16-row tile each per 128-input group: 128-bit loads of
//               the repacked quant tiles (the next group prefetched in registers), dequantise
//               to f16 (scale folded in) in registers, store into the 128-byte-swizzled
//               K-major operand tile in shared memory. When the weights are plain f16
//               matrices copied by TMA (BF16 layers; LUMEN_MOE_FLAG_PREFILL_F16_WEIGHTS) they
//               share the gate/up epilogue instead
//   warp 24     one thread feeds the activation operand (and TMA-fed weights) with
//               cp.async.bulk.tensor.2d boxes of 64 inputs x 128 rows
//   warp 25     one elected thread issues tcgen05.mma / tcgen05.commit
//   warp 26     one thread hands out the tiles: the CTA's first tile is its index, every further
//               one is claimed from a device-wide counter while the tile before it is being
//               multiplied, and reaches the roles through a small ring of descriptors
// Stages are handed over with mbarriers; every wait is bounded (on expiry the
// kernel raises a status word, drains and frees its TMEM instead of hanging).
//
// Inputs are 16-bit: activations pre-converted to f16, gathered into compact-column order
// and pre-permuted within each 32-block to the order the dequantiser emits
// (gather_permute_x16_kernel; natural order for TMA-fed weights); the SwiGLU output is
// written in the same order so the down product reads it back without any shuffle.
#include "mma_frag.cuh"
#include "tc_common.cuh"
#include <cstdlib>

namespace lumen {

namespace tc {

constexpr int EPI_WARPS = 8, A_WARPS = 16, B_WARPS = 1;  // B: one thread drives the TMA
constexpr int A_WARP0 = EPI_WARPS, B_WARP0 = A_WARP0 + A_WARPS, MMA_WARP = B_WARP0 + B_WARPS;
constexpr int SCHED_WARP = MMA_WARP + 1;  // one thread hands out the tiles
constexpr int THREADS = (SCHED_WARP + 1) * 32;
constexpr int SCHED_RING = 4;             // tile descriptors in flight between the scheduler and the roles

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// Position of element e (0..31) of a block in the permuted 16-bit layout:
// chunk t = (e mod 16) / 4, slot order (4t, 4t+2, 16+4t, 16+4t+2, 4t+1, 4t+3, 16+4t+1, 16+4t+3).
__host__ __device__ __forceinline__ int perm_pos(int e) {
    const int hi = e >> 4, r = e & 15, t = r >> 2, m = r & 3;
    const int slot = ((m & 1) ? 4 : 0) + (hi ? 2 : 0) + ((m >> 1) & 1);
    return t * 8 + slot;
}

struct Args {
    CUtensorMap tmap;            // activation operand [rows, kdim] f16, box 64 x 128, SWIZZLE_128B (first: 64-byte aligned)
    CUtensorMap tmap_a;          // ATMA form: the experts' plain f16 matrices as one 2-D array [E * a_rows_exp, kdim]
    int a_rows_exp;              // rows per expert there: 2 I (gate rows then up rows) or H (down)
    int a_row1;                  // second operand's rows relative to the first: I (up) or 128 (next row tile of down)
    LayerDev L;
    const int32_t* col_src_tok;  // unused by the GEMM (rows are pre-gathered); kept for diagnostics
    const int4* tiles;
    int32_t* n_tiles;            // [0..1] tiles of the gate/up and the down list, [2..3] the kernels' tile counters (zero at launch)
    const void* b_src;      // 16-bit activations [rows, kdim], permuted order
    __half* out16;          // gate/up: S16 [C, I] permuted order; down: D16 [C, H] natural order
    int32_t* status;
    int32_t* status_host;   // mapped pinned copy of the status word for the host (null = none)
    uint64_t wait_limit_ns; // limit of every mbarrier wait
    int debug_extra_tx;     // test hook: the first stage's barrier expects this many bytes too many
    int kdim;               // H (gate/up) or I (down)
    int out_ld;             // I or H
    const int32_t* out_row_map;  // down mode: output row of compact column c (null = c itself)
    TcPeerOut peer;              // down mode, expert parallel: output rows go to other ranks' buffers (ret_map null = off)
};

// Dequantise one lane's share of half a weight tile (16 rows x 64 k: blocks
// 2*sub and 2*sub+1) into the operand tile: 4 chunks of 16 bytes (rows g, g+8).
//
// Lanes with odd g handle the second block of the pair first: the eight lanes of a quarter
// warp then hit eight different 16-byte chunk positions (rows are 128 bytes apart, i.e. a
// whole bank cycle) and the 128-bit stores are conflict-free. The choice is made on the raw
// words (two selects per block for Q4_0, four for Q8_0), not on the sixteen unpacked ones.
template <int Q>
__device__ __forceinline__ void dequant_store(const WTile<Q>& w, int sub, uint32_t a_base, int rtl, int lane) {
    if constexpr (Q == BF16) return;  // BF16 layers feed this path from plain f16 matrices (ATMA): no producers
    const int g = lane >> 2, t = lane & 3;
    const bool odd = (g & 1) != 0;
    const int r0 = rtl * 16 + g, r1 = r0 + 8;
    const uint32_t s_g = (sub == 0) ? w.s.x : w.s.y;   // f16 scales of blocks 2 sub, 2 sub + 1: row g
    const uint32_t s_g8 = (sub == 0) ? w.s.z : w.s.w;  // row g + 8
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const bool second = (pass == 1) != odd;  // which block of the pair this lane handles in this pass
        uint32_t lo[4], hi[4];
        if (Q == Q4_0) {
            const uint4 v = w.q[sub];
            const uint32_t wg = second ? v.z : v.x;   // row g
            const uint32_t wg8 = second ? v.w : v.y;  // row g+8
            const uint32_t sub_lo = 0x64086408u;      // 1032 = 1024 + 8
            const uint32_t sub_hi = 0x54805480u;      // 72   = 64 + 8
            lo[0] = hsub2_u32(lop_and_or(wg, 0x000F000Fu, 0x64006400u), sub_lo);
            lo[1] = hsub2_u32(lop_and_or(wg8, 0x000F000Fu, 0x64006400u), sub_lo);
            lo[2] = hsub2_u32(lop_and_or(wg >> 8, 0x000F000Fu, 0x64006400u), sub_lo);
            lo[3] = hsub2_u32(lop_and_or(wg8 >> 8, 0x000F000Fu, 0x64006400u), sub_lo);
            hi[0] = hsub2_u32(lop_and_or(wg, 0x00F000F0u, 0x54005400u), sub_hi);
            hi[1] = hsub2_u32(lop_and_or(wg8, 0x00F000F0u, 0x54005400u), sub_hi);
            hi[2] = hsub2_u32(lop_and_or(wg >> 8, 0x00F000F0u, 0x54005400u), sub_hi);
            hi[3] = hsub2_u32(lop_and_or(wg8 >> 8, 0x00F000F0u, 0x54005400u), sub_hi);
        } else {
            const uint4 va = w.q[(2 * sub) % QTraits<Q>::NQ], vb = w.q[(2 * sub + 1) % QTraits<Q>::NQ];
            // bytes biased by 128 -> unsigned; 0x64xx = 1024 + xx; subtract 1152.
            const uint32_t sb = 0x64806480u;
            const uint32_t x0 = (second ? vb.x : va.x) ^ 0x80808080u, x1 = (second ? vb.y : va.y) ^ 0x80808080u;
            const uint32_t y0 = (second ? vb.z : va.z) ^ 0x80808080u, y1 = (second ? vb.w : va.w) ^ 0x80808080u;
            lo[0] = hsub2_u32(prmt(x0, 0x64646464u, 0x4240u), sb);
            lo[1] = hsub2_u32(prmt(y0, 0x64646464u, 0x4240u), sb);
            lo[2] = hsub2_u32(prmt(x0, 0x64646464u, 0x4341u), sb);
            lo[3] = hsub2_u32(prmt(y0, 0x64646464u, 0x4341u), sb);
            hi[0] = hsub2_u32(prmt(x1, 0x64646464u, 0x4240u), sb);
            hi[1] = hsub2_u32(prmt(y1, 0x64646464u, 0x4240u), sb);
            hi[2] = hsub2_u32(prmt(x1, 0x64646464u, 0x4341u), sb);
            hi[3] = hsub2_u32(prmt(y1, 0x64646464u, 0x4341u), sb);
        }
        const uint32_t bsel = second ? 0x3232u : 0x1010u;  // the block's scale, in both halves
        const uint32_t sg2 = prmt(s_g, s_g, bsel);
        const uint32_t sg82 = prmt(s_g8, s_g8, bsel);
        const int c = (second ? 4 : 0) + t;
        sts128(a_base + r0 * 128 + ((c ^ (r0 & 7)) << 4), hmul2_u32(lo[0], sg2), hmul2_u32(hi[0], sg2),
               hmul2_u32(lo[2], sg2), hmul2_u32(hi[2], sg2));
        sts128(a_base + r1 * 128 + ((c ^ (r1 & 7)) << 4), hmul2_u32(lo[1], sg82), hmul2_u32(hi[1], sg82),
               hmul2_u32(lo[3], sg82), hmul2_u32(hi[3], sg82));
    }
}

// ATMA: the weight operands are not dequantised here but copied by TMA from plain f16 matrices
// (BF16 layers; Q4_0 / Q8_0 layers of a context created with LUMEN_MOE_FLAG_PREFILL_F16_WEIGHTS): the
// producer warps have nothing to dequantise and every operand is in the natural input order.
//
// Operand stages. The dequantising producers prefetch the next 128-input group of quantised tiles
// into registers while they work on the current one: with sixteen producer warps of one tile
// each that is 3 (Q4_0) or 5 (Q8_0) uint4 per lane in flight, inside the 72 registers a thread has.
// (With eight warps of two tiles the Q8_0 prefetch spilled and a cp.async ring in shared memory
// replaced it, at the price of an operand stage; the ring is gone again: 0.540 -> 0.50 ms per
// 4096-token Q8_0 call.)
// STG (expert-parallel down product): an operand stage is given up for a staging tile from which
// the output rows leave as 256-byte bulk copies (see the epilogue).
template <int Q, int BN, bool ATMA, bool STG = false>
struct StagesOf {
    static constexpr int value = ((BN == 128) ? 4 : 3) - (STG ? 1 : 0);
};
constexpr int STG_ROW_BYTES = 256 + 16;                 // 128 f16 outputs of one token + padding (bank spread)
constexpr int STG_BYTES = 2 * 128 * STG_ROW_BYTES;      // two warp groups x 128 tokens

// Debug aid (compile with -DLUMEN_TC_TRACE): per CTA, the cycles the MMA thread and the first
// producer warp spend in their waits, read back with lumen_debug_tc_trace.
#ifdef LUMEN_TC_TRACE
__device__ unsigned long long g_tc_trace[2][160][8];
#define TRACE_WAIT(acc, expr) ([&] { const long long t0_ = clock64(); const bool r_ = (expr); (acc) += clock64() - t0_; return r_; }())
#define TRACE_PUT(slot, v) g_tc_trace[MODE][blockIdx.x][slot] = (unsigned long long)(v)
#else
#define TRACE_WAIT(acc, expr) (expr)
#define TRACE_PUT(slot, v)
#endif

template <int Q, int MODE, int BN, bool ATMA = false, bool STG = false>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_tc_kernel(const __grid_constant__ Args a) {
    static_assert(!STG || (MODE == 1 && BN == 128), "the staged epilogue belongs to the 128-token down product");
    // Two 128-row weight operands share every activation stage (gate and up rows of the
    // same I range; two adjacent row tiles of the down matrix): the activation operand,
    // which comes from L2 at 2 bytes per element, is then read at half the rate.
    // 256-column tiles (gate/up once the experts average more than 128 columns): each dequantised
    // weight tile serves 256 columns, and with K = H the main loop is long; the two 256-column f32
    // accumulators of a full tile fill TMEM (512 columns), so its epilogue is not overlapped with
    // the next tile's MMAs (its producers do run ahead).
    // 128-column tiles (down: K = I is short, 12 stages at I = 768, so the epilogue weighs
    // more; gate/up of small batches: fewer empty columns): TWO accumulator sets, the
    // epilogue of tile i runs under the MMAs of tile i+1.
    constexpr int NA = 2;
    // BN: columns per tile
    // Accumulator sets in TMEM (512 columns), always two.
    // Down: a set is 256 columns (the output rows of an m-tile) for 128 tokens; a 256-token tile of
    // the BN = 256 form takes both at once (its two token halves, one weight stage serving both),
    // a tile of up to 128 tokens takes one, and the epilogue works through the halves one by one.
    // Gate/up, BN = 128: a set is the gate and the up accumulator side by side (2 x 128 columns).
    // Gate/up, BN = 256: the gate accumulator lives in TMEM columns 0..255 and the up accumulator in
    // 256..511; a tile of up to 128 columns (the last chunk of most experts under skewed loads) takes
    // one HALF of each (set s: columns 128 s.. of both), so two such tiles are in flight and the
    // epilogue of one runs under the MMAs of the next; a wider tile takes both sets at once.
    constexpr int NACC = 2;
    constexpr bool WIDE_GU = (MODE == 0 && BN == 256);
    constexpr int ACC_COLS = WIDE_GU ? 128 : 256;  // TMEM columns from one set to the next
    // While a wide gate/up tile holds both sets the tensor pipe idles during its epilogue. When the weights come
    // by TMA the producer warps have nothing else to do and share the epilogue. (Dequantising
    // producers doing the same was measured slower, 0.52 -> 0.60 ms per 4096-token Q4_0 call: their
    // own work is what those kernels wait for; the same again for the 256-token down tiles, whose
    // epilogue between two such tiles is exposed too: Q4_0 0.463 -> 0.498 ms, Q8_0 and BF16 unchanged.)
    constexpr bool HELP = WIDE_GU && ATMA;
    constexpr int STAGES = StagesOf<Q, BN, ATMA, STG>::value;  // one stage = 64 inputs (one swizzle atom in K)
    constexpr int STAGE_BYTES = NA * SUB_BYTES + BN * 128;  // A operands then B
    constexpr int TMEM_COLS = 512;

    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full_bar[NACC], acc_empty_bar[NACC];
    __shared__ uint32_t tmem_base_s;
    __shared__ uint32_t abort_s;
    // Tiles are handed out dynamically: the CTA's first tile is blockIdx.x, every further one the next
    // of the list not yet taken by any CTA (a device-wide counter). One thread claims a tile while the
    // MMA thread is still inside the tile before it, and passes the descriptor to the roles through
    // this ring. (With tiles dealt round-robin the slowest CTA of a Zipf-loaded 4096-token call ran
    // 11 % longer than the median one in gate/up and 13 % in down.)
    __shared__ int4 sched_tile_s[SCHED_RING];
    __shared__ uint64_t sched_full_bar[SCHED_RING], sched_empty_bar[SCHED_RING], sched_go_bar;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t stage0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const AbortCtl abort_flag{&abort_s, a.wait_limit_ns};

    if (tid == 0) {
        abort_s = 0u;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), ATMA ? 1 : A_WARPS * 32 + 1);  // weight producers + the TMA thread's expect_tx arrive
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < NACC; ++b) {
            mbar_init(smem_u32(&acc_full_bar[b]), 1);
            mbar_init(smem_u32(&acc_empty_bar[b]), (HELP ? EPI_WARPS + A_WARPS : EPI_WARPS) * 32);
        }
        // readers of a descriptor: epilogue warps, the producer warps when they dequantise or share the
        // epilogue, the TMA thread and the MMA thread
        constexpr int SCHED_READERS = EPI_WARPS * 32 + ((!ATMA || HELP) ? A_WARPS * 32 : 0) + 2;
        for (int s = 0; s < SCHED_RING; ++s) {
            mbar_init(smem_u32(&sched_full_bar[s]), 1);
            mbar_init(smem_u32(&sched_empty_bar[s]), SCHED_READERS);
        }
        mbar_init(smem_u32(&sched_go_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    // (barriers and TMEM are set up above while the kernel before this one may still be running;
    // everything it wrote, the tile list first of all, is read from here on)
    grid_dep_sync();
    const int ntiles = a.n_tiles[MODE];
    const int kgs = a.kdim >> 7;   // 128-input groups (weight tile granularity)
    const int khs = kgs * 2;       // 64-input pipeline stages per tile
    // every operand is f16 here: BF16 weights are converted exactly (see dequant_store)
    const bool bf16_mode = false;
    // The n-th tile of this CTA (n counted by the calling thread): false when the list is exhausted
    // or the kernel gives up. The descriptor is copied and its ring slot released at once.
    auto next_tile = [&](int& n, int4& tile) -> bool {
        const int slot = n % SCHED_RING;
        if (!mbar_wait(smem_u32(&sched_full_bar[slot]), (n / SCHED_RING) & 1, abort_flag)) return false;
        tile = sched_tile_s[slot];
        mbar_arrive(smem_u32(&sched_empty_bar[slot]));
        ++n;
        return tile.z >= 0;
    };
    // stage of a tile at which the MMA thread lets the scheduler claim the CTA's next tile: late, so
    // that the last tiles of the list go to the CTAs that are free first, but early enough for the
    // claim (an atomic and a load, ~2 us) to be back when the producers reach the tile's last group
    // (the producers take the next descriptor before they fill the last two stages of a tile, so the
    // signal has to come before the MMA thread needs those: go_kh <= khs - 2)
    const int go_kh = (khs >= 24) ? khs / 2 - 4 : (khs >= 4 ? 1 : 0);

    // Epilogue of one tile by one warp: the warp's TMEM lanes are 32 (warp % 4).. (hardware rule);
    // of the tile's 16-column TMEM chunks it takes those with chunk % nparts == part.
    auto epilogue_part = [&](const int4& tile, int ab, int h, int part, int nparts) {
        const int row = (warp & 3) * 32 + lane;
        const int ncols = tile.z;
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + ab * ACC_COLS;
        if (MODE == 1) {
            // Down product: the tile's columns (tokens) are the TMEM lanes and the 256 output rows
            // of the m-tile the TMEM columns, so a thread owns one token and reads 16 consecutive
            // output rows per load: its stores are 32 bytes wide and each token's 512 bytes are
            // contiguous (a whole NVLink packet when the row lives on another rank).
            {
                const int tcol = h * 128 + row;  // token column of the tile (h: its half of a 256-token tile)
                bool live = tcol < ncols;
                __half* dst = a.out16;
                if (live) {
                    int orow_idx = tile.y + tcol;
                    if (a.out_row_map != nullptr) orow_idx = a.out_row_map[orow_idx];
                    dst = a.out16 + (size_t)orow_idx * a.out_ld;
                    if (a.peer.ret_map != nullptr) {
                        // plain stores into the return buffer of the rank the row came from
                        const int m = a.peer.ret_map[orow_idx];
                        const int pr = (m >> 24) & 0xff, prow = m & 0xffffff;
                        live = pr < a.peer.world && prow < a.peer.rows_cap;  // never leave the buffers
                        if (live) dst = a.peer.base[pr] + (size_t)prow * a.out_ld;
                    }
                    dst += (size_t)tile.w * 256;
                }
                // (every lane takes part in the loads: tcgen05.ld is a warp-wide instruction)
                // a contiguous share of the 256 output rows per warp group
                const int ow = 256 / nparts;
                if constexpr (STG) {
                    // Rows that leave for another GPU: a lane's direct stores are 32-byte pieces of 32
                    // different rows per warp instruction, which cross NVLink as small packets. Here the
                    // lane collects its token's 128 outputs (256 bytes) in shared memory and sends them
                    // as ONE asynchronous bulk copy. Row pitch 272 bytes: the eight lanes of a quarter
                    // warp hit eight different 16-byte bank groups.
                    const uint32_t srow = stage0 + STAGES * STAGE_BYTES + (uint32_t)(part * 128 + row) * STG_ROW_BYTES;
                    // the previous tile's copy of this row must have read its bytes before they are overwritten
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
#pragma unroll 2
                    for (int n0 = 0; n0 < 128; n0 += 16) {
                        uint32_t v[16];
                        tmem_ld16(taddr + part * 128 + n0, v);
                        tmem_ld_wait();
                        uint32_t hh[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const __half2 pr2 = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                            hh[j] = *reinterpret_cast<const uint32_t*>(&pr2);
                        }
                        sts128(srow + n0 * 2, hh[0], hh[1], hh[2], hh[3]);
                        sts128(srow + n0 * 2 + 16, hh[4], hh[5], hh[6], hh[7]);
                    }
                    fence_proxy_async();  // the lane's own writes, before the async proxy reads them
                    if (live)
                        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 256;" ::"l"(
                                         __cvta_generic_to_global(dst + part * 128)),
                                     "r"(srow)
                                     : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                if constexpr (!STG) {
#pragma unroll 2
                for (int n0 = part * ow; n0 < (part + 1) * ow; n0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(taddr + n0, v);
                    tmem_ld_wait();
                    if (live) {
                        uint32_t hh[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const __half2 pr2 = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                            hh[j] = *reinterpret_cast<const uint32_t*>(&pr2);
                        }
                        st_global_v8(dst + n0, hh);  // 16 outputs = one 32-byte sector of the token's row
                    }
                }
                }
            }
        } else {
            // Gate/up: a thread owns one row of I (its TMEM lane) and walks the token columns
            const int irow = tile.w * 128 + row;  // SwiGLU output is stored in the order the down product reads it
            const size_t off0 = ATMA ? (size_t)irow : (size_t)(irow & ~31) + perm_pos(irow & 31);
            // 8-column pieces of this warp's 16-column chunks, the TMEM loads of the next piece issued
            // before the current one is worked on
            auto piece_col = [&](int p) { return part * 16 + (p >> 1) * nparts * 16 + (p & 1) * 8; };
            auto work = [&](int col, const uint32_t (&g)[8], const uint32_t (&u)[8]) {
                __half* dst = a.out16 + (size_t)(tile.y + col) * a.out_ld + off0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (col + j < ncols) {
                        const float gt = __uint_as_float(g[j]);
                        // SwiGLU (cuda/shaders/moe_expert.cu:47-50) with the fast exp and divide: their
                        // error (~2^-21) is far below the f16 rounding of the result that follows
                        dst[(size_t)j * a.out_ld] =
                            __float2half_rn(__fdividef(gt, 1.0f + __expf(-gt)) * __uint_as_float(u[j]));
                    }
                }
            };
            uint32_t g0[8], u0[8], g1[8], u1[8];
            int p = 0;
            if (piece_col(0) < ncols) {
                tmem_ld8(taddr + piece_col(0), g0);
                tmem_ld8(taddr + BN + piece_col(0), u0);
            }
            while (piece_col(p) < ncols) {
                // (the loop condition is uniform over the warp: tcgen05.ld is a warp-wide instruction)
                tmem_ld_wait();
                tmem_ld_fence8(g0);
                tmem_ld_fence8(u0);
                const bool more1 = piece_col(p + 1) < ncols;
                if (more1) {
                    tmem_ld8(taddr + piece_col(p + 1), g1);
                    tmem_ld8(taddr + BN + piece_col(p + 1), u1);
                }
                work(piece_col(p), g0, u0);
                if (!more1) break;
                tmem_ld_wait();
                tmem_ld_fence8(g1);
                tmem_ld_fence8(u1);
                if (piece_col(p + 2) < ncols) {
                    tmem_ld8(taddr + piece_col(p + 2), g0);
                    tmem_ld8(taddr + BN + piece_col(p + 2), u0);
                }
                work(piece_col(p + 1), g1, u1);
                p += 2;
            }
        }
    };
    constexpr int EPI_PARTS = EPI_WARPS / 4 + (HELP ? A_WARPS / 4 : 0);  // groups of four warps sharing a tile's epilogue
    // A warp's share of one tile's epilogue. v: accumulator sets handed over so far (set v % NACC, used
    // v / NACC times before). A tile of more than 128 columns holds both sets: the down product works
    // through them one after the other (its two token halves), gate/up reads them as one tile.
    auto epilogue_tile = [&](const int4& tile, int& v, int part) -> bool {
        const int nsets = (tile.z > 128) ? 2 : 1;
        const int passes = (MODE == 1) ? nsets : 1, per_pass = (MODE == 1) ? 1 : nsets;
        for (int h = 0; h < passes; ++h) {
            for (int j = 0; j < per_pass; ++j)
                if (!mbar_wait(smem_u32(&acc_full_bar[(v + j) % NACC]), ((v + j) / NACC) & 1, abort_flag)) return false;
            tc_fence_after();
            epilogue_part(tile, per_pass == 2 ? 0 : v % NACC, h, part, EPI_PARTS);
            tc_fence_before();
            for (int j = 0; j < per_pass; ++j) mbar_arrive(smem_u32(&acc_empty_bar[(v + j) % NACC]));
            v += per_pass;
        }
        return true;
    };

    if (warp < EPI_WARPS) {
        // ------------------------------ epilogue ------------------------------
        int v = 0;  // accumulator sets handed over so far: set v % NACC, used v / NACC times before
        bool ok = true;
        int tn = 0;
        int4 tile;
        while (ok && next_tile(tn, tile)) ok = epilogue_tile(tile, v, warp >> 2);
        if constexpr (STG) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every row has been written
    } else if (warp < B_WARP0) {
        // --------------------------- weight producers --------------------------
        // Sixteen warps, one 16-row weight tile each per 128-input group: warps 0-7 the eight row
        // tiles of the stage's first operand, warps 8-15 those of the second.
        const int pw = warp - A_WARP0;
        const int op = pw >> 3, rtl = pw & 7;  // operand of the stage, 16-row tile within its 128 rows
        bool ok = true;
        int tn = 0;
        // quant words and scales of this warp's tile of 128-input group kg of a tile of the list
        auto tile_ptrs = [&](const int4& tile, int kg, const uint4*& qp, const uint4*& sp) {
            const int e = tile.x;
            int tidx;
            const uint4 *qb, *sb;
            if (MODE == 0) {
                // m-tile = 128 rows of I: operand 0 gate, operand 1 up
                qb = op ? a.L.up_q(e) : a.L.gate_q(e);
                sb = op ? a.L.up_s(e) : a.L.gate_s(e);
                tidx = (tile.w * 8 + rtl) * kgs + kg;
            } else {
                // m-tile = 256 rows of H: two adjacent 128-row tiles
                qb = a.L.down_q(e);
                sb = a.L.down_s(e);
                tidx = (tile.w * 16 + pw) * kgs + kg;
            }
            qp = qb + ((size_t)tidx * QTraits<Q>::NQ) * 32 + lane;
            sp = sb + (size_t)tidx * 8;
        };
        auto warp_wait = [&](uint32_t bar, uint32_t parity) -> bool { return mbar_wait(bar, parity, abort_flag); };
        auto warp_arrive = [&](uint32_t bar) {
            fence_proxy_async();
            mbar_arrive(bar);
        };
        if constexpr (!ATMA) {
            WTile<Q> cur, nxt;
            auto issue = [&](const int4& tile, int kg, WTile<Q>& dst) {
                const uint4 *qp, *sp;
                tile_ptrs(tile, kg, qp, sp);
    #pragma unroll
                for (int j = 0; j < QTraits<Q>::NQ; ++j) dst.q[j] = ldg_stream(qp + j * 32);
                if (Q != BF16) dst.s = ldg_stream(sp + (lane >> 2));
            };
            // The next tile's descriptor is taken before the last group of the current tile, so that
            // the first group of the next tile is in flight while the last one is dequantised.
            int4 tile_c, tile_n = make_int4(0, 0, -1, 0);
            bool have_c = next_tile(tn, tile_c), have_n = false;
            if (have_c) issue(tile_c, 0, cur);
            int it = 0, kg = 0;
            long long tr_w = 0;
            const long long tr_t0 = clock64();
            while (ok && have_c) {
                bool more = true;  // a group follows this one
                if (kg + 1 < kgs) {
                    issue(tile_c, kg + 1, nxt);
                } else {
                    have_n = next_tile(tn, tile_n);
                    if (have_n) issue(tile_n, 0, nxt);
                    more = have_n;
                }
    #pragma unroll
                for (int sub = 0; sub < 2; ++sub, ++it) {
                    const int s = it % STAGES, ph = (it / STAGES) & 1;
                    ok = ok && TRACE_WAIT(tr_w, warp_wait(smem_u32(&empty_bar[s]), ph ^ 1));
                    if (ok) {
                        dequant_store<Q>(cur, sub, stage0 + s * STAGE_BYTES + op * SUB_BYTES, rtl, lane);
                        warp_arrive(smem_u32(&full_bar[s]));
                    }
                }
                if (more) cur = nxt;
                if (++kg == kgs) {
                    kg = 0;
                    tile_c = tile_n;
                    have_c = have_n;
                    have_n = false;
                }
            }
            if (pw == 0 && lane == 0) {
                TRACE_PUT(0, tr_w);
                TRACE_PUT(1, clock64() - tr_t0);
            }
            (void)tr_w;
            (void)tr_t0;
        }
        if constexpr (HELP) {
            // TMA-fed weights, one accumulator set: nothing to dequantise, the warp takes a share of
            // every tile's epilogue instead
            int4 tile;
            int v = 0;
            while (ok && next_tile(tn, tile)) ok = epilogue_tile(tile, v, EPI_WARPS / 4 + (pw >> 2));
        }
        (void)warp_wait;
        (void)warp_arrive;
        (void)tile_ptrs;
    } else if (warp < MMA_WARP) {
        // ------------------------- activation producers ------------------------
        // One thread feeds the activation operand with TMA: per 64-input stage one or two
        // 128-row boxes of the compact (pre-gathered, pre-permuted) f16 activations land
        // in the SWIZZLE_128B layout the MMA descriptor expects; completion is counted in
        // bytes on the stage's full barrier.
        if (lane == 0) {
            const uint64_t tmap_addr = reinterpret_cast<uint64_t>(&a.tmap);
            const uint64_t tmap_a_addr = reinterpret_cast<uint64_t>(&a.tmap_a);
            int row0 = 0, nbox = 1, arow0 = 0;
            bool ok = true;
            int tn = 0;
            for (int n = 0; ok; ++n) {
                const int kh = n % khs;
                if (kh == 0) {
                    int4 tile;
                    if (!next_tile(tn, tile)) break;
                    row0 = tile.y;
                    nbox = (BN > 128 && tile.z > 128) ? 2 : 1;
                    arow0 = tile.x * a.a_rows_exp + tile.w * (MODE == 0 ? 128 : 256);
                }
                const int s = n % STAGES, ph = (n / STAGES) & 1;
                ok = mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag);
                if (!ok) break;
                const uint32_t bar = smem_u32(&full_bar[s]);
                const uint32_t bbase = stage0 + s * STAGE_BYTES + NA * SUB_BYTES;
                // (test hook: with debug_extra_tx the very first stage can never complete)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                             "r"((nbox + (ATMA ? NA : 0)) * SUB_BYTES + (n == 0 ? a.debug_extra_tx : 0))
                             : "memory");
                if (ATMA) {
#pragma unroll
                    for (int op = 0; op < NA; ++op)
                        asm volatile(
                            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                            "[%0], [%1, {%2, %3}], [%4];" ::"r"(stage0 + s * STAGE_BYTES + op * SUB_BYTES),
                            "l"(tmap_a_addr), "r"(kh * 64), "r"(arow0 + op * a.a_row1), "r"(bar)
                            : "memory");
                }
                for (int q = 0; q < nbox; ++q)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                        "[%0], [%1, {%2, %3}], [%4];" ::"r"(bbase + q * SUB_BYTES),
                        "l"(tmap_addr), "r"(kh * 64), "r"(row0 + q * 128), "r"(bar)
                        : "memory");
            }
        }
        __syncwarp();
    } else if (warp == MMA_WARP) {
        // -------------------------------- MMA ---------------------------------
        if (lane == 0) {
            int it = 0, tl = 0;
            bool ok = true;
            long long tr_wf = 0, tr_wa = 0;
            const long long tr_t0 = clock64();
            int v = 0;  // accumulator sets taken so far (see the epilogue)
            int tn = 0;
            int4 tile;
            for (; ok && next_tile(tn, tile); ++tl) {
                const int n16 = (tile.z + 15) & ~15;
                // down: D[128 tokens, 256 output rows] = X[128, k] W[256, k]^T, the two adjacent 128-row
                // weight operands of a stage forming one 256-row N operand; a tile of more than 128
                // tokens is two such products per 16 inputs, into two accumulator sets
                const uint32_t idesc = make_idesc(MODE == 1 ? 256 : n16, bf16_mode);
                const int nh = (tile.z > 128) ? 2 : 1;  // accumulator sets of the tile
                for (int h = 0; ok && h < nh; ++h) {
                    const int ab = (v + h) % NACC, use = (v + h) / NACC;
                    ok = TRACE_WAIT(tr_wa, mbar_wait(smem_u32(&acc_empty_bar[ab]), (use & 1) ^ 1, abort_flag));
                }
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc0 = tmem_base + (v % NACC) * ACC_COLS, acc1 = tmem_base + ((v + 1) % NACC) * ACC_COLS;
                for (int kh = 0; kh < khs; ++kh, ++it) {
                    const int s = it % STAGES, ph = (it / STAGES) & 1;
                    if (kh == go_kh) mbar_arrive(smem_u32(&sched_go_bar));  // the CTA's next tile may be claimed now
                    ok = TRACE_WAIT(tr_wf, mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sbase = stage0 + s * STAGE_BYTES;
                    const uint32_t bbase = sbase + NA * SUB_BYTES;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t bdesc = make_desc(bbase + j * 32);
                        const uint32_t acc = (kh > 0 || j > 0) ? 1u : 0u;
                        if (MODE == 1) {
                            const uint64_t wdesc = make_desc(sbase + j * 32);
                            umma(acc0, bdesc, wdesc, idesc, acc);
                            if (nh == 2) umma(acc1, make_desc(bbase + SUB_BYTES + j * 32), wdesc, idesc, acc);
                        } else {
#pragma unroll
                            for (int op = 0; op < NA; ++op) {
                                const uint64_t adesc = make_desc(sbase + op * SUB_BYTES + j * 32);
                                umma((nh == 2 ? tmem_base : acc0) + op * BN, adesc, bdesc, idesc, acc);
                            }
                        }
                    }
                    umma_commit(smem_u32(&empty_bar[s]));
                }
                if (!ok) break;
                for (int h = 0; h < nh; ++h) umma_commit(smem_u32(&acc_full_bar[(v + h) % NACC]));
                v += nh;
            }
            TRACE_PUT(2, tr_wf);
            TRACE_PUT(3, tr_wa);
            TRACE_PUT(4, clock64() - tr_t0);
            TRACE_PUT(5, tl);
            (void)tr_wf;
            (void)tr_wa;
            (void)tr_t0;
        }
        __syncwarp();
    } else {
        // ------------------------------ scheduler ------------------------------
        if (lane == 0) {
            for (int n = 0;; ++n) {
                const int slot = n % SCHED_RING;
                // tile n >= 1 is claimed once the MMA thread is far enough into tile n - 1 (the thread
                // cannot get two tiles ahead of this wait: tile n is not handed out before it)
                if (n > 0 && !mbar_wait(smem_u32(&sched_go_bar), (n - 1) & 1, abort_flag)) break;
                if (!mbar_wait(smem_u32(&sched_empty_bar[slot]), ((n / SCHED_RING) & 1) ^ 1, abort_flag)) break;
                const int t = (n == 0) ? (int)blockIdx.x : (int)gridDim.x + atomicAdd(a.n_tiles + 2 + MODE, 1);
                sched_tile_s[slot] = (t < ntiles) ? a.tiles[t] : make_int4(0, 0, -1, 0);  // columns < 0: no more tiles
                mbar_arrive(smem_u32(&sched_full_bar[slot]));
                if (t >= ntiles) break;
            }
        }
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
    if (tid == 0 && abort_s) raise_status(a.status, a.status_host, 4);  // LUMEN_MOE_TIMEOUT
}

// activations -> f16, gathered into compact-column order (row c = token
// col_src_tok[c]) and permuted within each 32-block: the grouped GEMM then reads
// plain 2-D boxes of it with TMA
template <typename XT, bool IS_F16 = false, bool NATURAL = false>
__global__ void __launch_bounds__(256)
gather_permute_x16_kernel(const XT* __restrict__ x, const int32_t* __restrict__ col_src_tok, int C, int H,
                          uint16_t* __restrict__ out) {
    grid_dep_sync();
    // one thread per output chunk of 8 values (16 bytes): chunk t of a 32-block holds inputs
    // (4t, 4t+2, 16+4t, 16+4t+2, 4t+1, 4t+3, 16+4t+1, 16+4t+3), i.e. perm_pos of two runs of four.
    // Four rows per step: their source rows are known first, then all eight loads of a thread are
    // in flight together (one row per CTA was a chain of dependent latencies: 43 us for 134 MB).
    auto to_h = [](XT v) -> uint16_t {
        if (sizeof(XT) == 4) return __half_as_ushort(__float2half_rn(*reinterpret_cast<const float*>(&v)));
        if (IS_F16) return *reinterpret_cast<const uint16_t*>(&v);
        return __half_as_ushort(__float2half_rn(__bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&v))));
    };
    struct __align__(4 * sizeof(XT)) Run { XT v[4]; };
    constexpr int R = 4;
    for (int c0 = blockIdx.x * R; c0 < C; c0 += gridDim.x * R) {
        int tok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) tok[r] = col_src_tok[min(c0 + r, C - 1)];
        for (int ch = threadIdx.x; ch < H / 8; ch += 256) {
            const int blk = ch >> 2, t = ch & 3;
            // NATURAL (TMA-fed weights): chunk ch holds inputs 8 ch .. 8 ch + 7 as they are
            const int oa = NATURAL ? ch * 8 : blk * 32 + 4 * t, ob = NATURAL ? ch * 8 + 4 : blk * 32 + 16 + 4 * t;
            Run a[R], b[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const XT* src = x + (size_t)tok[r] * H;
                a[r] = *reinterpret_cast<const Run*>(src + oa);
                b[r] = *reinterpret_cast<const Run*>(src + ob);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (c0 + r < C) {
                    __align__(16) uint16_t o[8];
                    if (NATURAL) {
                        o[0] = to_h(a[r].v[0]); o[1] = to_h(a[r].v[1]); o[2] = to_h(a[r].v[2]); o[3] = to_h(a[r].v[3]);
                        o[4] = to_h(b[r].v[0]); o[5] = to_h(b[r].v[1]); o[6] = to_h(b[r].v[2]); o[7] = to_h(b[r].v[3]);
                    } else {
                        o[0] = to_h(a[r].v[0]); o[1] = to_h(a[r].v[2]); o[2] = to_h(b[r].v[0]); o[3] = to_h(b[r].v[2]);
                        o[4] = to_h(a[r].v[1]); o[5] = to_h(a[r].v[3]); o[6] = to_h(b[r].v[1]); o[7] = to_h(b[r].v[3]);
                    }
                    *reinterpret_cast<uint4*>(out + (size_t)(c0 + r) * H + blk * 32 + t * 8) = *reinterpret_cast<const uint4*>(o);
                }
            }
        }
    }
}

}  // namespace tc

cudaError_t launch_gather_permute_x16(const void* x, int act_dtype, const int32_t* col_src_tok, int C, int H, void* out,
                                      cudaStream_t st, bool natural) {
    count_launch();
    if (C <= 0) return cudaSuccess;
    const int ggrid = (C + 3) / 4;  // four rows per CTA step; every CTA takes one step at these sizes
    cudaError_t lerr = cudaSuccess;
#define LUMEN_GATHER(XT, F16, NAT) \
    lerr = launch_dep(tc::gather_permute_x16_kernel<XT, F16, NAT>, dim3(ggrid), dim3(256), 0, st, (const XT*)x, col_src_tok, C, \
                      H, (uint16_t*)out)
    if (act_dtype == 0) {
        if (natural) LUMEN_GATHER(float, false, true);
        else LUMEN_GATHER(float, false, false);
    } else if (act_dtype == 2) {
        if (natural) LUMEN_GATHER(__half, true, true);
        else LUMEN_GATHER(__half, true, false);
    } else {
        if (natural) LUMEN_GATHER(__nv_bfloat16, false, true);
        else LUMEN_GATHER(__nv_bfloat16, false, false);
    }
#undef LUMEN_GATHER
    return lerr;
}

cudaError_t make_tmap_f16(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return e;
        if (qres != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <int Q, int MODE, int BN, bool ATMA = false, bool STG = false>
static cudaError_t launch_tc_one(const tc::Args& a, int grid, cudaStream_t st) {
    constexpr int NA = 2;
    constexpr int STAGES = tc::StagesOf<Q, BN, ATMA, STG>::value;
    const int smem = STAGES * (NA * tc::SUB_BYTES + BN * 128) + 1024 + (STG ? tc::STG_BYTES : 0);
    static SmemOptIn optin;
    {
        cudaError_t e = ensure_dyn_smem(tc::grouped_gemm_tc_kernel<Q, MODE, BN, ATMA, STG>, (size_t)smem, optin);
        if (e != cudaSuccess) return e;
    }
    count_launch();
    return launch_dep(tc::grouped_gemm_tc_kernel<Q, MODE, BN, ATMA, STG>, dim3(grid), dim3(tc::THREADS), (size_t)smem, st, a);
}

// gate/up + SwiGLU then down, both on tcgen05. x16: permuted 16-bit activations [T,H].
cudaError_t launch_grouped_tc(const PrefillArgs& p, const void* x16, int grid, cudaStream_t st, __half* out16_rows,
                              const TcPlan* plan, const TcPeerOut* peer) {
    const int C = plan ? plan->rows : p.T * p.K;
    const int gu_cols = plan ? plan->gu_cols : tc_gu_tile_cols(C, p.L.E);  // as the tile lists were built
    const int max_ct = C / gu_cols + p.L.E;
    // Down tiles: up to 256 tokens (two accumulator sets at once, no epilogue overlap between such
    // tiles) when the gate/up tiles are 256 wide, except with a tile plan of an expert-parallel call,
    // whose lists are built for 128: its epilogue stores into other GPUs' memory, and with two
    // independent accumulator sets those stores always run under the next tile's MMAs.
    const bool dn256 = (gu_cols == 256) && plan == nullptr;
    // rows that go to other ranks' return buffers leave through the staged epilogue (bulk copies)
    const bool stg = (peer != nullptr) && !dn256;
    const int mt_gu = p.L.I / 128;
    tc::Args gu{};
    cudaError_t te = make_tmap_f16(x16, (uint64_t)C, (uint64_t)p.L.H, 128, &gu.tmap);
    if (te != cudaSuccess) return te;
    gu.L = p.L;
    gu.col_src_tok = p.R.col_src_tok;
    gu.tiles = p.tiles;
    gu.n_tiles = p.n_tiles;
    gu.b_src = x16;
    gu.out16 = p.s16;
    gu.status = p.status;
    gu.status_host = p.status_host;
    gu.wait_limit_ns = p.wait_limit_us ? (uint64_t)p.wait_limit_us * 1000ull : tc::WAIT_LIMIT_NS;
    gu.debug_extra_tx = p.debug_extra_tx;
    gu.kdim = p.L.H;
    gu.out_ld = p.L.I;
    tc::Args dn = gu;
    te = make_tmap_f16(p.s16, (uint64_t)C, (uint64_t)p.L.I, 128, &dn.tmap);
    if (te != cudaSuccess) return te;
    dn.col_src_tok = nullptr;
    dn.debug_extra_tx = 0;  // the hook applies to the first kernel of the pair
    dn.tiles = p.tiles + (size_t)max_ct * (mt_gu > 0 ? mt_gu : 1);  // as laid out by launch_route_large
    dn.b_src = p.s16;
    // out16_rows: write the down product straight into caller rows (row = col_src_tok[column])
    dn.out16 = out16_rows ? out16_rows : p.d16;
    dn.out_row_map = out16_rows ? p.R.col_src_tok : nullptr;
    if (peer) dn.peer = *peer;
    dn.kdim = p.L.I;
    dn.out_ld = p.L.H;
    cudaError_t e;
    if (p.L.gu16 != nullptr) {
        // TMA-fed weights: the experts' plain f16 matrices as two 2-D arrays
        te = make_tmap_f16(p.L.gu16, (uint64_t)p.L.E * 2 * p.L.I, (uint64_t)p.L.H, 128, &gu.tmap_a);
        if (te != cudaSuccess) return te;
        gu.a_rows_exp = 2 * p.L.I;
        gu.a_row1 = p.L.I;
        te = make_tmap_f16(p.L.dn16, (uint64_t)p.L.E * p.L.H, (uint64_t)p.L.I, 128, &dn.tmap_a);
        if (te != cudaSuccess) return te;
        dn.a_rows_exp = p.L.H;
        dn.a_row1 = 128;
        e = (gu_cols == 256) ? launch_tc_one<BF16, 0, 256, true>(gu, grid, st) : launch_tc_one<BF16, 0, 128, true>(gu, grid, st);
        if (e != cudaSuccess) return e;
        if (stg) return launch_tc_one<BF16, 1, 128, true, true>(dn, grid, st);
        return dn256 ? launch_tc_one<BF16, 1, 256, true>(dn, grid, st) : launch_tc_one<BF16, 1, 128, true>(dn, grid, st);
    }
    switch (p.L.quant) {
        case Q4_0:
            e = (gu_cols == 256) ? launch_tc_one<Q4_0, 0, 256>(gu, grid, st) : launch_tc_one<Q4_0, 0, 128>(gu, grid, st);
            if (e != cudaSuccess) return e;
            if (stg) return launch_tc_one<Q4_0, 1, 128, false, true>(dn, grid, st);
            return dn256 ? launch_tc_one<Q4_0, 1, 256>(dn, grid, st) : launch_tc_one<Q4_0, 1, 128>(dn, grid, st);
        case Q8_0:
            e = (gu_cols == 256) ? launch_tc_one<Q8_0, 0, 256>(gu, grid, st) : launch_tc_one<Q8_0, 0, 128>(gu, grid, st);
            if (e != cudaSuccess) return e;
            if (stg) return launch_tc_one<Q8_0, 1, 128, false, true>(dn, grid, st);
            return dn256 ? launch_tc_one<Q8_0, 1, 256>(dn, grid, st) : launch_tc_one<Q8_0, 1, 128>(dn, grid, st);
        default:
            // BF16 layers always carry their plain f16 matrices on this path (see above)
            return cudaErrorInvalidValue;
    }
}

}  // namespace lumen

#ifdef LUMEN_TC_TRACE
extern "C" __attribute__((visibility("default"))) int lumen_debug_tc_trace(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, lumen::tc::g_tc_trace, sizeof(unsigned long long) * 2 * 160 * 8);
}
#endif
