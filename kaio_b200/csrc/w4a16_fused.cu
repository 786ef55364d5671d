// Fused W4A16 GEMM for 16 < M: out[M,N] = A[M,K] (f16) x dequant(W4[K,N]) with the int4 -> f16
// dequantisation inside the GEMM (no f16 copy of the weights in global memory).
//
// Replaces KAIO's `matmul_int4` / `qkv_project_int4` kernels
// (kaio-ops/src/matmul_int4_kernel.rs:1492-2070, qkv_project_int4_kernel.rs:714-1314), which
// dequantise per lane in front of mma.sync.  Arithmetic kept: w = f16(q) * f16(group scale)
// rounded to f16 (mul.f16, matmul_int4_kernel.rs:693-699) BEFORE the MMA, f32 accumulation.
//
// The product is computed transposed, like the decode kernel:
//     D^T[128 weight columns, NROWS activation rows] += W^T[128, k] * A^T[k, NROWS]
// The dequantising threads (thread = weight column = tensor-memory lane) write the f16 weights
// straight into TENSOR MEMORY as the 128-row operand; the activations arrive by TMA as the
// K-major shared-memory operand, so both stay in the layouts the reference uses (packed words
// K-contiguous per column, activations row-major).  The k order is natural here (the activations
// cannot be permuted by TMA): a byte-permute puts nibbles (2i, 2i+1) into the two halves of a
// register, one hfma2 with per-half constants makes them exact integers, one hmul2 applies the
// group scale.
//
// Per CTA (448 threads), persistent over tiles (projection, 128 columns, NROWS rows); a stage is
// BKS = 256 / 128 / 64 k long for NROWS <= 64 / = 128 / = 256 (what fits beside the activations):
//   warp 0      TMA producer: per stage one box of packed weights [128 columns][BKS / 2 bytes]
//               (swizzle = the row length), BKS / 64 boxes of activations [NROWS rows][64 k]
//               (128-byte swizzle) and the stage's group scales, all on one barrier.
//   warp 1      MMA issuer: BKS / 16 x tcgen05.mma kind::f16 M128 N=NROWS K16 per stage, A from
//               tensor memory, B from shared memory; D in tensor memory (two buffers for
//               NROWS <= 128).
//   warps 2-9   dequantisers (two per lane quarter: each takes half of the stage's k).
//   warps 10-13 epilogue: tcgen05.ld of D^T, f16 / f32 narrow, row-wise coalesced stores (to every
//               destination of a sharded all-gather call).
// When the tiles leave a good part of the SMs' last round idle, the (tile, stage) units are cut
// into gridDim contiguous ranges instead (stream-K): a tile that a cut splits is summed from f32
// partial tiles by the last CTA to arrive, in ascending CTA order, so the result does not depend
// on timing.
#include "common.cuh"
#include "kernels.h"

namespace kaio {
namespace w4f {

constexpr int BN = 128;  // weight columns per tile = UMMA M
constexpr int NUM_THREADS = 448;
constexpr int NUM_DEQUANT_WARPS = 8;
constexpr int MAX_PROBS = 3;
constexpr uint32_t TMEM_COLS = 512;

// NROWS = activation rows per tile (the UMMA N); BKS = k per stage.  Few rows leave room for
// long stages, which matter there: the per-stage hand-offs (barrier waits, votes, arrives) cost
// about as many instructions as the arithmetic of a 64-k stage, and with few rows the
// dequantisation, not the tensor pipe, sets the pace.
template <int NROWS, int BKS>
struct Cfg {
    static constexpr int W_ROW_BYTES = BKS / 2;            // packed k of one column, one stage
    static constexpr int W_BYTES = BN * W_ROW_BYTES;
    static constexpr int X_SUB_BYTES = NROWS * 128;        // one [NROWS rows][64 k] sub-tile
    static constexpr int X_BYTES = (BKS / 64) * X_SUB_BYTES;
    static constexpr int SC_GROUPS = BKS >= 128 ? BKS / 128 : 1;  // scale rows carried by a stage
    static constexpr int SC_BYTES = SC_GROUPS * BN * 2;
    static constexpr int STAGE_BYTES = X_BYTES + W_BYTES + SC_BYTES;
    static constexpr int RAW = (200 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = RAW >= 8 ? 8 : (RAW >= 6 ? 6 : 4);
    static constexpr int NBUF = NROWS <= 128 ? 2 : 1;      // D buffers in tensor memory
    static constexpr int A_COLS = BKS / 2;                 // tensor-memory columns of one block
    static constexpr uint32_t TMEM_A_COL = NBUF * NROWS;   // blocks follow the D buffers
    static constexpr int A_SLOTS_RAW = (512 - NBUF * NROWS) / A_COLS;
    static constexpr int A_SLOTS = A_SLOTS_RAW > 8 ? 8 : A_SLOTS_RAW;
    static constexpr int CHUNKS = BKS / 64;                // 16-byte chunks per dequantising thread
    static constexpr int NUM_BARS = 2 * STAGES + 2 * A_SLOTS + 4;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + NUM_BARS * 8 + 64;
    static constexpr uint32_t IDESC = make_idesc(/*d=f32*/ 1, /*a=f16*/ 0, /*b=f16*/ 0,
                                                 /*a K-major*/ 0, /*b K-major*/ 0, BN, NROWS);
    static_assert(A_SLOTS >= 2, "tensor-memory ring too shallow");
    static_assert(SMEM_BYTES <= 227 * 1024, "stage ring does not fit");
};

enum : uint32_t {
    SITE_EMPTY = 21, SITE_FULL = 22, SITE_A_FREE = 23, SITE_A_FULL = 24, SITE_D_EMPTY = 25,
    SITE_D_FULL = 26
};

struct Problem {
    const __half* scales;  // [K/128, N]
    void* out;             // f16 or f32 [M,N]
};

struct Params {
    Problem probs[MAX_PROBS];
    uint32_t num_probs;
    uint32_t m, n, k;
    int out_f16;
    // Single-projection calls may store the result to several destinations (the sharded
    // all-gather form: every rank's output buffer, peer memory); row stride `ld` elements.
    void* copies[8];
    uint32_t num_copies;  // 0 = store to probs[prob].out with row stride n
    uint32_t scatter_cols;  // see OutputCopies
    uint64_t ld;
    // Stream-K (too few tiles to fill the SMs' last round): the (tile, k stage) units are cut
    // into gridDim contiguous ranges; a tile that a cut splits is summed from f32 partial
    // tiles in a workspace by the last CTA to arrive, in ascending CTA order (deterministic).
    int streamk;
    float4* partials;    // [grid][2][NROWS / 4][128 columns] float4 (4 rows of one column)
    uint32_t* counters;  // [tiles], zero between launches
    uint32_t* status;
};

// One piece of work: k stages [kb0, kb1) of a tile.
struct Seg {
    uint32_t tile, kb0, kb1;
};

struct SegIter {
    uint32_t tile;   // tile-per-CTA mode: next tile
    uint32_t u, u1;  // stream-K mode: next unit, end of the range
};

__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t count)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_acq_rel_gpu()
{
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
}

// First unit of CTA c when `units` units are cut into `grid` contiguous ranges.
__device__ __forceinline__ uint32_t range_begin(uint32_t c, uint32_t units, uint32_t grid)
{
    return (uint32_t)(((uint64_t)c * units) / grid);
}

// The CTA whose range holds unit u.
__device__ __forceinline__ uint32_t owner_of(uint32_t u, uint32_t units, uint32_t grid)
{
    return (uint32_t)((((uint64_t)u + 1) * grid - 1) / units);
}

struct TensorMaps {
    CUtensorMap x;
    CUtensorMap w[MAX_PROBS];
    CUtensorMap sc[MAX_PROBS];
};

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h)
{
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ __half2 u32_as_h2(uint32_t u)
{
    return *reinterpret_cast<__half2*>(&u);
}

// Eight signed nibbles of `w` -> four half2 in natural order (n0,n1) (n2,n3) (n4,n5) (n6,n7),
// each f16(q) * s rounded once (mul.f16).  Byte i of w holds nibbles 2i (low) and 2i+1 (high):
// the byte is copied into both halves, the low half keeps the low nibble as 0x6400 | (n ^ 8)
// = 1024 + (q + 8), the high half the high nibble as 0x6400 | ((n ^ 8) << 4) = 1024 + 16 (q + 8);
// hfma2 with (1, 1/16) and (-1032, -72) turns both into q exactly.
__device__ __forceinline__ void dequant8_natural(uint32_t w, __half2 s2, uint32_t* p)
{
    const __half2 mul = u32_as_h2(0x2C003C00u);  // (1, 1/16)
    const __half2 add = u32_as_h2(0xD480E408u);  // (-1032, -72)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t t = __byte_perm(w, 0u, 0x4040u | (i << 0) | (i << 8));  // [b_i, 0, b_i, 0]
        const uint32_t x = (t & 0x00F0000Fu) ^ 0x64806408u;
        const __half2 q = __hfma2(u32_as_h2(x), mul, add);
        p[i] = h2_as_u32(__hmul2(q, s2));
    }
}

__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

template <int NROWS, int BKS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
w4a16_fused_kernel(const __grid_constant__ TensorMaps maps, const Params p)
{
    using C = Cfg<NROWS, BKS>;
    constexpr int STAGES = C::STAGES;
    constexpr int A_SLOTS = C::A_SLOTS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // [STAGES x activations (1024-aligned)] [STAGES x packed weights] [STAGES x scales]
    const uint32_t w_region = STAGES * C::X_BYTES;
    const uint32_t sc_region = w_region + STAGES * C::W_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * C::STAGE_BYTES);
    const uint32_t bar_base = smem_base + STAGES * C::STAGE_BYTES;
    auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
    // mma_done[s]: the MMAs that read shared-memory stage s have retired;  a_free[t]: the MMAs
    // that read tensor-memory block t have retired (the two rings have different depths)
    auto mma_done = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
    auto a_full = [&](uint32_t t) { return bar_base + 8u * (2 * STAGES + t); };
    auto a_free = [&](uint32_t t) { return bar_base + 8u * (2 * STAGES + A_SLOTS + t); };
    auto d_full = [&](uint32_t b) { return bar_base + 8u * (2 * STAGES + 2 * A_SLOTS + b); };
    auto d_empty = [&](uint32_t b) { return bar_base + 8u * (2 * STAGES + 2 * A_SLOTS + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + C::NUM_BARS);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* last_flag = tmem_slot + 2;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    const uint32_t tiles_m = (p.m + NROWS - 1) / NROWS;
    const uint32_t tiles_n = (p.n + BN - 1) / BN;
    const uint32_t tiles_per_prob = tiles_m * tiles_n;
    const uint32_t num_tiles = tiles_per_prob * p.num_probs;
    const uint32_t num_kb = (p.k + BKS - 1) / BKS;  // K % 128 == 0; a ragged last stage reads zeros

    // tile -> (projection, 128-column tile, row tile); rows fastest, so a weight panel is
    // dequantised for all its row tiles back to back while it is hot in L2
    auto decode_tile = [&](uint32_t tile, uint32_t& prob, uint32_t& m0, uint32_t& n0) {
        prob = tile / tiles_per_prob;
        const uint32_t r = tile - prob * tiles_per_prob;
        m0 = (r % tiles_m) * NROWS;
        n0 = (r / tiles_m) * BN;
    };

    const uint32_t units = num_tiles * num_kb;
    auto seg_begin = [&]() {
        SegIter it;
        it.tile = blockIdx.x;
        it.u = range_begin(blockIdx.x, units, gridDim.x);
        it.u1 = range_begin(blockIdx.x + 1, units, gridDim.x);
        return it;
    };
    auto seg_next = [&](SegIter& it, Seg& g) {
        if (!p.streamk) {
            if (it.tile >= num_tiles)
                return false;
            g.tile = it.tile;
            g.kb0 = 0;
            g.kb1 = num_kb;
            it.tile += gridDim.x;
            return true;
        }
        if (it.u >= it.u1)
            return false;
        g.tile = it.u / num_kb;
        g.kb0 = it.u - g.tile * num_kb;
        uint32_t len = num_kb - g.kb0;
        if (len > it.u1 - it.u)
            len = it.u1 - it.u;
        g.kb1 = g.kb0 + len;
        it.u += len;
        return true;
    };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < (uint32_t)STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(mma_done(s), 1);
        }
        for (uint32_t t = 0; t < (uint32_t)A_SLOTS; ++t) {
            mbar_init(a_full(t), NUM_DEQUANT_WARPS);
            mbar_init(a_free(t), 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(d_full(b), 1);
            mbar_init(d_empty(b), 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&maps.x);
        for (uint32_t i = 0; i < p.num_probs; ++i) {
            tma_prefetch_desc(&maps.w[i]);
            tma_prefetch_desc(&maps.sc[i]);
        }
    }
    if (warp == 1) {
        tmem_alloc<TMEM_COLS>(smem_u32(const_cast<uint32_t*>(tmem_slot)));
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        uint32_t s = 0, ph = 0;
        bool ok = true;
        SegIter it = seg_begin();
        Seg g;
        while (ok && seg_next(it, g)) {
            uint32_t prob, m0, n0;
            decode_tile(g.tile, prob, m0, n0);
            const CUtensorMap* wmap = &maps.w[prob];
            const CUtensorMap* scmap = &maps.sc[prob];
            for (uint32_t kb = g.kb0; kb < g.kb1; ++kb) {
                if (!mbar_wait_bounded(mma_done(s), ph ^ 1u, abort_flag, p.status, SITE_EMPTY,
                                       KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    // with 64-k stages a scale group spans two stages: its 128 scales ride with
                    // the even one (a tile has an even number of such stages, so stage parity
                    // = kb parity)
                    const bool with_scales = (BKS >= 128) || ((kb & 1u) == 0) || (kb == g.kb0);
                    mbar_expect_tx(full_bar(s),
                                   C::X_BYTES + C::W_BYTES + (with_scales ? C::SC_BYTES : 0));
#pragma unroll
                    for (int sub = 0; sub < BKS / 64; ++sub)
                        tma_load_2d(smem_base + s * C::X_BYTES + sub * C::X_SUB_BYTES, &maps.x,
                                    full_bar(s), (int32_t)(kb * BKS + sub * 64), (int32_t)m0);
                    tma_load_2d(smem_base + w_region + s * C::W_BYTES, wmap, full_bar(s),
                                (int32_t)(kb * (BKS / 8)), (int32_t)n0);
                    if (with_scales)
                        tma_load_2d(smem_base + sc_region + s * C::SC_BYTES, scmap, full_bar(s),
                                    (int32_t)n0, (int32_t)((kb * BKS) >> 7));
                }
                __syncwarp();
                if (++s == (uint32_t)STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
        if (*abort_flag)
            for (uint32_t spin = 0; spin < 2000; ++spin)
                __nanosleep(100);
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (converged warp)
        uint32_t s = 0, t = 0, aph = 0, local_tile = 0;
        bool ok = true;
        SegIter it = seg_begin();
        Seg g;
        for (; ok && seg_next(it, g); ++local_tile) {
            const uint32_t buf = C::NBUF == 2 ? (local_tile & 1u) : 0u;
            const uint32_t use = C::NBUF == 2 ? (local_tile >> 1) : local_tile;
            if (!mbar_wait_bounded(d_empty(buf), (use & 1u) ^ 1u, abort_flag, p.status, SITE_D_EMPTY,
                                   KERNEL_DQ_GEMM))
                break;
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * NROWS;
            for (uint32_t kb = g.kb0; kb < g.kb1; ++kb) {
                // a_full implies the stage's TMA data landed: the dequantisers waited for it
                if (!mbar_wait_bounded(a_full(t), aph, abort_flag, p.status, SITE_A_FULL,
                                       KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a_tmem = tmem_base + C::TMEM_A_COL + t * C::A_COLS;
                const uint64_t b_desc0 = make_smem_desc_sw128(smem_base + s * C::X_BYTES, 16, 1024);
                if (elect_one()) {
#pragma unroll
                    for (uint32_t kk = 0; kk < BKS / 16; ++kk) {
                        // activations: 64-k sub-tile kk / 4, 32 bytes per MMA inside the row;
                        // the descriptor's address field counts 16-byte units
                        const uint32_t off = (kk >> 2) * C::X_SUB_BYTES + (kk & 3u) * 32;
                        umma_f16_ts(d_tmem, a_tmem + kk * 8, b_desc0 + (uint64_t)(off >> 4), C::IDESC,
                                    (kb != g.kb0 || kk != 0) ? 1u : 0u);
                    }
                    umma_commit(mma_done(s));
                    umma_commit(a_free(t));
                    if (kb + 1 == g.kb1)
                        umma_commit(d_full(buf));
                }
                __syncwarp();
                if (++s == (uint32_t)STAGES)
                    s = 0;
                if (++t == (uint32_t)A_SLOTS) {
                    t = 0;
                    aph ^= 1u;
                }
            }
        }
    } else if (warp < 2 + NUM_DEQUANT_WARPS) {
        // ------------------------------------------------------------ dequantisers
        const uint32_t q = warp & 3u;         // tensor-memory lane quarter of this warp
        const uint32_t kh = (warp - 2) >> 2;  // which half of the stage's k
        const uint32_t row = q * 32 + lane;   // weight column inside the tile = TMEM lane
        // 16-byte chunk j of the row sits at j ^ f(row), f by the TMA swizzle of the row length
        const uint32_t swz = C::W_ROW_BYTES == 128 ? (row & 7u)
                                                   : (C::W_ROW_BYTES == 64 ? ((row >> 1) & 3u)
                                                                           : ((row >> 2) & 1u));
        uint32_t w_off[C::CHUNKS];
#pragma unroll
        for (int c = 0; c < C::CHUNKS; ++c)
            w_off[c] = STAGES * C::X_BYTES + row * C::W_ROW_BYTES + (((kh * C::CHUNKS + c) ^ swz) << 4);
        const uint32_t a_lane =
            tmem_base + ((q * 32u) << 16) + C::TMEM_A_COL + kh * (C::A_COLS / 2);
        // this thread's scale: group kh of the stage when a stage holds two groups
        const uint32_t sc_off = STAGES * (C::X_BYTES + C::W_BYTES) +
                                ((C::SC_GROUPS == 2 ? kh : 0u) * BN + row) * 2;
        uint32_t s = 0, ph = 0, t = 0, tph = 0;
        bool ok = true;
        __half2 sc = __half2half2(__float2half(0.0f));
        SegIter it = seg_begin();
        Seg g;
        while (ok && seg_next(it, g)) {
            for (uint32_t kb = g.kb0; kb < g.kb1; ++kb) {
                if (!mbar_wait_bounded(full_bar(s), ph, abort_flag, p.status, SITE_FULL,
                                       KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                uint4 wv[C::CHUNKS];
#pragma unroll
                for (int c = 0; c < C::CHUNKS; ++c)
                    wv[c] = *reinterpret_cast<const uint4*>(smem_gen + s * C::W_BYTES + w_off[c]);
                if (BKS >= 128 || (kb & 1u) == 0 || kb == g.kb0)  // scales arrived with this stage
                    sc = __half2half2(
                        *reinterpret_cast<const __half*>(smem_gen + sc_off + s * C::SC_BYTES));
                // the tensor-memory block is free once the MMAs that read it last have retired
                if (!mbar_wait_bounded(a_free(t), tph ^ 1u, abort_flag, p.status, SITE_A_FREE,
                                       KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < C::CHUNKS; ++c) {
                    uint32_t r[16];
                    dequant8_natural(wv[c].x, sc, r + 0);
                    dequant8_natural(wv[c].y, sc, r + 4);
                    dequant8_natural(wv[c].z, sc, r + 8);
                    dequant8_natural(wv[c].w, sc, r + 12);
                    tmem_st_32x32b_x16(a_lane + t * C::A_COLS + c * 16, r);
                }
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(a_full(t));
                if (++s == (uint32_t)STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
                if (++t == (uint32_t)A_SLOTS) {
                    t = 0;
                    tph ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 10..13)
        const uint32_t q = warp & 3u;
        const uint32_t tid = q * 32 + lane;  // weight column inside the tile = TMEM lane
        constexpr uint32_t PART_F4 = (NROWS / 4) * BN;  // float4 per parked partial tile
        const uint32_t first_tile = range_begin(blockIdx.x, units, gridDim.x) / num_kb;
        uint32_t local_tile = 0;
        SegIter it = seg_begin();
        Seg g;
        for (; seg_next(it, g); ++local_tile) {
            const uint32_t buf = C::NBUF == 2 ? (local_tile & 1u) : 0u;
            const uint32_t use = C::NBUF == 2 ? (local_tile >> 1) : local_tile;
            uint32_t prob, m0, n0;
            decode_tile(g.tile, prob, m0, n0);
            if (!mbar_wait_bounded(d_full(buf), use & 1u, abort_flag, p.status, SITE_D_FULL,
                                   KERNEL_DQ_GEMM))
                break;
            tc_fence_after_sync();
            const uint32_t col = n0 + tid;
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + buf * NROWS;
            // rows [m0 + c * 32, +32) of this thread's column, f32 -> output
            auto store_rows = [&](const uint32_t (&r)[32], uint32_t c) {
                if (col >= p.n)
                    return;
                // scatter form: this column belongs to one destination only
                const uint32_t d_lo = p.scatter_cols ? col / p.scatter_cols : 0u;
                const uint32_t d_hi = p.scatter_cols ? d_lo + 1u : (p.num_copies ? p.num_copies : 1u);
                const uint32_t dcol = p.scatter_cols ? col - d_lo * p.scatter_cols : col;
                for (uint32_t d = d_lo; d < d_hi; ++d) {
                    void* const dst = p.num_copies ? p.copies[d] : p.probs[prob].out;
                    const size_t ld = p.num_copies ? (size_t)p.ld : (size_t)p.n;
#pragma unroll
                    for (uint32_t i = 0; i < 32; ++i) {
                        const uint32_t rr = m0 + c * 32 + i;
                        if (rr < p.m) {
                            const size_t idx = (size_t)rr * ld + dcol;
                            if (p.out_f16)
                                reinterpret_cast<__half*>(dst)[idx] =
                                    __float2half_rn(__uint_as_float(r[i]));
                            else
                                reinterpret_cast<float*>(dst)[idx] = __uint_as_float(r[i]);
                        }
                    }
                }
            };
            auto release_d = [&]() {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(d_empty(buf));
            };

            if (g.kb0 == 0 && g.kb1 == num_kb) {  // the whole K range: write the tile
#pragma unroll 1
                for (uint32_t c = 0; c < NROWS / 32; ++c) {
                    if (m0 + c * 32 >= p.m)
                        break;  // uniform
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, r);
                    tmem_ld_wait();
                    store_rows(r, c);
                }
                release_d();
                continue;
            }

            // ---- part of a tile that a cut between two CTAs' ranges splits along K
            // slot 0: the segment that opens this CTA's range; slot 1: the one that closes it.
            // Parked layout: float4 (4 rows of one column) at [(row / 4) * 128 + column], so a warp
            // stores 512 contiguous bytes per instruction.
            const uint32_t slot = (g.tile == first_tile) ? 0u : 1u;
            float4* const mine = p.partials + (size_t)(blockIdx.x * 2 + slot) * PART_F4 + tid;
#pragma unroll 1
            for (uint32_t c = 0; c < NROWS / 32; ++c) {
                if (m0 + c * 32 >= p.m)
                    break;
                uint32_t r[32];
                tmem_ld_32x32b_x32(taddr + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    __stcg(mine + (c * 8 + j) * BN,
                           make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
            }
            release_d();
            const uint32_t c_first = owner_of(g.tile * num_kb, units, gridDim.x);
            const uint32_t c_last = owner_of(g.tile * num_kb + num_kb - 1, units, gridDim.x);
            // one thread fences for the four warps: the barrier in front orders their parked
            // stores before its release fence, the barrier behind orders its acquire fence before
            // their loads
            named_barrier(2, 128);
            if (tid == 0) {
                fence_acq_rel_gpu();
                const uint32_t prev = atomicAdd(p.counters + g.tile, 1u);
                const bool last = (prev == c_last - c_first);
                if (last)
                    p.counters[g.tile] = 0;  // self-resetting for the next launch
                fence_acq_rel_gpu();
                *last_flag = last ? 1u : 0u;
            }
            named_barrier(2, 128);
            const bool last = (*last_flag != 0);
            named_barrier(2, 128);  // last_flag may be rewritten after this point
            if (!last)
                continue;
#pragma unroll 1
            for (uint32_t c = 0; c < NROWS / 32; ++c) {
                if (m0 + c * 32 >= p.m)
                    break;
                float acc[32];
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    acc[i] = 0.0f;
#pragma unroll 2  // two contributors' loads in flight
                for (uint32_t cc = c_first; cc <= c_last; ++cc) {  // ascending: a fixed order
                    const uint32_t cc_tile0 = range_begin(cc, units, gridDim.x) / num_kb;
                    const uint32_t cslot = (g.tile == cc_tile0) ? 0u : 1u;
                    const float4* src = p.partials + (size_t)(cc * 2 + cslot) * PART_F4 + tid;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 v = __ldcg(src + (c * 8 + j) * BN);
                        acc[4 * j + 0] += v.x;
                        acc[4 * j + 1] += v.y;
                        acc[4 * j + 2] += v.z;
                        acc[4 * j + 3] += v.w;
                    }
                }
                uint32_t r[32];
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    r[i] = __float_as_uint(acc[i]);
                store_rows(r, c);
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<TMEM_COLS>(tmem_base);
    }
}

}  // namespace w4f

bool w4a16_fused_ok(const void* x, const DqProblem* probs, int num_probs, uint32_t m, uint32_t n,
                    uint32_t k)
{
    if (num_probs < 1 || num_probs > w4f::MAX_PROBS || m <= 16 || k % 128 != 0)
        return false;
    if ((uintptr_t)x % 16 != 0 || n % 8 != 0)  // TMA: 16-byte base and row pitch (scales [K/128,N])
        return false;
    for (int i = 0; i < num_probs; ++i)
        if ((uintptr_t)probs[i].w % 16 != 0 || probs[i].scales == nullptr ||
            (uintptr_t)probs[i].scales % 16 != 0)
            return false;
    return true;
}

// How a call is run: rows per tile (the UMMA N) and whether the units are spread stream-K.
struct FusedPlan {
    uint32_t rows;
    bool streamk;
};

// Cost model, from measurements on B200 (cycles per k of one tile's mainloop, and the cost of
// parking + adding the cut tiles of a stream-K run, in k of mainloop):
//   rows   32 / 64: 7.0 cycles/k (256-k stages, the dequantisation sets the pace), fix-up 2560 k
//   rows  128     : 9.5 cycles/k (128-k stages),                                   fix-up 2560 k
//   rows  256     : 17  cycles/k (64-k stages, dequantisation ~ tensor pipe),      fix-up 4096 k
// More rows per tile dequantise each weight fewer times, fewer rows give more tiles to fill the
// SMs; e.g. M = 256 runs as 256-row tiles on a whole 70B FFN matrix (224 column tiles) and as
// 128-row tiles on one eighth of it (28 column tiles).
static FusedPlan fused_plan(const DeviceCtx& ctx, int num_probs, uint32_t m, uint32_t n, uint32_t k)
{
    static const uint32_t kRows[4] = {32, 64, 128, 256};
    static const double kCyclesPerK[4] = {7.0, 7.0, 9.5, 17.0};
    static const double kFixupK[4] = {2560, 2560, 2560, 4096};
    const double sms = (double)ctx.num_sms;
    const uint32_t col_tiles = ((n + w4f::BN - 1) / w4f::BN) * (uint32_t)num_probs;
    FusedPlan best = {256, false};
    double best_cost = 1e300;
    for (int i = 3; i >= 0; --i) {  // descending: a tie keeps the larger tile (fewer dequantisations)
        const uint32_t rows = kRows[i];
        if (rows < 256 && m > 4 * rows)
            continue;  // more than four row tiles: the weights would be dequantised too often
        if (rows > 32 && rows / 2 >= m)
            continue;  // more than twice as tall as the problem
        const uint32_t tiles = ((m + rows - 1) / rows) * col_tiles;
        const double whole = kCyclesPerK[i] * (double)((tiles + ctx.num_sms - 1) / ctx.num_sms) * k;
        double even = kCyclesPerK[i] * ((double)tiles * k / sms + kFixupK[i]);
        if (k < 1024)
            even = 1e300;
        const double cost = whole < even ? whole : even;
        if (cost < best_cost * 0.999) {
            best_cost = cost;
            best.rows = rows;
            best.streamk = even < whole;
        }
    }
    return best;
}

size_t w4a16_fused_workspace_bytes(const DeviceCtx& ctx, int num_probs, uint32_t m, uint32_t n,
                                   uint32_t k)
{
    const FusedPlan plan = fused_plan(ctx, num_probs, m, n, k);
    if (!plan.streamk)
        return 0;
    return (size_t)ctx.num_sms * 2 * plan.rows * w4f::BN * sizeof(float);
}

size_t w4a16_fused_num_counters(const DeviceCtx& ctx, int num_probs, uint32_t m, uint32_t n,
                                uint32_t k)
{
    const FusedPlan plan = fused_plan(ctx, num_probs, m, n, k);
    if (!plan.streamk)
        return 0;
    return (size_t)((m + plan.rows - 1) / plan.rows) * ((n + w4f::BN - 1) / w4f::BN) * (size_t)num_probs;
}

template <int NROWS, int BKS>
static cudaError_t launch_fused_n(const DeviceCtx& ctx, const __half* x, const DqProblem* probs,
                                  int num_probs, bool out_f16, uint32_t m, uint32_t n, uint32_t k,
                                  void* workspace, uint32_t* counters, cudaStream_t stream,
                                  const OutputCopies* copies)
{
    using namespace w4f;
    using C = Cfg<NROWS, BKS>;
    TensorMaps maps;
    cudaError_t err = encode_tensor_map_2d(&maps.x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, k, m,
                                           (uint64_t)k * 2, 64, NROWS, CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess)
        return err;
    const CUtensorMapSwizzle w_swizzle = C::W_ROW_BYTES == 128
                                             ? CU_TENSOR_MAP_SWIZZLE_128B
                                             : (C::W_ROW_BYTES == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                                     : CU_TENSOR_MAP_SWIZZLE_32B);
    Params p = {};
    for (int i = 0; i < MAX_PROBS; ++i) {
        const int j = i < num_probs ? i : 0;
        // packed weights as a 2-D u32 tensor: inner = K/8 words of one column, outer = N columns
        err = encode_tensor_map_2d(&maps.w[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, probs[j].w, k / 8,
                                   n, (uint64_t)(k / 8) * 4, BKS / 8, BN, w_swizzle);
        if (err != cudaSuccess)
            return err;
        err = encode_tensor_map_2d(&maps.sc[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, probs[j].scales,
                                   n, k / 128, (uint64_t)n * 2, BN, C::SC_GROUPS,
                                   CU_TENSOR_MAP_SWIZZLE_NONE);
        if (err != cudaSuccess)
            return err;
        p.probs[i].scales = probs[j].scales;
        p.probs[i].out = probs[j].out;
    }
    p.num_probs = (uint32_t)num_probs;
    p.m = m;
    p.n = n;
    p.k = k;
    p.out_f16 = out_f16 ? 1 : 0;
    if (copies != nullptr && num_probs == 1) {
        for (uint32_t i = 0; i < copies->count && i < 8; ++i)
            p.copies[i] = copies->ptrs[i];
        p.num_copies = copies->count;
        p.ld = copies->ld;
        p.scatter_cols = copies->scatter_cols;
    }
    p.status = ctx.status;
    const uint32_t tiles = ((m + NROWS - 1) / NROWS) * ((n + BN - 1) / BN) * (uint32_t)num_probs;
    uint32_t grid = tiles < (uint32_t)ctx.num_sms ? tiles : (uint32_t)ctx.num_sms;
    p.streamk = 0;
    p.partials = reinterpret_cast<float4*>(workspace);
    p.counters = counters;
    if (workspace != nullptr && counters != nullptr && fused_plan(ctx, num_probs, m, n, k).streamk) {
        p.streamk = 1;
        const uint32_t units = tiles * ((k + BKS - 1) / BKS);
        grid = units < (uint32_t)ctx.num_sms ? units : (uint32_t)ctx.num_sms;
    }
    static bool attr_set[64] = {};
    if (!attr_set[ctx.device]) {
        err = cudaFuncSetAttribute(w4a16_fused_kernel<NROWS, BKS>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (err != cudaSuccess)
            return err;
        attr_set[ctx.device] = true;
    }
    w4a16_fused_kernel<NROWS, BKS><<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(maps, p);
    return cudaGetLastError();
}

cudaError_t launch_w4a16_fused(const DeviceCtx& ctx, const __half* x, const DqProblem* probs,
                               int num_probs, bool out_f16, uint32_t m, uint32_t n, uint32_t k,
                               void* workspace, uint32_t* counters, cudaStream_t stream,
                               const OutputCopies* copies)
{
    switch (fused_plan(ctx, num_probs, m, n, k).rows) {
    case 32:
        return launch_fused_n<32, 256>(ctx, x, probs, num_probs, out_f16, m, n, k, workspace,
                                       counters, stream, copies);
    case 64:
        return launch_fused_n<64, 256>(ctx, x, probs, num_probs, out_f16, m, n, k, workspace,
                                       counters, stream, copies);
    case 128:
        return launch_fused_n<128, 128>(ctx, x, probs, num_probs, out_f16, m, n, k, workspace,
                                        counters, stream, copies);
    default:
        return launch_fused_n<256, 64>(ctx, x, probs, num_probs, out_f16, m, n, k, workspace,
                                       counters, stream, copies);
    }
}

}  // namespace kaio
