// W4A16 GEMM for decode shapes (M <= 16): out[M,N] = A[M,K] (f16) x dequant(W4[K,N]), f32
// accumulation, f32 or f16 output.  HBM-bound: the packed weights (K*N/2 bytes) are streamed
// once; everything else is small and L2-resident.
//
// Replaces the M <= 16 use of KAIO's `matmul_int4` kernel
// (kaio-ops/src/matmul_int4_kernel.rs:1492-2070), whose 64x64 block tile wastes 75-98 % of
// every mma at these M.  Arithmetic kept from the reference: w = f16(q) * f16(scale) rounded to
// f16 (mul.f16, :693-699), products accumulated in f32.
//
// The product is computed transposed on the 5th-generation tensor cores:
//     D^T[128 weight columns, 16 activation rows] += W^T[128, k] * A^T[k, 16]
// with the dequantised weights as the 128-row operand in TENSOR MEMORY (tcgen05.st from the
// dequantising threads, no shared-memory round trip) and the activations as the K-major
// shared-memory operand.  (mma.sync runs at 256 FMA/clk/SM on this part and was the bound of
// an earlier version of this kernel.)
//
// Work decomposition (stream-K, deterministic):
//   unit  = (column tile of 128, K block of 256); units are numbered tile-major and cut into
//           gridDim.x contiguous ranges, so every SM streams the same number of bytes (+-1 unit).
//   A CTA that covers a tile's whole K range writes the output directly.  Otherwise each
//   contributor writes its f32 partial tile to a workspace slot and bumps the tile's counter;
//   the last one to arrive sums the partials in ascending CTA order -- a fixed order, so the
//   result does not depend on timing -- and writes the output.
//
// CTA = 18 warps:
//   warp 0       TMA producer: one box [128 columns][128 B = 256 k] of packed weights per stage,
//                128-byte swizzle, L2 evict-first, 6-stage ring.
//   warp 1       MMA issuer: 16 x tcgen05.mma kind::f16 (M128 N16 K16) per stage, A from tensor
//                memory, B (activations) from shared memory; D double-buffered in tensor memory.
//   warps 2,3,16,17  loaders: the stage's activation slice, written in the UMMA K-major
//                128-byte-swizzle layout with each group of 8 k permuted to the order the
//                dequantiser emits, and the stage's 2 x 128 group scales.
//   warps 4-11   dequantisers: thread = weight column = tensor-memory lane (two warps per
//                lane quarter, each taking one 128-k scale group of the stage).  16-byte
//                conflict-free reads of the packed nibbles, 0x6400 magic-number conversion
//                (exact), hmul2 by the group scale (the reference's rounding), tcgen05.st.
//   warps 12-15  epilogue: tcgen05.ld of D^T (thread = column, 16 rows), split-K fix-up,
//                coalesced stores.
#include "common.cuh"
#include "kernels.h"

namespace kaio {
namespace w4dec {

constexpr int BN = 128;   // weight columns per tile = UMMA M
constexpr int BKK = 256;  // k per stage (128 bytes of nibbles per column)
constexpr int NROWS = 16; // activation rows = UMMA N
constexpr int STAGES = 6;
constexpr int A_SLOTS = 3;              // tensor-memory ring of dequantised weight blocks
constexpr int W_BYTES = BN * 128;       // 16 KiB packed weights
constexpr int X_BYTES = NROWS * BKK * 2;  // 8 KiB activations, 4 sub-tiles [16 rows][128 B]
constexpr int S_BYTES = 2 * BN * 2;     // 512 B: 2 groups x 128 columns f16
constexpr int STAGE_BYTES = 25 * 1024;  // W | X | scales, padded to keep W and X 1024-aligned
constexpr int NUM_LOADER_WARPS = 4;
constexpr int NUM_DEQUANT_WARPS = 8;
constexpr int NUM_WARPS = 18;
constexpr int NUM_THREADS = NUM_WARPS * 32;
constexpr int NUM_BARRIERS = 3 * STAGES + A_SLOTS + 4;
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + NUM_BARRIERS * 8 + 64;
constexpr int PARTIAL_FLOATS = NROWS * BN;  // one partial tile, [column][row]
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_D_COL = 0;      // 2 x 16 columns
constexpr uint32_t TMEM_A_COL = 128;    // A_SLOTS x 128 columns (256 k of f16 pairs)

constexpr uint32_t IDESC = make_idesc(/*d=f32*/ 1, /*a=f16*/ 0, /*b=f16*/ 0, /*a K-major*/ 0,
                                      /*b K-major*/ 0, BN, NROWS);

enum : uint32_t {
    SITE_W_EMPTY = 1, SITE_W_FULL = 2, SITE_X_EMPTY = 3, SITE_A_EMPTY = 5,
    SITE_A_FULL = 6, SITE_D_EMPTY = 7, SITE_D_FULL = 8
};

struct Params {
    const __half* a;       // [M,K]
    const __half* scales;  // [K/128, N]
    void* out[8];          // destinations, f32 or f16, row stride `ld` (one entry unless sharded)
    uint32_t copies;
    uint32_t scatter_cols;  // see OutputCopies
    uint64_t ld;
    float* partials;       // [grid][2][128*16]
    uint32_t* counters;    // [tiles]
    uint32_t m, n, k;
    uint32_t num_kb;       // ceil(K / 256)
    uint32_t num_tiles;    // ceil(N / 128)
    uint32_t* status;
};

__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t count)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h)
{
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ __half2 u32_as_h2(uint32_t u)
{
    return *reinterpret_cast<__half2*>(&u);
}

// Eight signed nibbles of `w` -> four half2 of exact integers times `s2` (rounded once, like
// mul.f16): pa = (n0,n4), pb = (n1,n5), pc = (n2,n6), pd = (n3,n7).
__device__ __forceinline__ void dequant8(uint32_t w, __half2 s2, uint32_t& pa, uint32_t& pb,
                                         uint32_t& pc, uint32_t& pd)
{
    const __half2 k1032 = u32_as_h2(0x64086408u);  // 1032, 1032
    const __half2 k16th = u32_as_h2(0x2C002C00u);  // 1/16
    const __half2 km72 = u32_as_h2(0xD480D480u);   // -72
    const uint32_t w8 = w >> 8;
    // low nibble of a byte: 0x6400 | (nib ^ 8) == 1024 + (q + 8)
    const uint32_t xa = (w & 0x000F000Fu) ^ 0x64086408u;
    const uint32_t xc = (w8 & 0x000F000Fu) ^ 0x64086408u;
    // high nibble of a byte: 0x6400 | ((nib ^ 8) << 4) == 1024 + 16 (q + 8)
    const uint32_t xb = (w & 0x00F000F0u) ^ 0x64806480u;
    const uint32_t xd = (w8 & 0x00F000F0u) ^ 0x64806480u;
    const __half2 qa = __hsub2(u32_as_h2(xa), k1032);
    const __half2 qc = __hsub2(u32_as_h2(xc), k1032);
    const __half2 qb = __hfma2(u32_as_h2(xb), k16th, km72);
    const __half2 qd = __hfma2(u32_as_h2(xd), k16th, km72);
    pa = h2_as_u32(__hmul2(qa, s2));
    pb = h2_as_u32(__hmul2(qb, s2));
    pc = h2_as_u32(__hmul2(qc, s2));
    pd = h2_as_u32(__hmul2(qd, s2));
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

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem], f16 x f16 -> f32.
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

#ifdef KAIO_TRACE
// Development aid (never compiled into the shipped library): per-CTA cycle stamps of the
// pipeline hand-offs, [cta][unit][8].
__device__ unsigned long long* g_trace = nullptr;
#define KAIO_STAMP(it, slot)                                                            \
    do {                                                                                \
        if (trace_ptr && (it) < 16)                                                     \
            trace_ptr[((it)) * 8 + (slot)] = clock64();                                 \
    } while (0)
#else
#define KAIO_STAMP(it, slot) do { } while (0)
#endif

template <bool OUT_F16>
__global__ void __launch_bounds__(NUM_THREADS, 1)
w4a16_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * STAGE_BYTES);
    const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
    auto w_full = [&](uint32_t s) { return bar_base + 8u * s; };
    auto w_empty = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
    // mma_done[s]: the MMAs of the unit that used ring slot s have retired (one commit per unit
    // frees both the unit's activation slot and its tensor-memory block)
    auto mma_done = [&](uint32_t s) { return bar_base + 8u * (2 * STAGES + s); };
    auto a_full = [&](uint32_t t) { return bar_base + 8u * (3 * STAGES + t); };
    auto d_full = [&](uint32_t b) { return bar_base + 8u * (3 * STAGES + A_SLOTS + b); };
    auto d_empty = [&](uint32_t b) { return bar_base + 8u * (3 * STAGES + A_SLOTS + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + NUM_BARRIERS);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* last_flag = tmem_slot + 2;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
#ifdef KAIO_TRACE
    unsigned long long* const trace_ptr = g_trace ? g_trace + (size_t)blockIdx.x * 128 : nullptr;
#endif

    const uint32_t units = p.num_tiles * p.num_kb;
    const uint32_t u_begin = range_begin(blockIdx.x, units, gridDim.x);
    const uint32_t u_end = range_begin(blockIdx.x + 1, units, gridDim.x);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            mbar_init(w_full(s), 2);  // TMA (expect_tx) + the stage's loader warp
            mbar_init(w_empty(s), NUM_DEQUANT_WARPS);
            mbar_init(mma_done(s), 1);
        }
        for (uint32_t t = 0; t < A_SLOTS; ++t) {
            mbar_init(a_full(t), NUM_DEQUANT_WARPS);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(d_full(b), 1);
            mbar_init(d_empty(b), 4);
        }
        *abort_flag = 0;
        *last_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_w);
    }
    if (warp == 1) {
        tmem_alloc<TMEM_COLS>(smem_u32(const_cast<uint32_t*>(tmem_slot)));
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0)
        KAIO_STAMP(15, 7);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (weights)
        // The whole warp runs the loop so that its control flow and address arithmetic stay
        // warp-uniform (uniform registers feed the TMA instruction directly); one elected lane
        // issues.
        const uint64_t policy = l2_policy_evict_first();
        uint32_t tile = u_begin / p.num_kb, kb = u_begin % p.num_kb;
        uint32_t s = 0, ph = 0;
        for (uint32_t u = u_begin; u < u_end; ++u) {
            if (!mbar_wait_bounded(w_empty(s), ph ^ 1u, abort_flag, p.status, SITE_W_EMPTY,
                                   KERNEL_W4A16_DECODE))
                break;
            if (elect_one()) {
                mbar_expect_tx(w_full(s), W_BYTES);
                tma_load_2d_hint(smem_base + s * STAGE_BYTES, &tmap_w, w_full(s),
                                 (int32_t)(kb * (BKK / 8)), (int32_t)(tile * BN), policy);
                KAIO_STAMP(u - u_begin, 0);
            }
            __syncwarp();
            if (++kb == p.num_kb) {
                kb = 0;
                ++tile;
            }
            if (++s == STAGES) {
                s = 0;
                ph ^= 1u;
            }
        }
        if (*abort_flag)
            for (uint32_t spin = 0; spin < 2000; ++spin)
                __nanosleep(100);
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // Converged warp, one elected lane issues: descriptors and addresses are then computed
        // in the uniform datapath instead of being moved there per instruction, which is what
        // bounds the issue rate of these short (N = 16) MMAs.
        uint32_t seg = 0, s = 0, ph = 0, t = 0, aph = 0;
        uint32_t kb = u_begin % p.num_kb;
        bool seg_first = true;
        for (uint32_t u = u_begin; u < u_end; ++u) {
            const bool seg_last = (kb + 1 == p.num_kb) || (u + 1 == u_end);
            const uint32_t buf = seg & 1u;
            if (lane == 0)
                KAIO_STAMP(u - u_begin, 7);
            if (seg_first &&
                !mbar_wait_bounded(d_empty(buf), ((seg >> 1) & 1u) ^ 1u, abort_flag, p.status,
                                   SITE_D_EMPTY, KERNEL_W4A16_DECODE))
                break;
            // a_full implies the stage's activations are in place: the dequantisers waited for
            // the loader's arrival on w_full before they produced this block
            if (!mbar_wait_bounded(a_full(t), aph, abort_flag, p.status, SITE_A_FULL,
                                   KERNEL_W4A16_DECODE))
                break;
            tc_fence_after_sync();
            if (lane == 0)
                KAIO_STAMP(u - u_begin, 5);
            const uint32_t d_tmem = tmem_base + TMEM_D_COL + buf * NROWS;
            const uint32_t a_tmem = tmem_base + TMEM_A_COL + t * (BKK / 2);
            const uint64_t b_desc0 =
                make_smem_desc_sw128(smem_base + s * STAGE_BYTES + W_BYTES, 16, 1024);
            if (elect_one()) {
                umma_f16_ts(d_tmem, a_tmem, b_desc0, IDESC, seg_first ? 0u : 1u);
#pragma unroll
                for (uint32_t kk = 1; kk < BKK / 16; ++kk) {
                    // activations: sub-tile kk/4 (64 k, 2 KiB apart), 32 bytes per MMA inside
                    // the row; the descriptor's address field counts 16-byte units
                    umma_f16_ts(d_tmem, a_tmem + kk * 8,
                                b_desc0 + (uint64_t)((kk >> 2) * 128 + (kk & 3u) * 2), IDESC, 1u);
                }
                umma_commit(mma_done(s));
                if (seg_last)
                    umma_commit(d_full(buf));
            }
            __syncwarp();
            if (lane == 0)
                KAIO_STAMP(u - u_begin, 6);
            seg_first = false;
            if (seg_last) {
                ++seg;
                seg_first = true;
            }
            if (++kb == p.num_kb)
                kb = 0;
            if (++s == STAGES) {
                s = 0;
                ph ^= 1u;
            }
            if (++t == A_SLOTS) {
                t = 0;
                aph ^= 1u;
            }
        }
        (void)ph;
    } else if (warp == 2 || warp == 3 || warp == 16 || warp == 17) {
        // ------------------------------------------------------------ activation / scale loaders
        const uint32_t lw = warp < 4 ? warp - 2 : warp - 14;
        const uint32_t groups = p.k >> 7;
        for (uint32_t it = lw; u_begin + it < u_end; it += NUM_LOADER_WARPS) {
            const uint32_t u = u_begin + it;
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
            // the slot is free when the MMAs that read the activations and the dequantisers
            // that read the scales have both finished with it
            if (!mbar_wait_bounded(mma_done(s), ph ^ 1u, abort_flag, p.status, SITE_X_EMPTY,
                                   KERNEL_W4A16_DECODE) ||
                !mbar_wait_bounded(w_empty(s), ph ^ 1u, abort_flag, p.status, SITE_W_EMPTY,
                                   KERNEL_W4A16_DECODE))
                break;
            const uint32_t tile = u / p.num_kb, kb = u % p.num_kb;
            uint8_t* stage = smem_gen + s * STAGE_BYTES;
            uint8_t* x_s = stage + W_BYTES;
            __half* s_s = reinterpret_cast<__half*>(stage + W_BYTES + X_BYTES);
            const uint32_t k0 = kb * BKK;
            // lane = 8-k group cj of the stage (32 groups); one activation row per step
            const uint32_t cj = lane;
            const uint32_t kk = k0 + cj * 8;
            __half sv[8];
#pragma unroll
            for (uint32_t x = 0; x < 8; ++x) {
                const uint32_t i = lane + 32 * x;
                const uint32_t grp = kb * 2 + (i >> 7), col = tile * BN + (i & 127u);
                sv[x] = __float2half(0.0f);
                if (grp < groups && col < p.n)
                    sv[x] = __ldg(p.scales + (size_t)grp * p.n + col);
            }
#pragma unroll
            for (uint32_t r0 = 0; r0 < NROWS; r0 += 8) {
                if (r0 >= p.m)
                    break;  // rows >= M feed output rows that are never stored
                uint4 v[8];
#pragma unroll
                for (uint32_t r = 0; r < 8; ++r) {
                    v[r] = make_uint4(0, 0, 0, 0);
                    if (r0 + r < p.m && kk < p.k)
                        v[r] = __ldg(
                            reinterpret_cast<const uint4*>(p.a + (size_t)(r0 + r) * p.k + kk));
                }
#pragma unroll
                for (uint32_t r = 0; r < 8; ++r) {
                    if (r0 + r < p.m) {
                        uint4 o;  // memory order [0..7] -> dequantiser order [0,4,1,5,2,6,3,7]
                        o.x = __byte_perm(v[r].x, v[r].z, 0x5410);  // (h0, h4)
                        o.y = __byte_perm(v[r].x, v[r].z, 0x7632);  // (h1, h5)
                        o.z = __byte_perm(v[r].y, v[r].w, 0x5410);  // (h2, h6)
                        o.w = __byte_perm(v[r].y, v[r].w, 0x7632);  // (h3, h7)
                        // K-major 128-byte-swizzle tile: sub-tile cj/8, row, 16-byte chunk cj%8
                        *reinterpret_cast<uint4*>(x_s + (cj >> 3) * 2048 +
                                                  sw128_offset(r0 + r, cj & 7u)) = o;
                    }
                }
            }
#pragma unroll
            for (uint32_t x = 0; x < 8; ++x)
                s_s[lane + 32 * x] = sv[x];
            fence_proxy_async_smem();  // the activations are read by the tensor core (async proxy)
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(w_full(s));
                KAIO_STAMP(it, 1);
            }
        }
    } else if (warp >= 4 && warp < 12) {
        // ------------------------------------------------------------ dequantisers
        const uint32_t q = warp & 3u;          // tensor-memory lane quarter of this warp
        const uint32_t wg = (warp - 4) >> 2;   // which 128-k half (= scale group) of the stage
        const uint32_t row = q * 32 + lane;    // weight column inside the tile = TMEM lane
        // loop-invariant offsets: this thread's four 16-byte chunks and its group scale
        uint32_t w_off[4];
#pragma unroll
        for (uint32_t c = 0; c < 4; ++c)
            w_off[c] = sw128_offset(row, wg * 4 + c);
        const uint32_t sc_off = (wg * BN + row) * 2;
        const uint32_t a_lane = tmem_base + ((q * 32u) << 16) + TMEM_A_COL + wg * 64;
        uint32_t it = 0;
        for (uint32_t u = u_begin; u < u_end; ++u, ++it) {
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
            const uint32_t t = it % A_SLOTS;
            // w_full completes when both the TMA box and the loader's activations/scales landed
            if (!mbar_wait_bounded(w_full(s), ph, abort_flag, p.status, SITE_W_FULL,
                                   KERNEL_W4A16_DECODE))
                break;
            if (warp == 4 && lane == 0)
                KAIO_STAMP(it, 2);
            const uint8_t* stage = smem_gen + s * STAGE_BYTES;
            uint4 wv[4];
#pragma unroll
            for (uint32_t c = 0; c < 4; ++c)
                wv[c] = *reinterpret_cast<const uint4*>(stage + w_off[c]);
            const __half2 sc =
                __half2half2(*reinterpret_cast<const __half*>(stage + W_BYTES + X_BYTES + sc_off));
            // the tensor-memory block is free once the MMAs of unit it - A_SLOTS have retired
            if (it >= A_SLOTS) {
                const uint32_t pit = it - A_SLOTS;
                if (!mbar_wait_bounded(mma_done(pit % STAGES), (pit / STAGES) & 1u, abort_flag,
                                       p.status, SITE_A_EMPTY, KERNEL_W4A16_DECODE))
                    break;
            }
            tc_fence_after_sync();
            if (warp == 4 && lane == 0)
                KAIO_STAMP(it, 3);
            const uint32_t a_tmem = a_lane + t * (BKK / 2);
#pragma unroll
            for (uint32_t c = 0; c < 4; ++c) {
                uint32_t r[16];
                dequant8(wv[c].x, sc, r[0], r[1], r[2], r[3]);
                dequant8(wv[c].y, sc, r[4], r[5], r[6], r[7]);
                dequant8(wv[c].z, sc, r[8], r[9], r[10], r[11]);
                dequant8(wv[c].w, sc, r[12], r[13], r[14], r[15]);
                tmem_st_32x32b_x16(a_tmem + c * 16, r);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                // The stage is released only here, behind the instructions that consumed the
                // loaded words.  Releasing it right after the loads is not safe: nothing in the
                // instruction stream then ties a load to the arrive, a load scheduled close to
                // its use ran about a microsecond after the arrive, and the refill of the stage
                // (six units ahead) occasionally landed first -- seen as a few columns computed
                // from the wrong k block once in several hundred launches.
                mbar_arrive(w_empty(s));
                mbar_arrive(a_full(t));
            }
#ifdef KAIO_TRACE
            if (lane == 0 && trace_ptr && it < 16)
                atomicMax(&trace_ptr[it * 8 + 4], (unsigned long long)clock64());
#endif
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 12..15)
        const uint32_t q = warp & 3u;
        const uint32_t tid = q * 32 + lane;  // weight column inside the tile = TMEM lane
        uint32_t seg = 0;
        uint32_t seg_kb_lo = u_begin % p.num_kb;
        for (uint32_t u = u_begin; u < u_end; ++u) {
            const uint32_t tile = u / p.num_kb, kb = u % p.num_kb;
            if (!((kb + 1 == p.num_kb) || (u + 1 == u_end)))
                continue;
            const uint32_t buf = seg & 1u;
            if (!mbar_wait_bounded(d_full(buf), (seg >> 1) & 1u, abort_flag, p.status, SITE_D_FULL,
                                   KERNEL_W4A16_DECODE))
                break;
            tc_fence_after_sync();
            uint32_t raw[16];
            tmem_ld_32x32b_x16(tmem_base + ((q * 32u) << 16) + TMEM_D_COL + buf * NROWS, raw);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(d_empty(buf));
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                acc[i] = __uint_as_float(raw[i]);

            const bool complete = (seg_kb_lo == 0) && (kb + 1 == p.num_kb);
            bool write_out = complete;
            if (!complete) {
                // slot 0: the segment that opens this CTA's range; slot 1: the one that closes it
                const uint32_t first_tile = u_begin / p.num_kb;
                const uint32_t slot = (tile == first_tile) ? 0u : 1u;
                float* mine =
                    p.partials + ((size_t)(blockIdx.x * 2 + slot) * PARTIAL_FLOATS) + tid * 16;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    __stcg(reinterpret_cast<float4*>(mine + i * 4),
                           make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]));
                // One thread fences for the four warps: the barrier in front orders their parked
                // stores before its release fence, the barrier behind orders its acquire fence
                // before their loads (both fences are cumulative).  A fence in every thread costs
                // about a microsecond per launch here.
                named_barrier(2, 128);
                const uint32_t c_first = owner_of(tile * p.num_kb, units, gridDim.x);
                const uint32_t c_last = owner_of(tile * p.num_kb + p.num_kb - 1, units, gridDim.x);
                if (tid == 0) {
                    asm volatile("fence.acq_rel.gpu;" ::: "memory");
                    const uint32_t prev = atomicAdd(p.counters + tile, 1u);
                    const bool last = (prev == c_last - c_first);
                    if (last)
                        p.counters[tile] = 0;  // self-resetting for the next launch
                    asm volatile("fence.acq_rel.gpu;" ::: "memory");
                    *last_flag = last ? 1u : 0u;
                }
                named_barrier(2, 128);
                write_out = (*last_flag != 0);
                if (write_out) {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        acc[i] = 0.0f;
#pragma unroll 2  // two contributors' loads in flight
                    for (uint32_t c = c_first; c <= c_last; ++c) {
                        const uint32_t c_tile0 = range_begin(c, units, gridDim.x) / p.num_kb;
                        const uint32_t cslot = (tile == c_tile0) ? 0u : 1u;
                        const float* src =
                            p.partials + ((size_t)(c * 2 + cslot) * PARTIAL_FLOATS) + tid * 16;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float4 v4 = __ldcg(reinterpret_cast<const float4*>(src + i * 4));
                            acc[4 * i] += v4.x;
                            acc[4 * i + 1] += v4.y;
                            acc[4 * i + 2] += v4.z;
                            acc[4 * i + 3] += v4.w;
                        }
                    }
                }
                named_barrier(2, 128);  // last_flag may be rewritten after this point
            }
            if (write_out) {
                const uint32_t col = tile * BN + tid;
                if (col < p.n) {
                    // scatter form: this column belongs to one destination only
                    const uint32_t d_lo = p.scatter_cols ? col / p.scatter_cols : 0u;
                    const uint32_t d_hi = p.scatter_cols ? d_lo + 1u : p.copies;
                    const uint32_t dcol = p.scatter_cols ? col - d_lo * p.scatter_cols : col;
                    for (uint32_t d = d_lo; d < d_hi; ++d) {
#pragma unroll
                        for (uint32_t r = 0; r < NROWS; ++r) {
                            if (r < p.m) {
                                const size_t idx = (size_t)r * p.ld + dcol;
                                if (OUT_F16)
                                    reinterpret_cast<__half*>(p.out[d])[idx] = __float2half_rn(acc[r]);
                                else
                                    reinterpret_cast<float*>(p.out[d])[idx] = acc[r];
                            }
                        }
                    }
                }
            }
            ++seg;
            seg_kb_lo = 0;  // the next segment starts a new tile
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

}  // namespace w4dec

#ifdef KAIO_TRACE
extern "C" __attribute__((visibility("default"))) int kaio_b200_debug_set_trace(void* ptr)
{
    return (int)cudaMemcpyToSymbol(w4dec::g_trace, &ptr, sizeof(ptr));
}
#endif

bool w4a16_decode_ok(const void* x, const DqProblem* probs, int num_probs, uint32_t m, uint32_t n,
                     uint32_t k)
{
    (void)n;
    if (num_probs != 1 || m > 16 || k % 128 != 0)
        return false;
    return ((uintptr_t)x % 16 == 0) && ((uintptr_t)probs[0].w % 16 == 0);
}

static uint32_t decode_grid(const DeviceCtx& ctx, uint32_t n, uint32_t k)
{
    const uint32_t units = ((n + w4dec::BN - 1) / w4dec::BN) * ((k + w4dec::BKK - 1) / w4dec::BKK);
    return units < (uint32_t)ctx.num_sms ? units : (uint32_t)ctx.num_sms;
}

size_t w4a16_decode_workspace_bytes(const DeviceCtx& ctx, uint32_t n, uint32_t k)
{
    return (size_t)decode_grid(ctx, n, k) * 2 * w4dec::PARTIAL_FLOATS * sizeof(float);
}

size_t w4a16_decode_num_counters(uint32_t n)
{
    return (n + w4dec::BN - 1) / w4dec::BN;
}

cudaError_t launch_w4a16_decode(const DeviceCtx& ctx, const __half* x, const DqProblem& prob,
                                bool out_f16, uint32_t m, uint32_t n, uint32_t k, void* workspace,
                                uint32_t* counters, cudaStream_t stream, const OutputCopies* copies)
{
    using namespace w4dec;
    CUtensorMap tmap_w;
    // packed weights as a 2-D u32 tensor: inner = K/8 words of one column, outer = N columns
    cudaError_t err =
        encode_tensor_map_2d(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, prob.w, k / 8, n,
                             (uint64_t)(k / 8) * 4, BKK / 8, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess)
        return err;
    Params p;
    p.a = x;
    p.scales = prob.scales;
    for (int i = 0; i < 8; ++i)
        p.out[i] = copies ? copies->ptrs[(uint32_t)i < copies->count ? i : 0] : prob.out;
    p.copies = copies ? copies->count : 1u;
    p.ld = copies ? copies->ld : n;
    p.scatter_cols = copies ? copies->scatter_cols : 0u;
    p.partials = reinterpret_cast<float*>(workspace);
    p.counters = counters;
    p.m = m;
    p.n = n;
    p.k = k;
    p.num_kb = (k + BKK - 1) / BKK;
    p.num_tiles = (n + BN - 1) / BN;
    p.status = ctx.status;
    const uint32_t grid = decode_grid(ctx, n, k);

    static bool attr_set[2][64] = {};
#define KAIO_LAUNCH_W4DEC(F16)                                                                    \
    do {                                                                                          \
        if (!attr_set[F16 ? 1 : 0][ctx.device]) {                                                 \
            err = cudaFuncSetAttribute(w4a16_decode_kernel<F16>,                                  \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);  \
            if (err != cudaSuccess)                                                               \
                return err;                                                                       \
            attr_set[F16 ? 1 : 0][ctx.device] = true;                                             \
        }                                                                                         \
        w4a16_decode_kernel<F16><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmap_w, p);           \
    } while (0)

    if (out_f16)
        KAIO_LAUNCH_W4DEC(true);
    else
        KAIO_LAUNCH_W4DEC(false);
#undef KAIO_LAUNCH_W4DEC
    return cudaGetLastError();
}

}  // namespace kaio
