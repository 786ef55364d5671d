// W4A16 GEMM for decode shapes (M <= 16): out[M,N] = A[M,K] (f16) x dequant(W4[K,N]), f32
// accumulation, f32 or f16 output.  HBM-bound: the packed weights (K*N/2 bytes) are streamed
// once; everything else is small and L2-resident.
//
// Replaces the M <= 16 use of KAIO's `matmul_int4` kernel
// (kaio-ops/src/matmul_int4_kernel.rs:1492-2070), whose 64x64 block tile wastes 75-98 % of
// every mma at these M.  Arithmetic kept from the reference: w = f16(q) * f16(scale) rounded to
// f16 (mul.f16, :693-699), products accumulated in f32.
//
// Work decomposition (stream-K, deterministic):
//   unit  = (column tile of 128, K block of 256); units are numbered tile-major and cut into
//           gridDim.x contiguous ranges, so every SM streams the same number of bytes (+-1 unit).
//   A CTA that covers a tile's whole K range writes the output directly.  Otherwise each
//   contributor writes its f32 partial tile to a workspace slot and bumps the tile's counter;
//   the last one to arrive sums the partials in ascending CTA order -- a fixed order, so the
//   result does not depend on timing -- and writes the output.
//
// CTA = 15 warps:
//   warps 0-7  consumers: (k-half h, column quarter nq).  Per stage each lane takes one 16-byte
//              chunk (32 nibbles of one column) per 8-column group, dequantises in registers
//              with the 0x6400 magic-number trick (exact), multiplies by the group scale with
//              hmul2 (the reference's rounding) and feeds mma.sync.m16n8k16.  The k order inside
//              an MMA is a fixed permutation of the memory order; the activations are staged in
//              the same permutation, so no nibble shuffling is needed.
//   warp 8     TMA producer: one 2-D box [128 columns][128 B = 256 k] per stage, 128-byte swizzle
//              (conflict-free 16-byte reads), L2 evict-first.
//   warps 9-14 activation/scale loaders, one per ring slot: A[:, k-block] permuted into the
//              fragment order and the 2x128 group scales of the stage, through plain loads.
#include "common.cuh"
#include "kernels.h"

namespace kaio {
namespace w4dec {

constexpr int BN = 128;          // columns per tile
constexpr int BKK = 256;         // k per stage (128 bytes of nibbles per column)
constexpr int STAGES = 6;
constexpr int W_BYTES = BN * 128;       // 16 KiB
constexpr int A_BYTES = 16 * BKK * 2;   // 8 KiB: 16 rows x 256 k f16, fragment-permuted
constexpr int S_BYTES = 2 * BN * 2;     // 512 B: 2 groups x 128 columns f16
constexpr int STAGE_BYTES = 25 * 1024;  // W | A | scales, padded to keep W 1024-aligned
constexpr int RED_BYTES = 4 * 32 * 16 * 4;  // 8 KiB cross-warp reduction buffer
constexpr int NUM_CONSUMER_WARPS = 8;
constexpr int NUM_LOADER_WARPS = STAGES;  // loader warp w fills stage w
constexpr int NUM_THREADS = (NUM_CONSUMER_WARPS + 1 + NUM_LOADER_WARPS) * 32;  // 480
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + RED_BYTES + 256;
constexpr int PARTIAL_FLOATS = 16 * BN;  // one partial tile

enum : uint32_t { SITE_EMPTY_P = 1, SITE_EMPTY_L = 2, SITE_FULL = 3 };

struct Params {
    const __half* a;       // [M,K]
    const __half* scales;  // [K/128, N]
    void* out;             // f32 or f16 [M,N]
    float* partials;       // [grid][2][16*128]
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

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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

// 16-byte slot of (row r, 8-k group cj) in a stage's activation tile [16 rows][32 groups].  The
// XOR terms make both access patterns bank-conflict free: the loader writes 32 consecutive cj of
// one row, a consumer quarter-warp reads rows {2q, 2q+1} x groups {8t + const}.
__device__ __forceinline__ uint32_t a_slot(uint32_t r, uint32_t cj)
{
    return r * 32 + (cj & 0x18u) + (((cj & 7u) ^ (2u * ((cj >> 3) & 3u)) ^ (r & 1u)));
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

template <bool OUT_F16, bool M_LE_8>
__global__ void __launch_bounds__(NUM_THREADS, 1)
w4a16_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    float* red = reinterpret_cast<float*>(smem_gen + STAGES * STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * STAGE_BYTES + RED_BYTES);
    const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES + RED_BYTES;
    auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES);
    volatile uint32_t* last_flag = abort_flag + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    const uint32_t units = p.num_tiles * p.num_kb;
    const uint32_t u_begin = range_begin(blockIdx.x, units, gridDim.x);
    const uint32_t u_end = range_begin(blockIdx.x + 1, units, gridDim.x);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 2);  // TMA producer's expect_tx + the stage's loader warp
            mbar_init(empty_bar(s), NUM_CONSUMER_WARPS);
        }
        *abort_flag = 0;
        *last_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_w);
    }
    __syncthreads();

    if (warp == NUM_CONSUMER_WARPS) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint64_t policy = l2_policy_evict_first();
            uint32_t it = 0;
            for (uint32_t u = u_begin; u < u_end; ++u, ++it) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                if (!mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag, p.status, SITE_EMPTY_P,
                                       KERNEL_W4A16_DECODE))
                    break;
                const uint32_t tile = u / p.num_kb, kb = u % p.num_kb;
                mbar_expect_tx(full_bar(s), W_BYTES);
                tma_load_2d_hint(smem_base + s * STAGE_BYTES, &tmap_w, full_bar(s),
                                 (int32_t)(kb * (BKK / 8)), (int32_t)(tile * BN), policy);
            }
            if (*abort_flag)
                for (uint32_t spin = 0; spin < 2000; ++spin)
                    __nanosleep(100);
        }
    } else if (warp > NUM_CONSUMER_WARPS) {
        // ------------------------------------------------------------ activation / scale loaders
        // Loader warp lw owns ring slot lw, so up to STAGES activation slices are in flight at
        // once and the L2 latency of one slice is hidden behind the others.
        const uint32_t lw = warp - (NUM_CONSUMER_WARPS + 1);
        const uint32_t groups = p.k >> 7;
        for (uint32_t it = lw; u_begin + it < u_end; it += NUM_LOADER_WARPS) {
            const uint32_t u = u_begin + it;
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
            if (!mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag, p.status, SITE_EMPTY_L,
                                   KERNEL_W4A16_DECODE))
                break;
            const uint32_t tile = u / p.num_kb, kb = u % p.num_kb;
            uint8_t* stage = smem_gen + s * STAGE_BYTES;
            uint4* a_s = reinterpret_cast<uint4*>(stage + W_BYTES);
            __half* s_s = reinterpret_cast<__half*>(stage + W_BYTES + A_BYTES);
            const uint32_t k0 = kb * BKK;
            constexpr uint32_t ROWS = M_LE_8 ? 8 : 16;
            // lane = 8-k group cj of the stage; one row per step: A[r][k0 + 8 cj .. +8)
            const uint32_t cj = lane;
            const uint32_t kk = k0 + cj * 8;
            uint4 v[ROWS];
#pragma unroll
            for (uint32_t r = 0; r < ROWS; ++r) {
                v[r] = make_uint4(0, 0, 0, 0);
                if (r < p.m && kk < p.k)
                    v[r] = __ldg(reinterpret_cast<const uint4*>(p.a + (size_t)r * p.k + kk));
            }
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
            for (uint32_t r = 0; r < ROWS; ++r) {
                uint4 o;  // memory order [0..7] -> fragment order [0,4,1,5,2,6,3,7]
                o.x = __byte_perm(v[r].x, v[r].z, 0x5410);  // (h0, h4)
                o.y = __byte_perm(v[r].x, v[r].z, 0x7632);  // (h1, h5)
                o.z = __byte_perm(v[r].y, v[r].w, 0x5410);  // (h2, h6)
                o.w = __byte_perm(v[r].y, v[r].w, 0x7632);  // (h3, h7)
                a_s[a_slot(r, cj)] = o;
            }
#pragma unroll
            for (uint32_t x = 0; x < 8; ++x)
                s_s[lane + 32 * x] = sv[x];
            __syncwarp();
            if (lane == 0)
                mbar_arrive(full_bar(s));  // release: the stores above are visible to waiters
        }
    } else {
        // ------------------------------------------------------------ consumers
        const uint32_t h = warp >> 2;   // which 32-k chunks of the stage: chunk = 2t + h
        const uint32_t nq = warp & 3u;  // column quarter of the tile
        const uint32_t g = lane >> 2, t = lane & 3u;
        const uint32_t chunk = 2 * t + h;
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                acc[i][j] = 0.0f;

        uint32_t it = 0;
        uint32_t seg_kb_lo = u_begin % p.num_kb;  // first K block of the current segment
        bool ok = true;
        for (uint32_t u = u_begin; u < u_end; ++u, ++it) {
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
            const uint32_t tile = u / p.num_kb, kb = u % p.num_kb;
            if (!mbar_wait_bounded(full_bar(s), ph, abort_flag, p.status, SITE_FULL,
                                   KERNEL_W4A16_DECODE)) {
                ok = false;
                break;
            }
            const uint8_t* stage = smem_gen + s * STAGE_BYTES;
            const uint8_t* a_s = stage + W_BYTES;
            const __half* s_s = reinterpret_cast<const __half*>(stage + W_BYTES + A_BYTES);

            uint4 wv[4];
            __half2 sc[4];
#pragma unroll
            for (int ng = 0; ng < 4; ++ng) {
                const uint32_t col = nq * 32 + ng * 8 + g;  // col & 7 == g
                wv[ng] = *reinterpret_cast<const uint4*>(stage + col * 128 + ((chunk ^ g) << 4));
                sc[ng] = __half2half2(s_s[(t >> 1) * BN + col]);
            }
            uint4 alo[4], ahi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t slot = a_slot(g, chunk * 4 + j);
                alo[j] = *reinterpret_cast<const uint4*>(a_s + slot * 16);
                if (!M_LE_8)
                    ahi[j] = *reinterpret_cast<const uint4*>(a_s + (slot + 8 * 32) * 16);
                else
                    ahi[j] = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
            if (lane == 0)
                mbar_arrive(empty_bar(s));  // all shared-memory reads of this stage are done

#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int ng = 0; ng < 4; ++ng) {
                    const uint32_t w = j == 0 ? wv[ng].x : j == 1 ? wv[ng].y : j == 2 ? wv[ng].z
                                                                                      : wv[ng].w;
                    uint32_t pa, pb, pc, pd;
                    dequant8(w, sc[ng], pa, pb, pc, pd);
                    mma_16816(acc[ng], alo[j].x, ahi[j].x, alo[j].y, ahi[j].y, pa, pb);
                    mma_16816(acc[ng], alo[j].z, ahi[j].z, alo[j].w, ahi[j].w, pc, pd);
                }
            }

            // ---------------------------------------------------------- end of a segment?
            if (kb + 1 == p.num_kb || u + 1 == u_end) {
                float* myred = red + (nq * 32 + lane) * 16;
                if (h == 1) {
#pragma unroll
                    for (int ng = 0; ng < 4; ++ng)
                        *reinterpret_cast<float4*>(myred + ng * 4) =
                            make_float4(acc[ng][0], acc[ng][1], acc[ng][2], acc[ng][3]);
                }
                named_barrier(1, NUM_CONSUMER_WARPS * 32);
                if (h == 0) {
#pragma unroll
                    for (int ng = 0; ng < 4; ++ng) {
                        const float4 r4 = *reinterpret_cast<const float4*>(myred + ng * 4);
                        acc[ng][0] += r4.x;
                        acc[ng][1] += r4.y;
                        acc[ng][2] += r4.z;
                        acc[ng][3] += r4.w;
                    }
                }
                named_barrier(1, NUM_CONSUMER_WARPS * 32);

                if (h == 0) {
                    const bool complete = (seg_kb_lo == 0) && (kb + 1 == p.num_kb);
                    bool write_out = complete;
                    if (!complete) {
                        // slot 0: the segment that opens this CTA's range; slot 1: the one that closes it
                        const uint32_t first_tile = u_begin / p.num_kb;
                        const uint32_t slot = (tile == first_tile) ? 0u : 1u;
                        float* mine = p.partials +
                                      ((size_t)(blockIdx.x * 2 + slot) * PARTIAL_FLOATS) +
                                      (nq * 32 + lane) * 16;
#pragma unroll
                        for (int ng = 0; ng < 4; ++ng)
                            __stcg(reinterpret_cast<float4*>(mine + ng * 4),
                                   make_float4(acc[ng][0], acc[ng][1], acc[ng][2], acc[ng][3]));
                        __threadfence();
                        named_barrier(2, 128);
                        const uint32_t c_first = owner_of(tile * p.num_kb, units, gridDim.x);
                        const uint32_t c_last =
                            owner_of(tile * p.num_kb + p.num_kb - 1, units, gridDim.x);
                        if (threadIdx.x == 0) {
                            const uint32_t prev = atomicAdd(p.counters + tile, 1u);
                            const bool last = (prev == c_last - c_first);
                            if (last)
                                p.counters[tile] = 0;  // self-resetting for the next launch
                            *last_flag = last ? 1u : 0u;
                        }
                        named_barrier(2, 128);
                        write_out = (*last_flag != 0);
                        if (write_out) {
                            __threadfence();
#pragma unroll
                            for (int ng = 0; ng < 4; ++ng)
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    acc[ng][e] = 0.0f;
                            for (uint32_t c = c_first; c <= c_last; ++c) {
                                const uint32_t c_tile0 = range_begin(c, units, gridDim.x) / p.num_kb;
                                const uint32_t cslot = (tile == c_tile0) ? 0u : 1u;
                                const float* src = p.partials +
                                                   ((size_t)(c * 2 + cslot) * PARTIAL_FLOATS) +
                                                   (nq * 32 + lane) * 16;
#pragma unroll
                                for (int ng = 0; ng < 4; ++ng) {
                                    const float4 v =
                                        __ldcg(reinterpret_cast<const float4*>(src + ng * 4));
                                    acc[ng][0] += v.x;
                                    acc[ng][1] += v.y;
                                    acc[ng][2] += v.z;
                                    acc[ng][3] += v.w;
                                }
                            }
                        }
                        named_barrier(2, 128);  // last_flag may be rewritten after this point
                    }
                    if (write_out) {
                        // C fragment: (row g, cols 2t,2t+1) and (row g+8, cols 2t,2t+1)
#pragma unroll
                        for (int ng = 0; ng < 4; ++ng) {
                            const uint32_t col = tile * BN + nq * 32 + ng * 8 + 2 * t;
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                const uint32_t row = g + 8 * half;
                                if (row >= p.m)
                                    continue;
                                const float v0 = acc[ng][2 * half], v1 = acc[ng][2 * half + 1];
                                const size_t idx = (size_t)row * p.n + col;
                                if (OUT_F16) {
                                    __half* o = reinterpret_cast<__half*>(p.out);
                                    if (col < p.n)
                                        o[idx] = __float2half_rn(v0);
                                    if (col + 1 < p.n)
                                        o[idx + 1] = __float2half_rn(v1);
                                } else {
                                    float* o = reinterpret_cast<float*>(p.out);
                                    if (col < p.n)
                                        o[idx] = v0;
                                    if (col + 1 < p.n)
                                        o[idx + 1] = v1;
                                }
                            }
                        }
                    }
                }
#pragma unroll
                for (int ng = 0; ng < 4; ++ng)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        acc[ng][e] = 0.0f;
                seg_kb_lo = 0;  // the next segment starts a new tile
            }
        }
        (void)ok;
    }
}

}  // namespace w4dec

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
                                uint32_t* counters, cudaStream_t stream)
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
    p.out = prob.out;
    p.partials = reinterpret_cast<float*>(workspace);
    p.counters = counters;
    p.m = m;
    p.n = n;
    p.k = k;
    p.num_kb = (k + BKK - 1) / BKK;
    p.num_tiles = (n + BN - 1) / BN;
    p.status = ctx.status;
    const uint32_t grid = decode_grid(ctx, n, k);

    static bool attr_set[4][64] = {};
#define KAIO_LAUNCH_W4DEC(F16, M8)                                                                \
    do {                                                                                          \
        const int slot = (F16 ? 2 : 0) + (M8 ? 1 : 0);                                            \
        if (!attr_set[slot][ctx.device]) {                                                        \
            err = cudaFuncSetAttribute(w4a16_decode_kernel<F16, M8>,                              \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);  \
            if (err != cudaSuccess)                                                               \
                return err;                                                                       \
            attr_set[slot][ctx.device] = true;                                                    \
        }                                                                                         \
        w4a16_decode_kernel<F16, M8><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmap_w, p);       \
    } while (0)

    const bool m8 = m <= 8;
    if (out_f16) {
        if (m8)
            KAIO_LAUNCH_W4DEC(true, true);
        else
            KAIO_LAUNCH_W4DEC(true, false);
    } else {
        if (m8)
            KAIO_LAUNCH_W4DEC(false, true);
        else
            KAIO_LAUNCH_W4DEC(false, false);
    }
#undef KAIO_LAUNCH_W4DEC
    return cudaGetLastError();
}

}  // namespace kaio
