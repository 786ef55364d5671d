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
// Per CTA (448 threads), persistent over tiles (projection, 128 columns, NROWS rows):
//   warp 0      TMA producer: per 64-k stage one box of packed weights [128 columns][32 B]
//               (32-byte swizzle) and one box of activations [NROWS rows][64 k] (128-byte swizzle).
//   warp 1      MMA issuer: 4 x tcgen05.mma kind::f16 M128 N=NROWS K16 per stage, A from tensor
//               memory, B from shared memory; D in tensor memory (double buffered for NROWS <= 128).
//   warps 2-9   dequantisers (two per lane quarter: each takes 32 of the stage's 64 k).
//   warps 10-13 epilogue: tcgen05.ld of D^T, f16 / f32 narrow, row-wise coalesced stores.
#include "common.cuh"
#include "kernels.h"

namespace kaio {
namespace w4f {

constexpr int BN = 128;   // weight columns per tile = UMMA M
constexpr int BKS = 64;   // k per stage
constexpr int A_SLOTS = 8;  // tensor-memory ring of dequantised blocks (32 columns each)
constexpr int W_BYTES = BN * (BKS / 2);  // 4 KiB packed weights per stage
constexpr int SC_BYTES = BN * 2;         // one scale group x 128 columns (every second stage)
constexpr int NUM_THREADS = 448;
constexpr int NUM_DEQUANT_WARPS = 8;
constexpr int MAX_PROBS = 3;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_A_COL = 256;

template <int NROWS>
struct Cfg {
    static constexpr int X_BYTES = NROWS * 128;  // [NROWS rows][64 k f16]
    static constexpr int STAGE_BYTES = X_BYTES + W_BYTES + SC_BYTES;
    static constexpr int TMA_BYTES = X_BYTES + W_BYTES;  // without the scales
    // as many stages as fit in ~200 KB, at most 12
    static constexpr int RAW = (200 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = RAW >= 12 ? 12 : (RAW >= 8 ? 8 : 4);
    static constexpr int NBUF = NROWS <= 128 ? 2 : 1;  // D buffers in tensor memory
    static constexpr int NUM_BARS = 2 * STAGES + 2 * A_SLOTS + 4;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + NUM_BARS * 8 + 64;
    static constexpr uint32_t IDESC = make_idesc(/*d=f32*/ 1, /*a=f16*/ 0, /*b=f16*/ 0,
                                                 /*a K-major*/ 0, /*b K-major*/ 0, BN, NROWS);
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
    uint32_t* status;
};

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
__device__ __forceinline__ void dequant8_natural(uint32_t w, __half2 s2, uint32_t (&p)[4])
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

template <int NROWS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
w4a16_fused_kernel(const __grid_constant__ TensorMaps maps, const Params p)
{
    using C = Cfg<NROWS>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // [STAGES x activations (1024-aligned)] [STAGES x packed weights] [STAGES x scales]
    const uint32_t w_region = STAGES * C::X_BYTES;
    const uint32_t sc_region = w_region + STAGES * W_BYTES;
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

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    const uint32_t tiles_m = (p.m + NROWS - 1) / NROWS;
    const uint32_t tiles_n = (p.n + BN - 1) / BN;
    const uint32_t tiles_per_prob = tiles_m * tiles_n;
    const uint32_t num_tiles = tiles_per_prob * p.num_probs;
    const uint32_t num_kb = p.k / BKS;  // K % 128 == 0

    // tile -> (projection, 128-column tile, row tile); rows fastest, so a weight panel is
    // dequantised for all its row tiles back to back while it is hot in L2
    auto decode_tile = [&](uint32_t tile, uint32_t& prob, uint32_t& m0, uint32_t& n0) {
        prob = tile / tiles_per_prob;
        const uint32_t r = tile - prob * tiles_per_prob;
        m0 = (r % tiles_m) * NROWS;
        n0 = (r / tiles_m) * BN;
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
        for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            uint32_t prob, m0, n0;
            decode_tile(tile, prob, m0, n0);
            const CUtensorMap* wmap = &maps.w[prob];
            const CUtensorMap* scmap = &maps.sc[prob];
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_bounded(mma_done(s), ph ^ 1u, abort_flag, p.status, SITE_EMPTY,
                                       KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    // a scale group spans two stages: its 128 scales ride with the even one
                    // (every tile has an even number of stages, so stage parity = kb parity)
                    mbar_expect_tx(full_bar(s), C::TMA_BYTES + ((kb & 1u) ? 0 : SC_BYTES));
                    if ((kb & 1u) == 0)
                        tma_load_2d(smem_base + sc_region + s * SC_BYTES, scmap, full_bar(s),
                                    (int32_t)n0, (int32_t)(kb >> 1));
                    tma_load_2d(smem_base + s * C::X_BYTES, &maps.x, full_bar(s),
                                (int32_t)(kb * BKS), (int32_t)m0);
                    tma_load_2d(smem_base + w_region + s * W_BYTES, wmap, full_bar(s),
                                (int32_t)(kb * (BKS / 8)), (int32_t)n0);
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
        for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const uint32_t buf = C::NBUF == 2 ? (local_tile & 1u) : 0u;
            const uint32_t use = C::NBUF == 2 ? (local_tile >> 1) : local_tile;
            if (!mbar_wait_bounded(d_empty(buf), (use & 1u) ^ 1u, abort_flag, p.status, SITE_D_EMPTY,
                                   KERNEL_DQ_GEMM))
                break;
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * NROWS;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                // a_full implies the stage's TMA data landed: the dequantisers waited for it
                if (!mbar_wait_bounded(a_full(t), aph, abort_flag, p.status, SITE_A_FULL,
                                       KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a_tmem = tmem_base + TMEM_A_COL + t * (BKS / 2);
                const uint64_t b_desc0 = make_smem_desc_sw128(smem_base + s * C::X_BYTES, 16, 1024);
                if (elect_one()) {
#pragma unroll
                    for (uint32_t kk = 0; kk < BKS / 16; ++kk)
                        umma_f16_ts(d_tmem, a_tmem + kk * 8, b_desc0 + (uint64_t)(kk * 2), C::IDESC,
                                    (kb | kk) != 0 ? 1u : 0u);
                    umma_commit(mma_done(s));
                    umma_commit(a_free(t));
                    if (kb + 1 == num_kb)
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
        const uint32_t q = warp & 3u;        // tensor-memory lane quarter of this warp
        const uint32_t kh = (warp - 2) >> 2; // which 32-k half of the stage
        const uint32_t row = q * 32 + lane;  // weight column inside the tile = TMEM lane
        // 32-byte swizzle: the 16-byte chunk index is XORed with bit 2 of the row
        const uint32_t w_off = row * 32 + ((kh ^ ((row >> 2) & 1u)) << 4);
        const uint32_t a_lane = tmem_base + ((q * 32u) << 16) + TMEM_A_COL + kh * 16;
        const uint32_t sc_off = STAGES * (C::X_BYTES + W_BYTES) + row * 2;
        uint32_t s = 0, ph = 0, t = 0, tph = 0;
        bool ok = true;
        __half2 sc = __half2half2(__float2half(0.0f));
        for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_bounded(full_bar(s), ph, abort_flag, p.status, SITE_FULL,
                                       KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                const uint4 wv = *reinterpret_cast<const uint4*>(
                    smem_gen + STAGES * C::X_BYTES + s * W_BYTES + w_off);
                if ((kb & 1u) == 0)  // a new group of 128 k: its scales arrived with this stage
                    sc = __half2half2(
                        *reinterpret_cast<const __half*>(smem_gen + sc_off + s * SC_BYTES));
                // the tensor-memory block is free once the MMAs of stage it - A_SLOTS retired
                if (!mbar_wait_bounded(a_free(t), tph ^ 1u, abort_flag, p.status, SITE_A_FREE,
                                       KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                uint32_t r[16];
                uint32_t q4[4];
                dequant8_natural(wv.x, sc, q4);
                r[0] = q4[0]; r[1] = q4[1]; r[2] = q4[2]; r[3] = q4[3];
                dequant8_natural(wv.y, sc, q4);
                r[4] = q4[0]; r[5] = q4[1]; r[6] = q4[2]; r[7] = q4[3];
                dequant8_natural(wv.z, sc, q4);
                r[8] = q4[0]; r[9] = q4[1]; r[10] = q4[2]; r[11] = q4[3];
                dequant8_natural(wv.w, sc, q4);
                r[12] = q4[0]; r[13] = q4[1]; r[14] = q4[2]; r[15] = q4[3];
                tmem_st_32x32b_x16(a_lane + t * (BKS / 2), r);
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
        uint32_t local_tile = 0;
        for (uint32_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const uint32_t buf = C::NBUF == 2 ? (local_tile & 1u) : 0u;
            const uint32_t use = C::NBUF == 2 ? (local_tile >> 1) : local_tile;
            uint32_t prob, m0, n0;
            decode_tile(tile, prob, m0, n0);
            if (!mbar_wait_bounded(d_full(buf), use & 1u, abort_flag, p.status, SITE_D_FULL,
                                   KERNEL_DQ_GEMM))
                break;
            tc_fence_after_sync();
            const uint32_t col = n0 + tid;
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + buf * NROWS;
#pragma unroll 1
            for (uint32_t c = 0; c < NROWS / 32; ++c) {
                if (m0 + c * 32 >= p.m)
                    break;  // uniform
                uint32_t r[32];
                tmem_ld_32x32b_x32(taddr + c * 32, r);
                tmem_ld_wait();
                if (col < p.n) {
#pragma unroll
                    for (uint32_t i = 0; i < 32; ++i) {
                        const uint32_t rr = m0 + c * 32 + i;
                        if (rr < p.m) {
                            const size_t idx = (size_t)rr * p.n + col;
                            if (p.out_f16)
                                reinterpret_cast<__half*>(p.probs[prob].out)[idx] =
                                    __float2half_rn(__uint_as_float(r[i]));
                            else
                                reinterpret_cast<float*>(p.probs[prob].out)[idx] =
                                    __uint_as_float(r[i]);
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(d_empty(buf));
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

template <int NROWS>
static cudaError_t launch_fused_n(const DeviceCtx& ctx, const __half* x, const DqProblem* probs,
                                  int num_probs, bool out_f16, uint32_t m, uint32_t n, uint32_t k,
                                  cudaStream_t stream)
{
    using namespace w4f;
    using C = Cfg<NROWS>;
    TensorMaps maps;
    cudaError_t err = encode_tensor_map_2d(&maps.x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, k, m,
                                           (uint64_t)k * 2, BKS, NROWS, CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess)
        return err;
    Params p = {};
    for (int i = 0; i < MAX_PROBS; ++i) {
        const int j = i < num_probs ? i : 0;
        // packed weights as a 2-D u32 tensor: inner = K/8 words of one column, outer = N columns
        err = encode_tensor_map_2d(&maps.w[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, probs[j].w, k / 8,
                                   n, (uint64_t)(k / 8) * 4, BKS / 8, BN, CU_TENSOR_MAP_SWIZZLE_32B);
        if (err != cudaSuccess)
            return err;
        err = encode_tensor_map_2d(&maps.sc[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, probs[j].scales,
                                   n, k / 128, (uint64_t)n * 2, BN, 1, CU_TENSOR_MAP_SWIZZLE_NONE);
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
    p.status = ctx.status;
    const uint32_t tiles = ((m + NROWS - 1) / NROWS) * ((n + BN - 1) / BN) * (uint32_t)num_probs;
    const uint32_t grid = tiles < (uint32_t)ctx.num_sms ? tiles : (uint32_t)ctx.num_sms;
    static bool attr_set[64] = {};
    if (!attr_set[ctx.device]) {
        err = cudaFuncSetAttribute(w4a16_fused_kernel<NROWS>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (err != cudaSuccess)
            return err;
        attr_set[ctx.device] = true;
    }
    w4a16_fused_kernel<NROWS><<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(maps, p);
    return cudaGetLastError();
}

cudaError_t launch_w4a16_fused(const DeviceCtx& ctx, const __half* x, const DqProblem* probs,
                               int num_probs, bool out_f16, uint32_t m, uint32_t n, uint32_t k,
                               cudaStream_t stream)
{
    if (m <= 32)
        return launch_fused_n<32>(ctx, x, probs, num_probs, out_f16, m, n, k, stream);
    if (m <= 64)
        return launch_fused_n<64>(ctx, x, probs, num_probs, out_f16, m, n, k, stream);
    if (m <= 128)
        return launch_fused_n<128>(ctx, x, probs, num_probs, out_f16, m, n, k, stream);
    return launch_fused_n<256>(ctx, x, probs, num_probs, out_f16, m, n, k, stream);
}

}  // namespace kaio
