// W8A8 GEMM for sm_100a: C[M,N] = epilogue( sum_k A[M,K] (s8) * B[K,N] (s8) ), s32 accumulation.
//
// Replaces the run-time-emitted `matmul_int8` kernel of KAIO
// (kaio-ops/src/matmul_int8_kernel.rs:934-1429: 64x64 tile, mma.sync.m16n8k32.s8).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: A tile [128 rows][128 B of K] and B tile [128 k][256 B of N]
//               (two 128-byte-wide boxes) per stage, 128-byte swizzle, 4-stage ring.
//   warp 1      MMA issuer: one thread issues tcgen05.mma kind::i8, M=128 N=256 K=32;
//               A is K-major, B is read MN-major straight from its row-major [K,N] layout,
//               so no transpose or repack of the weights is needed.  Accumulators live in
//               tensor memory, double buffered (2 x 256 columns).
//   warps 2-5   epilogue: tcgen05.ld the s32 accumulators, cvt.rn.f32.s32, scale, stage a
//               [32 rows][32 columns] block in swizzled shared memory and hand it to a TMA bulk
//               store (full 128-byte lines; tile edges are clipped by the tensor map).  Runs on
//               buffer b while the mainloop fills buffer b^1.  (Per-thread row-strided 16-byte
//               stores were the bottleneck of an earlier version: 2.3 vs 3.4 POPS without them.)
//
// Shapes: K % 32 == 0 (reference contract), N % 16 == 0 and 16-byte aligned bases (TMA
// stride/alignment rules).  Ragged M and N tile edges are zero-filled by TMA on the way in
// and predicated on the way out.  Other shapes take the generic kernel.
#include "common.cuh"
#include "kernels.h"

namespace kaio {
namespace w8a8 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // bytes == int8 elements per stage along K
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;        // 16 KiB
constexpr int B_HALF_BYTES = BK * 128;  // 16 KiB: [BK k-rows][128 B of N]
constexpr int B_BYTES = 2 * B_HALF_BYTES;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KiB
constexpr int TMEM_COLS = 512;                  // 2 accumulator buffers x 256 columns
constexpr int NUM_THREADS = 192;
constexpr int STG_BYTES = 32 * 128;              // one staged block: 32 rows x 128 B
constexpr int STG_TOTAL = 4 * 2 * STG_BYTES;     // 4 epilogue warps x 2 buffers
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STG_TOTAL + 256;

constexpr uint32_t IDESC = make_idesc(/*d=s32*/ 2, /*a=s8*/ 1, /*b=s8*/ 1, /*a K-major*/ 0,
                                      /*b MN-major*/ 1, BM, BN);

enum : uint32_t { SITE_EMPTY = 1, SITE_FULL = 2, SITE_TMEM_EMPTY = 3, SITE_TMEM_FULL = 4 };

struct Params {
    void* out;             // f32 [M,N] or s32 [M,N]
    const float* a_scale;  // per-row (EPI_ROWCOL) or nullptr
    const float* w_scale;  // per-column (EPI_ROWCOL) or nullptr
    float scale;           // EPI_SCALAR
    uint32_t m, n, k;
    uint32_t* status;
};

template <int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
w8a8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle pattern.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* stg_gen = smem_gen + STAGES * STAGE_BYTES;
    const uint32_t stg_base = smem_base + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * STAGE_BYTES + STG_TOTAL);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
    const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES + STG_TOTAL;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    const uint32_t tiles_m = (p.m + BM - 1) / BM;
    const uint32_t tiles_n = (p.n + BN - 1) / BN;
    const uint32_t num_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), 4);  // one arrive per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_c);
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
        // Converged warp, one elected lane issues (keeps addresses in uniform registers).
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            const int32_t m0 = (tile % tiles_m) * BM;
            const int32_t n0 = (tile / tiles_m) * BN;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag, p.status, SITE_EMPTY,
                                       KERNEL_W8A8)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    const uint32_t stage = smem_base + s * STAGE_BYTES;
                    mbar_expect_tx(full_bar(s), STAGE_BYTES);
                    const int32_t k0 = kb * BK;
                    tma_load_2d(stage, &tmap_a, full_bar(s), k0, m0);
                    tma_load_2d(stage + A_BYTES, &tmap_b, full_bar(s), n0, k0);
                    tma_load_2d(stage + A_BYTES + B_HALF_BYTES, &tmap_b, full_bar(s), n0 + 128, k0);
                }
                __syncwarp();
                if (++s == STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
        if (!ok) {
            // Give copies already in flight a bounded time to land before the CTA exits.
            for (uint32_t spin = 0; spin < 2000; ++spin)
                __nanosleep(100);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // Converged warp, one elected lane issues.
        uint32_t s = 0, ph = 0, local_tile = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const uint32_t buf = local_tile & 1u;
            const uint32_t acc_ph = (local_tile >> 1) & 1u;
            if (!mbar_wait_bounded(tmem_empty_bar(buf), acc_ph ^ 1u, abort_flag, p.status,
                                   SITE_TMEM_EMPTY, KERNEL_W8A8)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_bounded(full_bar(s), ph, abort_flag, p.status, SITE_FULL,
                                       KERNEL_W8A8)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t stage = smem_base + s * STAGE_BYTES;
                // A: K-major, 8-row groups 1024 B apart.  B: MN-major, 8-k groups 1024 B
                // apart, the two 128-byte N chunks B_HALF_BYTES apart.
                const uint64_t a_desc = make_smem_desc_sw128(stage, 16, 1024);
                const uint64_t b_desc = make_smem_desc_sw128(stage + A_BYTES, B_HALF_BYTES, 1024);
                if (elect_one()) {
#pragma unroll
                    for (uint32_t kk = 0; kk < BK / UMMA_K; ++kk) {
                        // advance A by 32 bytes inside the swizzled row, B by 32 k-rows of 128 B
                        umma_i8(d_tmem, a_desc + (uint64_t)((kk * UMMA_K) >> 4),
                                b_desc + (uint64_t)((kk * UMMA_K * 128) >> 4), IDESC,
                                (kb | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));  // frees the stage when these MMAs retire
                    if (kb + 1 == num_kb)
                        umma_commit(tmem_full_bar(buf));
                }
                __syncwarp();
                if (++s == STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const uint32_t quarter = warp & 3u;  // TMEM lane quarter this warp may read
        uint32_t local_tile = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const uint32_t buf = local_tile & 1u;
            const uint32_t acc_ph = (local_tile >> 1) & 1u;
            const uint32_t m0 = (tile % tiles_m) * BM;
            const uint32_t n0 = (tile / tiles_m) * BN;
            if (!mbar_wait_bounded(tmem_full_bar(buf), acc_ph, abort_flag, p.status, SITE_TMEM_FULL,
                                   KERNEL_W8A8)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t row = m0 + quarter * 32 + lane;
            float row_scale = 1.0f;
            if (EPI == EPI_ROWCOL && row < p.m)
                row_scale = __ldg(p.a_scale + row);
            const uint32_t taddr = tmem_base + buf * BN + ((quarter * 32u) << 16);
            const uint32_t ewarp = warp - 2;
#pragma unroll 1
            for (uint32_t c = 0; c < BN / 32; ++c) {
                const uint32_t col0 = n0 + c * 32;
                if (col0 >= p.n)
                    break;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32b_x32(taddr + c * 32, r);
                tmem_ld_wait();
                if (EPI != EPI_S32) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        float f0 = __int2float_rn((int32_t)r[j + 0]);
                        float f1 = __int2float_rn((int32_t)r[j + 1]);
                        float f2 = __int2float_rn((int32_t)r[j + 2]);
                        float f3 = __int2float_rn((int32_t)r[j + 3]);
                        if (EPI == EPI_SCALAR) {
                            f0 = __fmul_rn(f0, p.scale);
                            f1 = __fmul_rn(f1, p.scale);
                            f2 = __fmul_rn(f2, p.scale);
                            f3 = __fmul_rn(f3, p.scale);
                        } else {
                            float4 ws = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (col0 + j < p.n)  // N % 16 == 0: whole vector in or out
                                ws = __ldg(reinterpret_cast<const float4*>(p.w_scale + col0 + j));
                            f0 = __fmul_rn(__fmul_rn(f0, row_scale), ws.x);
                            f1 = __fmul_rn(__fmul_rn(f1, row_scale), ws.y);
                            f2 = __fmul_rn(__fmul_rn(f2, row_scale), ws.z);
                            f3 = __fmul_rn(__fmul_rn(f3, row_scale), ws.w);
                        }
                        r[j + 0] = __float_as_uint(f0);
                        r[j + 1] = __float_as_uint(f1);
                        r[j + 2] = __float_as_uint(f2);
                        r[j + 3] = __float_as_uint(f3);
                    }
                }
                // stage the [32 rows][32 columns] block (128-byte rows, 128-byte swizzle) and
                // store it with one TMA bulk store; the buffer used two blocks ago must have
                // been read out by its store first
                if (lane == 0)
                    tma_store_wait_read<1>();
                __syncwarp();
                const uint32_t stg_off = (ewarp * 2 + (c & 1u)) * STG_BYTES;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<uint4*>(stg_gen + stg_off + sw128_offset(lane, j)) =
                        make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&tmap_c, stg_base + stg_off, (int32_t)col0,
                                 (int32_t)(m0 + quarter * 32));
                    tma_store_commit();
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(tmem_empty_bar(buf));
        }
    }

    // ---------------------------------------------------------------- teardown
    if (warp >= 2 && lane == 0)
        tma_store_wait_all<0>();  // the staged blocks must be out before shared memory goes away
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<TMEM_COLS>(tmem_base);
    }
}

}  // namespace w8a8

static cudaError_t encode_2d_u8(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                                uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer)
{
    return encode_tensor_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, inner, outer,
                                row_stride_bytes, box_inner, box_outer,
                                CU_TENSOR_MAP_SWIZZLE_128B);
}

bool w8a8_fast_path_ok(const void* a, const void* b, const void* out, uint32_t m, uint32_t n,
                       uint32_t k)
{
    (void)m;
    return (n % 16 == 0) && (k % 32 == 0) && ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) &&
           ((uintptr_t)out % 16 == 0);
}

cudaError_t launch_w8a8_gemm(const DeviceCtx& ctx, int epi, const int8_t* a, const int8_t* b,
                             void* out, float scale, const float* a_scale, const float* w_scale,
                             uint32_t m, uint32_t n, uint32_t k, cudaStream_t stream)
{
    using namespace w8a8;
    CUtensorMap tmap_a, tmap_b;
    cudaError_t err = encode_2d_u8(&tmap_a, a, k, m, k, BK, BM);
    if (err != cudaSuccess)
        return err;
    err = encode_2d_u8(&tmap_b, b, n, k, n, 128, BK);
    if (err != cudaSuccess)
        return err;
    CUtensorMap tmap_c;  // f32 and s32 outputs have the same geometry
    err = encode_tensor_map_2d(&tmap_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, out, n, m,
                               (uint64_t)n * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess)
        return err;

    Params p;
    p.out = out;
    p.a_scale = a_scale;
    p.w_scale = w_scale;
    p.scale = scale;
    p.m = m;
    p.n = n;
    p.k = k;
    p.status = ctx.status;

    const uint32_t tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    const uint32_t grid = tiles < (uint32_t)ctx.num_sms ? tiles : (uint32_t)ctx.num_sms;

    // The opt-in shared-memory size is a per-device function attribute.
    static bool attr_set[3][64] = {};
#define KAIO_LAUNCH_W8A8(E)                                                                       \
    do {                                                                                          \
        if (!attr_set[E][ctx.device]) {                                                           \
            err = cudaFuncSetAttribute(w8a8_gemm_kernel<E>,                                       \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);  \
            if (err != cudaSuccess)                                                               \
                return err;                                                                       \
            attr_set[E][ctx.device] = true;                                                       \
        }                                                                                         \
        w8a8_gemm_kernel<E><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmap_a, tmap_b, tmap_c, p); \
    } while (0)

    switch (epi) {
    case EPI_SCALAR:
        KAIO_LAUNCH_W8A8(EPI_SCALAR);
        break;
    case EPI_ROWCOL:
        KAIO_LAUNCH_W8A8(EPI_ROWCOL);
        break;
    default:
        KAIO_LAUNCH_W8A8(EPI_S32);
        break;
    }
#undef KAIO_LAUNCH_W8A8
    return cudaGetLastError();
}

}  // namespace kaio
