// W8A8 GEMM on CTA pairs (tcgen05 cta_group::2): C[M,N] = epilogue(A[M,K] (s8) * B[K,N] (s8)).
//
// Same arithmetic and the same operand layouts as the single-CTA kernel in w8a8_gemm.cu (which
// stays the path for M <= 128); this one is for the prefill shapes, where a 128x256 tile per SM
// needs 96 bytes of operands per clock from L2 and shared memory -- more than either delivers.
// A pair of CTAs (a cluster of 2 on neighbouring SMs) computes a 256x256 tile with one
// tcgen05.mma.cta_group::2 M256 N256 K32 per step: each CTA stages its own 128 rows of A and
// only ITS HALF (128 columns) of B, and the tensor cores of both SMs read both halves.  Operand
// traffic per SM drops by a third (64 B/clk at full rate) with plain, un-multicast TMA loads.
//
// Per CTA (192 threads):
//   warp 0     TMA producer: A box [128 rows][128 B of K], B box [128 k][128 B of N] (this CTA's
//              column half), 128-byte swizzle, 6-stage ring of 32 KiB.
//              Both CTAs' loads credit their bytes to the LEADER's "stage full" barrier (the
//              pair form of the TMA load lets the barrier live in the peer CTA), so the leader
//              learns of the peer's data without a software relay -- a remote mbarrier arrive
//              costs ~1800 cycles here and made a forwarding warp the bottleneck.
//   warp 1     leader CTA only: waits for the stage (64 KiB from both CTAs), issues 4 pair MMAs
//              per stage, and commits with a multicast arrive that frees the stage in both CTAs.
//   warps 2-5  epilogue on this CTA's 128 accumulator rows (double-buffered tensor memory):
//              tcgen05.ld, cvt.rn.f32.s32, scale, swizzled staging, TMA bulk store; then an
//              arrive on the leader's "accumulator free" barrier.
//
// Half-width tail tiles.  With T tiles on P pairs the last round is only partly filled (256
// tiles on 74 pairs: 3 full rounds and 34 tiles).  When the left-over tiles number at most P / 2
// each is cut into two 256 x 128 tiles (M256 N128 MMAs, each CTA staging 64 columns of B in the
// 64-byte swizzle), so the last round has twice the tiles of half the work.  A half tile moves
// 96 bytes of operands per clock per SM instead of 64, so it runs below the full rate, but the
// round is still shorter than a full-tile round; no reduction across CTAs is needed and the
// result stays bit-exact.
//
// Grouped form (NP = 3): the fused W8A8 QKV projection.  The three weight matrices share A (the
// activations quantised to s8 per row) and are walked as one [K, 3N] problem -- a column tile's
// index selects the projection's B and C tensor maps and its per-column scales -- so the rows of
// A a rasterisation group holds in L2 serve all three projections.  Its epilogue narrows to f16:
// out = f16_rn(((acc as f32) * a_scale[i]) * w_scale_P[j]), 64 columns per staged block.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace kaio {
namespace w8a8x2 {

constexpr int BM_CTA = 128;   // rows per CTA
constexpr int BM = 256;       // rows per pair tile
constexpr int BN = 256;
constexpr int BK = 128;       // bytes == s8 elements per stage along K
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM_CTA * BK;   // 16 KiB
constexpr int B_BYTES = BK * 128;      // 16 KiB: [BK k-rows][this CTA's 128 B of N]
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 32 KiB
constexpr int STG_BYTES = 32 * 128;
constexpr int STG_TOTAL = 4 * 2 * STG_BYTES;
constexpr int TMEM_COLS = 512;  // 2 accumulator buffers x 256 columns, in each CTA
constexpr int NUM_THREADS = 192;
constexpr int NUM_BARS = 2 * STAGES + 4;
constexpr uint32_t RASTER_GM = 8;  // m-tiles per rasterisation group
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STG_TOTAL + NUM_BARS * 8 + 64;

constexpr uint32_t IDESC = make_idesc(/*d=s32*/ 2, /*a=s8*/ 1, /*b=s8*/ 1, /*a K-major*/ 0,
                                      /*b MN-major*/ 1, BM, BN);
constexpr int BN_HALF = 128;              // half-width tail tile
constexpr int B_HALF_BYTES = BK * 64;     // 8 KiB: [BK k-rows][this CTA's 64 B of N]
constexpr uint32_t IDESC_HALF = make_idesc(2, 1, 1, 0, 1, BM, BN_HALF);

enum : uint32_t {
    SITE_EMPTY = 11, SITE_FULL = 12, SITE_PEER_FULL = 13, SITE_TMEM_EMPTY = 14, SITE_TMEM_FULL = 15
};

struct Params {
    const float* a_scale;
    const float* w_scale[3];  // per problem
    float scale;
    uint32_t m, n, k;     // n = columns of ONE problem
    uint32_t full_tiles;  // tiles [0, full_tiles) run whole; each later tile runs as two halves
    uint32_t* status;
};

// Tensor maps of a launch: A, and per problem B (whole and half-width boxes) and C.
template <int NP>
struct alignas(64) TensorMaps {
    CUtensorMap a;
    CUtensorMap b[NP];
    CUtensorMap b_half[NP];
    CUtensorMap c[NP];
};

template <int EPI, int NP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
w8a8_gemm_2cta_kernel(const __grid_constant__ TensorMaps<NP> maps,
                      const __grid_constant__ Params p)
{
    constexpr bool OUT_F16 = (EPI == EPI_ROWCOL_F16);
    constexpr uint32_t CHUNK = OUT_F16 ? 64u : 32u;  // columns per staged 128-byte-row block
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* stg_gen = smem_gen + STAGES * STAGE_BYTES;
    const uint32_t stg_base = smem_base + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * STAGE_BYTES + STG_TOTAL);
    const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES + STG_TOTAL;
    auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar = [&](uint32_t b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tmem_empty_bar = [&](uint32_t b) { return bar_base + 8u * (2 * STAGES + 2 + b); };  // leader
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + NUM_BARS);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;

    const uint32_t tiles_m = (p.m + BM - 1) / BM;
    const uint32_t tiles_n1 = (p.n + BN - 1) / BN;  // column tiles of one problem
    const uint32_t tiles_n = tiles_n1 * NP;         // of all problems side by side
    const uint32_t num_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = (p.k + BK - 1) / BK;
    // work item -> (tile, which half); half = 2 means the whole tile
    const uint32_t num_items = p.full_tiles + 2 * (num_tiles - p.full_tiles);
    auto item_tile = [&](uint32_t item, uint32_t& tile, uint32_t& half) {
        if (item < p.full_tiles) {
            tile = item;
            half = 2;
        } else {
            tile = p.full_tiles + ((item - p.full_tiles) >> 1);
            half = (item - p.full_tiles) & 1u;
        }
    };

    // Tiles are walked in groups of RASTER_GM m-tiles (m fastest inside the group, then n, then
    // the next group): pairs running side by side cover a near-square patch, the group's rows of
    // A stay in L2 while the B panels sweep past, and B stays in L2 from group to group.
    auto tile_origin = [&](uint32_t tile, uint32_t& tm, uint32_t& tn) {
        const uint32_t group_tiles = RASTER_GM * tiles_n;
        const uint32_t g = tile / group_tiles;
        const uint32_t rem = tile - g * group_tiles;
        const uint32_t gm = (tiles_m - g * RASTER_GM) < RASTER_GM ? (tiles_m - g * RASTER_GM) : RASTER_GM;
        tn = rem / gm;
        tm = g * RASTER_GM + (rem - tn * gm);
    };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), 8);  // 4 epilogue warps of each CTA
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&maps.a);
        tma_prefetch_desc(&maps.b[0]);
        tma_prefetch_desc(&maps.c[0]);
    }
    if (warp == 1) {
        tmem_alloc_2cta<TMEM_COLS>(smem_u32(const_cast<uint32_t*>(tmem_slot)));
        tmem_relinquish_2cta();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anyone arrives remotely
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (uint32_t item = pair; ok && item < num_items; item += num_pairs) {
            uint32_t tile, half, tm, tn;
            item_tile(item, tile, half);
            tile_origin(tile, tm, tn);
            const uint32_t prob = NP == 1 ? 0u : tn / tiles_n1;
            tn -= prob * tiles_n1;
            const int32_t m0 = tm * BM + rank * BM_CTA;
            const int32_t n0 = half == 2 ? tn * BN + rank * 128 : tn * BN + half * BN_HALF + rank * 64;
            const CUtensorMap* map_b = half == 2 ? &maps.b[prob] : &maps.b_half[prob];
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_bounded_cluster(empty_bar(s), ph ^ 1u, abort_flag, p.status,
                                               SITE_EMPTY, KERNEL_W8A8)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    const uint32_t stage = smem_base + s * STAGE_BYTES;
                    const int32_t k0 = kb * BK;
                    const uint32_t leader_full = mapa_shared(full_bar(s), 0);
                    if (rank == 0)  // both CTAs' boxes
                        mbar_expect_tx(full_bar(s),
                                       2 * (A_BYTES + (half == 2 ? B_BYTES : B_HALF_BYTES)));
                    tma_load_2d_pair(stage, &maps.a, leader_full, k0, m0);
                    tma_load_2d_pair(stage + A_BYTES, map_b, leader_full, n0, k0);
                }
                __syncwarp();
                if (++s == STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
        if (!ok)
            for (uint32_t spin = 0; spin < 2000; ++spin)
                __nanosleep(100);
    } else if (warp == 1 && rank == 1) {
        // the peer CTA issues no MMAs: the leader's instruction drives both tensor cores
    } else if (warp == 1) {
        // ------------------------------------------------------------ leader: MMA issuer
        uint32_t s = 0, ph = 0, local_tile = 0;
        bool ok = true;
        for (uint32_t item = pair; ok && item < num_items; item += num_pairs, ++local_tile) {
            const bool whole = item < p.full_tiles;
            const uint32_t buf = local_tile & 1u;
            const uint32_t acc_ph = (local_tile >> 1) & 1u;
            if (!mbar_wait_bounded_cluster(tmem_empty_bar(buf), acc_ph ^ 1u, abort_flag, p.status,
                                           SITE_TMEM_EMPTY, KERNEL_W8A8)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_bounded_cluster(full_bar(s), ph, abort_flag, p.status, SITE_FULL,
                                               KERNEL_W8A8)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t stage = smem_base + s * STAGE_BYTES;
                // the same offsets address the operands in both CTAs' shared memory
                const uint64_t a_desc = make_smem_desc_sw128(stage, 16, 1024);
                // B rows (one per k) are 128 bytes in a whole tile, 64 bytes in a half tile
                const uint64_t b_desc = whole ? make_smem_desc_sw128(stage + A_BYTES, 16, 1024)
                                              : make_smem_desc_sw64(stage + A_BYTES, 16, 512);
                const uint32_t b_row = whole ? 128u : 64u;
                const uint32_t idesc = whole ? IDESC : IDESC_HALF;
                if (elect_one()) {
#pragma unroll
                    for (uint32_t kk = 0; kk < BK / UMMA_K; ++kk) {
                        umma_i8_2cta(d_tmem, a_desc + (uint64_t)((kk * UMMA_K) >> 4),
                                     b_desc + (uint64_t)((kk * UMMA_K * b_row) >> 4), idesc,
                                     (kb | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit_2cta(empty_bar(s), 3);  // frees the stage in both CTAs
                    if (kb + 1 == num_kb)
                        umma_commit_2cta(tmem_full_bar(buf), 3);
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
        const uint32_t quarter = warp & 3u;
        const uint32_t ewarp = warp - 2;
        const uint32_t leader_empty0 = mapa_shared(tmem_empty_bar(0), 0);
        const uint32_t leader_empty1 = mapa_shared(tmem_empty_bar(1), 0);
        uint32_t local_tile = 0;
        for (uint32_t item = pair; item < num_items; item += num_pairs, ++local_tile) {
            const uint32_t buf = local_tile & 1u;
            const uint32_t acc_ph = (local_tile >> 1) & 1u;
            uint32_t tile, half, tm, tn;
            item_tile(item, tile, half);
            tile_origin(tile, tm, tn);
            const uint32_t prob = NP == 1 ? 0u : tn / tiles_n1;
            tn -= prob * tiles_n1;
            const float* const w_scale = p.w_scale[prob];
            const CUtensorMap* const map_c = &maps.c[prob];
            const uint32_t m0 = tm * BM + rank * BM_CTA;
            const uint32_t n0 = tn * BN + (half == 2 ? 0u : half * BN_HALF);
            const uint32_t n_chunks = (half == 2 ? BN : BN_HALF) / CHUNK;
            if (!mbar_wait_bounded_cluster(tmem_full_bar(buf), acc_ph, abort_flag, p.status,
                                           SITE_TMEM_FULL, KERNEL_W8A8))
                break;
            tc_fence_after_sync();
            const uint32_t row = m0 + quarter * 32 + lane;
            float row_scale = 1.0f;
            if ((EPI == EPI_ROWCOL || OUT_F16) && row < p.m)
                row_scale = __ldg(p.a_scale + row);
            const uint32_t taddr = tmem_base + buf * BN + ((quarter * 32u) << 16);
#pragma unroll 1
            for (uint32_t c = 0; c < n_chunks; ++c) {
                const uint32_t col0 = n0 + c * CHUNK;
                if (col0 >= p.n)
                    break;  // warp-uniform
                uint32_t r[32];
                if (OUT_F16) {
                    // 64 columns: two tensor-memory loads, scaled and narrowed to 32 f16 pairs
                    uint32_t lo[32], hi[32];
                    tmem_ld_32x32b_x32(taddr + c * 64, lo);
                    tmem_ld_32x32b_x32(taddr + c * 64 + 32, hi);
                    tmem_ld_wait();
                    auto narrow = [&](const uint32_t (&src)[32], const int part) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const uint32_t cc = col0 + part * 32 + j;
                            float4 ws = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (cc < p.n)  // N % 16 == 0: whole vector in or out
                                ws = __ldg(reinterpret_cast<const float4*>(w_scale + cc));
                            const float f0 = __fmul_rn(__fmul_rn(__int2float_rn((int32_t)src[j + 0]), row_scale), ws.x);
                            const float f1 = __fmul_rn(__fmul_rn(__int2float_rn((int32_t)src[j + 1]), row_scale), ws.y);
                            const float f2 = __fmul_rn(__fmul_rn(__int2float_rn((int32_t)src[j + 2]), row_scale), ws.z);
                            const float f3 = __fmul_rn(__fmul_rn(__int2float_rn((int32_t)src[j + 3]), row_scale), ws.w);
                            const __half2 h01 = __floats2half2_rn(f0, f1);
                            const __half2 h23 = __floats2half2_rn(f2, f3);
                            r[part * 16 + j / 2] = *reinterpret_cast<const uint32_t*>(&h01);
                            r[part * 16 + j / 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);
                        }
                    };
                    narrow(lo, 0);
                    narrow(hi, 1);
                } else {
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
                                ws = __ldg(reinterpret_cast<const float4*>(w_scale + col0 + j));
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
                }
                if (lane == 0)
                    tma_store_wait_read<1>();  // the buffer used two blocks ago has been read out
                __syncwarp();
                const uint32_t stg_off = (ewarp * 2 + (c & 1u)) * STG_BYTES;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<uint4*>(stg_gen + stg_off + sw128_offset(lane, j)) =
                        make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(map_c, stg_base + stg_off, (int32_t)col0,
                                 (int32_t)(m0 + quarter * 32));
                    tma_store_commit();
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                mbar_arrive_cluster(buf ? leader_empty1 : leader_empty0);
        }
    }

    // ---------------------------------------------------------------- teardown
    if (warp >= 2 && lane == 0)
        tma_store_wait_all<0>();
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves while the other may still touch its barriers
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_2cta<TMEM_COLS>(tmem_base);
    }
}

}  // namespace w8a8x2

// KAIO_B200_HALF_TILES=0 keeps every tile whole (tuning aid).
static bool half_tiles_disabled()
{
    static const bool off = [] {
        const char* e = getenv("KAIO_B200_HALF_TILES");
        return e != nullptr && e[0] == '0';
    }();
    return off;
}

bool w8a8_2cta_ok(uint32_t m, uint32_t n, uint32_t k)
{
    (void)n;
    (void)k;
    return m > 128;
}

// Encodes the maps and launches; NP problems share A and the shape.
template <int EPI, int NP>
static cudaError_t launch_pair_kernel(const DeviceCtx& ctx, const int8_t* a,
                                      const int8_t* const* b, void* const* out, float scale,
                                      const float* a_scale, const float* const* w_scale,
                                      uint32_t m, uint32_t n, uint32_t k, cudaStream_t stream)
{
    using namespace w8a8x2;
    constexpr bool OUT_F16 = (EPI == EPI_ROWCOL_F16);
    TensorMaps<NP> maps;
    cudaError_t err = encode_tensor_map_2d(&maps.a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, k, m, k,
                                           BK, BM_CTA, CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess)
        return err;
    for (int i = 0; i < NP; ++i) {
        err = encode_tensor_map_2d(&maps.b[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b[i], n, k, n, 128,
                                   BK, CU_TENSOR_MAP_SWIZZLE_128B);
        if (err != cudaSuccess)
            return err;
        err = encode_tensor_map_2d(&maps.b_half[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b[i], n, k, n,
                                   64, BK, CU_TENSOR_MAP_SWIZZLE_64B);
        if (err != cudaSuccess)
            return err;
        // one staged block = 32 rows x 128 bytes: 32 f32 / s32 columns or 64 f16 columns
        err = OUT_F16 ? encode_tensor_map_2d(&maps.c[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, out[i],
                                             n, m, (uint64_t)n * 2, 64, 32,
                                             CU_TENSOR_MAP_SWIZZLE_128B)
                      : encode_tensor_map_2d(&maps.c[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, out[i],
                                             n, m, (uint64_t)n * 4, 32, 32,
                                             CU_TENSOR_MAP_SWIZZLE_128B);
        if (err != cudaSuccess)
            return err;
    }
    Params p;
    p.a_scale = a_scale;
    for (int i = 0; i < 3; ++i)
        p.w_scale[i] = (w_scale != nullptr && i < NP) ? w_scale[i] : nullptr;
    p.scale = scale;
    p.m = m;
    p.n = n;
    p.k = k;
    p.status = ctx.status;
    const uint32_t tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN) * NP;
    const uint32_t max_pairs = (uint32_t)ctx.num_sms / 2;
    const uint32_t pairs = tiles < max_pairs ? tiles : max_pairs;
    // the left-over tiles of the last round run as halves when those fit in one round
    const uint32_t rem = tiles % max_pairs;
    p.full_tiles = tiles;
    if (tiles > max_pairs && rem != 0 && 2 * rem <= max_pairs && !half_tiles_disabled())
        p.full_tiles = tiles - rem;

    static bool attr_set[64] = {};
    if (!attr_set[ctx.device]) {
        err = cudaFuncSetAttribute(w8a8_gemm_2cta_kernel<EPI, NP>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (err != cudaSuccess)
            return err;
        attr_set[ctx.device] = true;
    }
    w8a8_gemm_2cta_kernel<EPI, NP><<<pairs * 2, NUM_THREADS, SMEM_BYTES, stream>>>(maps, p);
    return cudaGetLastError();
}

cudaError_t launch_w8a8_gemm_2cta(const DeviceCtx& ctx, int epi, const int8_t* a, const int8_t* b,
                                  void* out, float scale, const float* a_scale,
                                  const float* w_scale, uint32_t m, uint32_t n, uint32_t k,
                                  cudaStream_t stream)
{
    const int8_t* bs[1] = {b};
    void* outs[1] = {out};
    const float* ws[1] = {w_scale};
    switch (epi) {
    case EPI_SCALAR:
        return launch_pair_kernel<EPI_SCALAR, 1>(ctx, a, bs, outs, scale, a_scale, ws, m, n, k, stream);
    case EPI_ROWCOL:
        return launch_pair_kernel<EPI_ROWCOL, 1>(ctx, a, bs, outs, scale, a_scale, ws, m, n, k, stream);
    default:
        return launch_pair_kernel<EPI_S32, 1>(ctx, a, bs, outs, scale, a_scale, ws, m, n, k, stream);
    }
}

cudaError_t launch_w8a8_qkv_2cta(const DeviceCtx& ctx, const int8_t* xq, const float* x_scale,
                                 const int8_t* const w[3], const float* const col_scale[3],
                                 void* const out[3], uint32_t m, uint32_t n, uint32_t k,
                                 cudaStream_t stream)
{
    return launch_pair_kernel<EPI_ROWCOL_F16, 3>(ctx, xq, w, out, 1.0f, x_scale, col_scale, m, n, k,
                                                 stream);
}

}  // namespace kaio
