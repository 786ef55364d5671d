// Dequantising GEMMs for M > 16 on the tensor cores: W4A16 (`matmul_int4`, `qkv_project_int4`)
// and W8A16 (`qkv_project_int8`).
//
// Replaces KAIO's kernels `matmul_int4` (kaio-ops/src/matmul_int4_kernel.rs:1492-2070),
// `qkv_project_int4` (qkv_project_int4_kernel.rs:714-1314) and `qkv_project_int8`
// (qkv_project_int8_kernel.rs:1093-1861), which dequantise per lane in front of mma.sync.
//
// Two launches per call:
//   1. dequant_*_kernel: the weights, exactly as the reference dequantises them
//      (s4: f16(q) * f16(group scale) rounded to f16, matmul_int4_kernel.rs:655-713;
//       s8: cvt.rn.f16.s8, qkv_project_int8_kernel.rs:631-638), written once as f16 [K,N]
//      row-major into a library-owned workspace.  HBM-bound, 2.5 bytes (s4) / 3 bytes (s8) of
//      traffic per weight; for the prefill shapes this is a few percent of the GEMM.
//   2. f16_gemm_kernel: one persistent launch over all (up to three) weight matrices -- the
//      tile scheduler walks (projection, m-tile, n-tile), so the fused QKV ops stay one GEMM
//      launch with three outputs.  For M > 128 the workers are CTA pairs (tcgen05 cta_group::2,
//      256x256 tiles: each CTA stages its 128 rows of x and its 128 weight columns, plain TMA
//      loads credited to the leader's barrier, multicast commit); for smaller M single CTAs with
//      128x256 tiles.  Per CTA: warp 0 TMA producer (128-byte swizzle ring), warp 1 issues
//      tcgen05.mma kind::f16 K16 (x K-major, weights MN-major straight from the row-major [K,N]
//      layout), f32 accumulators double-buffered in tensor memory, warps 2-5 epilogue
//      (post-scale, f16/f32 narrow, swizzled staging, TMA bulk stores clipped at the edges).
//
// Shapes: N % 8 == 0 and 16-byte aligned bases (TMA).  Everything else takes the generic kernel.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "silu.cuh"

namespace kaio {
namespace f16g {

constexpr int BM_CTA = 128;  // rows per CTA
constexpr int BN = 256;
constexpr int BK = 64;       // f16 elements per stage along K (128 bytes of x per row)
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM_CTA * 128;    // 16 KiB: [128 rows][64 k f16]
constexpr int B_CHUNK_BYTES = BK * 128;  // 8 KiB: [64 k][64 n f16]
constexpr int STG_BYTES = 32 * 128;      // one staged output block: 32 rows x 128 B
constexpr int STG_TOTAL = 4 * 2 * STG_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 192;
constexpr int MAX_PROBS = 3;
constexpr uint32_t RASTER_GM = 8;  // m-tiles per rasterisation group
constexpr int MAX_OUT_MAPS = 8;  // 3 projections, or up to 8 copies of one output (sharded all-gather)

// PAIR = false: one CTA per 128x256 tile, 4 weight chunks per stage, 4 stages of 48 KiB.
// PAIR = true : a CTA pair per 256x256 tile (tcgen05 cta_group::2); each CTA stages its 128
//               rows of x and ITS 128 weight columns (2 chunks), 6 stages of 32 KiB.
template <bool PAIR>
struct Cfg {
    static constexpr int B_CHUNKS = PAIR ? 2 : 4;
    static constexpr int STAGES = PAIR ? 6 : 4;
    static constexpr int STAGE_BYTES = A_BYTES + B_CHUNKS * B_CHUNK_BYTES;
    static constexpr int BM = PAIR ? 256 : 128;
    static constexpr int NUM_BARS = 2 * STAGES + 4;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STG_TOTAL + NUM_BARS * 8 + 64;
    static constexpr uint32_t IDESC = make_idesc(/*d=f32*/ 1, /*a=f16*/ 0, /*b=f16*/ 0,
                                                 /*a K-major*/ 0, /*b MN-major*/ 1, BM, BN);
};

enum : uint32_t { SITE_EMPTY = 1, SITE_FULL = 2, SITE_TMEM_EMPTY = 3, SITE_TMEM_FULL = 4 };

struct Problem {
    const float* col_scale;  // per-column post-scale or nullptr
    float scale;             // scalar post-scale
};

struct Params {
    Problem probs[MAX_PROBS];
    uint32_t num_probs;
    uint32_t copies;  // each output block is stored to `copies` tensor maps (out[prob*copies + r])
    uint32_t scatter_cols;  // > 0: a block goes only to map col0 / scatter_cols (see OutputCopies)
    uint32_t m, n, k;
    uint32_t nt_rot;  // the walk over the column tiles starts at tile nt_rot (see OutputCopies)
    void* mc_out;     // non-null: multicast address of the output (see OutputCopies::multicast)
    uint64_t mc_ld;   // its row stride in elements
    int post_scale;
    int silu_gate;  // f16 out only: column blocks of 64 alternate between two projections a, b;
                    // the epilogue stores silu(f16(a)) * f16(b) as [m, n/2]
    uint32_t* status;
};

struct TensorMaps {
    CUtensorMap x;
    CUtensorMap w[MAX_PROBS];
    CUtensorMap out[MAX_OUT_MAPS];
};

template <bool PAIR, bool OUT_F16>
__global__ void __launch_bounds__(NUM_THREADS, 1)
f16_gemm_kernel(const __grid_constant__ TensorMaps maps, const Params p)
{
    using C = Cfg<PAIR>;
    constexpr int STAGES = C::STAGES;
    constexpr int STAGE_BYTES = C::STAGE_BYTES;
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
    auto tmem_empty_bar = [&](uint32_t b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + C::NUM_BARS);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // 0 = leader
    const uint32_t worker = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
    const uint32_t num_workers = PAIR ? (gridDim.x >> 1) : gridDim.x;

    const uint32_t tiles_m = (p.m + C::BM - 1) / C::BM;
    const uint32_t tiles_n = (p.n + BN - 1) / BN;
    const uint32_t tiles_per_prob = tiles_m * tiles_n;
    const uint32_t num_tiles = tiles_per_prob * p.num_probs;
    const uint32_t num_kb = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < (uint32_t)STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), PAIR ? 8 : 4);  // epilogue warps (of both CTAs)
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&maps.x);
        for (uint32_t i = 0; i < p.num_probs; ++i)
            tma_prefetch_desc(&maps.w[i]);
        for (uint32_t i = 0; i < p.num_probs * p.copies; ++i)
            tma_prefetch_desc(&maps.out[i]);
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_2cta<TMEM_COLS>(smem_u32(const_cast<uint32_t*>(tmem_slot)));
            tmem_relinquish_2cta();
        } else {
            tmem_alloc<TMEM_COLS>(smem_u32(const_cast<uint32_t*>(tmem_slot)));
            tmem_relinquish();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR)
        cluster_sync_all();  // both CTAs' barriers exist before anyone signals remotely
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // tile -> (projection, m-tile, n-tile).  Within a projection the tiles are walked in groups of
    // RASTER_GM m-tiles: m fastest inside the group, then n, then the next group.  The workers
    // running side by side then cover a near-square patch (few x rows x few weight panels), the
    // group's x rows stay in L2 while the weight panels sweep past, and the weights (tens of MB)
    // stay in L2 from one group to the next: each operand comes from DRAM about once.
    auto decode_tile = [&](uint32_t tile, uint32_t& prob, uint32_t& m0, uint32_t& n0) {
        prob = tile / tiles_per_prob;
        const uint32_t r = tile - prob * tiles_per_prob;
        const uint32_t group_tiles = RASTER_GM * tiles_n;
        const uint32_t g = r / group_tiles;
        const uint32_t rem = r - g * group_tiles;
        const uint32_t gm = (tiles_m - g * RASTER_GM) < RASTER_GM ? (tiles_m - g * RASTER_GM) : RASTER_GM;
        const uint32_t nt = rem / gm, mi = rem - nt * gm;
        m0 = (g * RASTER_GM + mi) * C::BM + rank * BM_CTA;
        uint32_t ntr = nt + p.nt_rot;
        if (ntr >= tiles_n)
            ntr -= tiles_n;
        n0 = ntr * BN;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (converged warp)
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (uint32_t tile = worker; ok && tile < num_tiles; tile += num_workers) {
            uint32_t prob, m0, n0;
            decode_tile(tile, prob, m0, n0);
            const CUtensorMap* wmap = &maps.w[prob];
            const uint32_t ncol0 = n0 + (PAIR ? rank * 128 : 0);  // this CTA's weight columns
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_bounded_cluster(empty_bar(s), ph ^ 1u, abort_flag, p.status,
                                               SITE_EMPTY, KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    const uint32_t stage = smem_base + s * STAGE_BYTES;
                    const int32_t k0 = kb * BK;
                    if (PAIR) {
                        // both CTAs credit their bytes to the leader's barrier
                        const uint32_t leader_full = mapa_shared(full_bar(s), 0);
                        if (rank == 0)
                            mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
                        tma_load_2d_pair(stage, &maps.x, leader_full, k0, (int32_t)m0);
#pragma unroll
                        for (int c = 0; c < C::B_CHUNKS; ++c)
                            tma_load_2d_pair(stage + A_BYTES + c * B_CHUNK_BYTES, wmap, leader_full,
                                             (int32_t)ncol0 + c * 64, k0);
                    } else {
                        mbar_expect_tx(full_bar(s), STAGE_BYTES);
                        tma_load_2d(stage, &maps.x, full_bar(s), k0, (int32_t)m0);
#pragma unroll
                        for (int c = 0; c < C::B_CHUNKS; ++c)
                            tma_load_2d(stage + A_BYTES + c * B_CHUNK_BYTES, wmap, full_bar(s),
                                        (int32_t)ncol0 + c * 64, k0);
                    }
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
    } else if (warp == 1 && rank == 0) {
        // ------------------------------------------------------------ MMA issuer (leader, converged warp)
        uint32_t s = 0, ph = 0, local_tile = 0;
        bool ok = true;
        for (uint32_t tile = worker; ok && tile < num_tiles; tile += num_workers, ++local_tile) {
            const uint32_t buf = local_tile & 1u;
            const uint32_t acc_ph = (local_tile >> 1) & 1u;
            if (!mbar_wait_bounded_cluster(tmem_empty_bar(buf), acc_ph ^ 1u, abort_flag, p.status,
                                           SITE_TMEM_EMPTY, KERNEL_DQ_GEMM))
                break;
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_bounded_cluster(full_bar(s), ph, abort_flag, p.status, SITE_FULL,
                                               KERNEL_DQ_GEMM)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t stage = smem_base + s * STAGE_BYTES;
                // x: K-major, 8-row groups 1024 B apart.  weights: MN-major, 8-k groups 1024 B
                // apart, the 64-column chunks B_CHUNK_BYTES apart.
                const uint64_t a_desc = make_smem_desc_sw128(stage, 16, 1024);
                const uint64_t b_desc = make_smem_desc_sw128(stage + A_BYTES, B_CHUNK_BYTES, 1024);
                if (elect_one()) {
#pragma unroll
                    for (uint32_t kk = 0; kk < BK / UMMA_K; ++kk) {
                        // x advances 32 bytes inside its swizzled row, weights 16 k-rows of 128 B
                        if (PAIR)
                            umma_f16_2cta(d_tmem, a_desc + (uint64_t)(kk * 2),
                                          b_desc + (uint64_t)(kk * 128), C::IDESC,
                                          (kb | kk) != 0 ? 1u : 0u);
                        else
                            umma_f16(d_tmem, a_desc + (uint64_t)(kk * 2),
                                     b_desc + (uint64_t)(kk * 128), C::IDESC,
                                     (kb | kk) != 0 ? 1u : 0u);
                    }
                    if (PAIR) {
                        umma_commit_2cta(empty_bar(s), 3);  // frees the stage in both CTAs
                        if (kb + 1 == num_kb)
                            umma_commit_2cta(tmem_full_bar(buf), 3);
                    } else {
                        umma_commit(empty_bar(s));
                        if (kb + 1 == num_kb)
                            umma_commit(tmem_full_bar(buf));
                    }
                }
                __syncwarp();
                if (++s == (uint32_t)STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const uint32_t quarter = warp & 3u;
        const uint32_t ewarp = warp - 2;
        const uint32_t leader_empty0 = PAIR ? mapa_shared(tmem_empty_bar(0), 0) : tmem_empty_bar(0);
        const uint32_t leader_empty1 = PAIR ? mapa_shared(tmem_empty_bar(1), 0) : tmem_empty_bar(1);
        constexpr uint32_t COLS_PER_BLOCK = OUT_F16 ? 64 : 32;  // 128 bytes of output per row
        uint32_t local_tile = 0;
        for (uint32_t tile = worker; tile < num_tiles; tile += num_workers, ++local_tile) {
            const uint32_t buf = local_tile & 1u;
            const uint32_t acc_ph = (local_tile >> 1) & 1u;
            uint32_t prob, m0, n0;
            decode_tile(tile, prob, m0, n0);
            const Problem& pr = p.probs[prob];
            const CUtensorMap* omap = &maps.out[prob * p.copies];
            if (!mbar_wait_bounded_cluster(tmem_full_bar(buf), acc_ph, abort_flag, p.status,
                                           SITE_TMEM_FULL, KERNEL_DQ_GEMM))
                break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + buf * BN + ((quarter * 32u) << 16);
#pragma unroll 1
            for (uint32_t c = 0; c < BN / COLS_PER_BLOCK; ++c) {
                const uint32_t col0 = n0 + c * COLS_PER_BLOCK;
                if (col0 >= p.n)
                    break;  // warp-uniform
                uint32_t stg[32];  // one 128-byte output row
                if (OUT_F16 && p.silu_gate) {
                    // blocks c (projection a) and c+1 (projection b) make one output block
                    if (c & 1u)
                        continue;
#pragma unroll
                    for (uint32_t half = 0; half < 2; ++half) {
                        uint32_t ra[32], rb[32];
                        tmem_ld_32x32b_x32(taddr + c * 64 + half * 32, ra);
                        tmem_ld_32x32b_x32(taddr + (c + 1) * 64 + half * 32, rb);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            // both projections are rounded to f16 first: the bits of the f16-out
                            // GEMM followed by the stand-alone pass
                            const __half2 ha = __floats2half2_rn(__uint_as_float(ra[j]),
                                                                 __uint_as_float(ra[j + 1]));
                            const __half2 hb = __floats2half2_rn(__uint_as_float(rb[j]),
                                                                 __uint_as_float(rb[j + 1]));
                            stg[half * 16 + (j >> 1)] =
                                silu_gate_h2(*reinterpret_cast<const uint32_t*>(&ha),
                                             *reinterpret_cast<const uint32_t*>(&hb));
                        }
                    }
                    if (lane == 0)
                        tma_store_wait_read<1>();
                    __syncwarp();
                    const uint32_t stg_off = (ewarp * 2 + ((c >> 1) & 1u)) * STG_BYTES;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<uint4*>(stg_gen + stg_off + sw128_offset(lane, j)) =
                            make_uint4(stg[4 * j], stg[4 * j + 1], stg[4 * j + 2], stg[4 * j + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(omap, stg_base + stg_off, (int32_t)(col0 >> 1),
                                     (int32_t)(m0 + quarter * 32));
                        tma_store_commit();
                    }
                    continue;
                }
#pragma unroll
                for (uint32_t half = 0; half < COLS_PER_BLOCK / 32; ++half) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(taddr + c * COLS_PER_BLOCK + half * 32, r);
                    tmem_ld_wait();
                    if (p.post_scale) {
                        const uint32_t cbase = col0 + half * 32;
                        if (pr.col_scale != nullptr) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (cbase + j < p.n)  // N % 8 == 0 and 16-byte aligned: whole vector
                                    cs = __ldg(reinterpret_cast<const float4*>(pr.col_scale + cbase + j));
                                r[j] = __float_as_uint(__fmul_rn(__uint_as_float(r[j]), cs.x));
                                r[j + 1] = __float_as_uint(__fmul_rn(__uint_as_float(r[j + 1]), cs.y));
                                r[j + 2] = __float_as_uint(__fmul_rn(__uint_as_float(r[j + 2]), cs.z));
                                r[j + 3] = __float_as_uint(__fmul_rn(__uint_as_float(r[j + 3]), cs.w));
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                r[j] = __float_as_uint(__fmul_rn(__uint_as_float(r[j]), pr.scale));
                        }
                    }
                    if (OUT_F16) {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const __half2 h = __floats2half2_rn(__uint_as_float(r[j]),
                                                                __uint_as_float(r[j + 1]));
                            stg[half * 16 + (j >> 1)] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            stg[j] = r[j];
                    }
                }
                // stage the [32 rows][128 B] block (128-byte swizzle) and bulk-store it; the
                // buffer used two blocks ago must have been read out first
                if (lane == 0)
                    tma_store_wait_read<1>();
                __syncwarp();
                const uint32_t stg_off = (ewarp * 2 + (c & 1u)) * STG_BYTES;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<uint4*>(stg_gen + stg_off + sw128_offset(lane, j)) =
                        make_uint4(stg[4 * j], stg[4 * j + 1], stg[4 * j + 2], stg[4 * j + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (p.mc_out != nullptr) {
                    // all destinations at once: the staged block goes out as 16-byte multimem
                    // stores (8 lanes = one 128-byte row, 4 rows per instruction) and the switch
                    // copies it into every rank's buffer
                    constexpr uint32_t ELEM = OUT_F16 ? 2 : 4;
                    uint8_t* const mc = reinterpret_cast<uint8_t*>(p.mc_out);
#pragma unroll
                    for (uint32_t it = 0; it < 8; ++it) {
                        const uint32_t row = it * 4 + (lane >> 3), chunk = lane & 7u;
                        const uint32_t grow = m0 + quarter * 32 + row;
                        const uint32_t gcol = col0 + chunk * (16 / ELEM);
                        if (grow < p.m && gcol < p.n) {
                            const uint4 v = *reinterpret_cast<const uint4*>(
                                stg_gen + stg_off + sw128_offset(row, chunk));
                            asm volatile(
                                "multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                                :
                                : "l"(mc + ((size_t)grow * p.mc_ld + gcol) * ELEM),
                                  "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
                                  "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                                : "memory");
                        }
                    }
                    __syncwarp();  // the block has been read out before the buffer is staged again
                } else if (lane == 0) {
                    // one store per destination: with the sharded all-gather the destinations are
                    // the [M, N] buffers of every rank (peer memory), so the transfer overlaps the
                    // GEMM tile by tile
                    if (p.scatter_cols) {
                        // scatter_cols is a multiple of the block width: one owner per block
                        const uint32_t r = col0 / p.scatter_cols;
                        tma_store_2d(omap + r, stg_base + stg_off,
                                     (int32_t)(col0 - r * p.scatter_cols),
                                     (int32_t)(m0 + quarter * 32));
                    } else {
                        for (uint32_t r = 0; r < p.copies; ++r)
                            tma_store_2d(omap + r, stg_base + stg_off, (int32_t)col0,
                                         (int32_t)(m0 + quarter * 32));
                    }
                    tma_store_commit();
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (PAIR)
                    mbar_arrive_cluster(buf ? leader_empty1 : leader_empty0);
                else
                    mbar_arrive(buf ? leader_empty1 : leader_empty0);
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (warp >= 2 && lane == 0)
        tma_store_wait_all<0>();  // staged blocks must be out before shared memory goes away
    tc_fence_before_sync();
    __syncthreads();
    if (PAIR)
        cluster_sync_all();  // neither CTA leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after_sync();
        if (PAIR)
            tmem_dealloc_2cta<TMEM_COLS>(tmem_base);
        else
            tmem_dealloc<TMEM_COLS>(tmem_base);
    }
}

}  // namespace f16g

// ---------------------------------------------------------------- dequantisation pre-pass
struct DequantArgs {
    const void* w[3];
    const __half* scales[3];
    __half* out[3];
};

// s4 packed (word k/8 of column j at (k/8) + j*(K/8)) -> f16 [K,N] row-major.  Block = 64 columns
// x 64 k through a shared-memory transpose so that both the packed reads (K-contiguous per column)
// and the f16 writes (N-contiguous per k) are coalesced.
__global__ void __launch_bounds__(256)
dequant_s4_kernel(const DequantArgs args, uint32_t n, uint32_t k)
{
    __shared__ __half tile[64][64 + 2];
    const uint32_t* w = reinterpret_cast<const uint32_t*>(args.w[blockIdx.z]);
    const __half* scales = args.scales[blockIdx.z];
    __half* out = args.out[blockIdx.z];
    const uint32_t n0 = blockIdx.x * 64, k0 = blockIdx.y * 64;
    const uint32_t k_words = k >> 3;
    // 64 columns x 8 words: thread -> (column, word)
    for (uint32_t i = threadIdx.x; i < 64 * 8; i += 256) {
        const uint32_t col = i >> 3, wi = i & 7u;
        const uint32_t gc = n0 + col, gk = k0 + wi * 8;
        if (gc < n && gk < k) {
            const uint32_t word = w[(gk >> 3) + (size_t)gc * k_words];
            const __half sc = scales[(size_t)(gk >> 7) * n + gc];
#pragma unroll
            for (int nib = 0; nib < 8; ++nib) {
                const int32_t q = ((int32_t)(word << (28 - 4 * nib))) >> 28;
                tile[wi * 8 + nib][col] = __hmul(__int2half_rn(q), sc);
            }
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 64 * 32; i += 256) {
        const uint32_t kk = i >> 5, c2 = (i & 31u) * 2;
        const uint32_t gk = k0 + kk, gc = n0 + c2;
        if (gk < k && gc < n) {  // N is even on this path
            const __half2 v = __halves2half2(tile[kk][c2], tile[kk][c2 + 1]);
            *reinterpret_cast<__half2*>(out + (size_t)gk * n + gc) = v;
        }
    }
}

// The same conversion without the shared-memory transpose, for K % 32 == 0 and even N: a thread owns
// two neighbouring columns and 32 k (one 16-byte load per column; the two halves of a 32-byte sector
// are fetched by consecutive k chunks of the same warp), and for each k the warp writes 64 columns
// as one full 128-byte line of half2.  Streams at about twice the rate of the tiled kernel, which
// spends its time in two block barriers per 4096 weights.
__global__ void __launch_bounds__(256)
dequant_s4_stream_kernel(const DequantArgs args, uint32_t n, uint32_t k)
{
    const uint32_t* w = reinterpret_cast<const uint32_t*>(args.w[blockIdx.z]);
    const __half* scales = args.scales[blockIdx.z];
    __half* out = args.out[blockIdx.z];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t col = blockIdx.x * 64 + lane * 2;
    if (col >= n)
        return;
    const uint32_t k_words = k >> 3;
    // 8 warps of a block take 8 consecutive 32-k chunks; blocks stride over K
    for (uint32_t k0 = (blockIdx.y * 8 + warp) * 32; k0 < k; k0 += gridDim.y * 8 * 32) {
        const uint4 a = *reinterpret_cast<const uint4*>(w + (k0 >> 3) + (size_t)col * k_words);
        const uint4 b = *reinterpret_cast<const uint4*>(w + (k0 >> 3) + (size_t)(col + 1) * k_words);
        const __half2 sc = *reinterpret_cast<const __half2*>(scales + (size_t)(k0 >> 7) * n + col);
        const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
        __half* dst = out + (size_t)k0 * n + col;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
            for (int nib = 0; nib < 8; ++nib) {
                const int32_t qa = ((int32_t)(wa[wi] << (28 - 4 * nib))) >> 28;
                const int32_t qb = ((int32_t)(wb[wi] << (28 - 4 * nib))) >> 28;
                const __half2 q = __halves2half2(__int2half_rn(qa), __int2half_rn(qb));
                *reinterpret_cast<__half2*>(dst + (size_t)(wi * 8 + nib) * n) = __hmul2(q, sc);
            }
        }
    }
}

static void launch_dequant_s4_any(const DequantArgs& da, uint32_t n, uint32_t k, int num_probs,
                                  cudaStream_t stream)
{
    bool aligned = true;  // 16-byte loads of the packed words, 4-byte accesses of scales and output
    for (int i = 0; i < num_probs; ++i)
        aligned = aligned && (uintptr_t)da.w[i] % 16 == 0 && (uintptr_t)da.scales[i] % 4 == 0 &&
                  (uintptr_t)da.out[i] % 4 == 0;
    if (k % 32 == 0 && n % 2 == 0 && aligned) {
        const uint32_t gx = (n + 63) / 64;
        uint32_t gy = (k + 255) / 256;
        // enough blocks to fill the GPU several times over, not more
        const uint32_t want = (148u * 32u + gx - 1) / gx;
        gy = gy < want ? gy : want;
        dequant_s4_stream_kernel<<<dim3(gx, gy < 1 ? 1 : gy, num_probs), 256, 0, stream>>>(da, n, k);
    } else {
        dim3 grid((n + 63) / 64, (k + 63) / 64, num_probs);
        dequant_s4_kernel<<<grid, 256, 0, stream>>>(da, n, k);
    }
}

// s8 [K,N] -> f16 [K,N] (exact).  One 8-byte load and one 16-byte store per thread and step: every
// store instruction of a warp covers 512 contiguous bytes.  (A 16-byte load with two 16-byte stores
// per thread was measured slower: each store instruction then fills only half of every sector.)
__global__ void __launch_bounds__(256)
dequant_s8_kernel(const DequantArgs args, size_t count)
{
    const int8_t* w = reinterpret_cast<const int8_t*>(args.w[blockIdx.y]);
    __half* out = args.out[blockIdx.y];
    const size_t stride = (size_t)gridDim.x * blockDim.x * 8;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < count; i += stride) {
        // count % 8 == 0 and 8-byte aligned bases on this path
        const int2 raw = *reinterpret_cast<const int2*>(w + i);
        const int8_t* b = reinterpret_cast<const int8_t*>(&raw);
        __half2 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            h[j] = __halves2half2(__int2half_rn((int)b[2 * j]), __int2half_rn((int)b[2 * j + 1]));
        *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<uint4*>(h);
    }
}

bool dq_gemm_fast_path_ok(int wfmt, const void* x, const DqProblem* probs, int num_probs,
                          bool out_f16, uint32_t m, uint32_t n, uint32_t k)
{
    (void)m;
    if (num_probs < 1 || num_probs > f16g::MAX_PROBS)
        return false;
    if (n % 8 != 0 || k % 8 != 0 || (uintptr_t)x % 16 != 0)
        return false;
    for (int i = 0; i < num_probs; ++i) {
        if ((uintptr_t)probs[i].w % 16 != 0 || (uintptr_t)probs[i].out % 16 != 0)
            return false;
        if (probs[i].col_scale != nullptr && (uintptr_t)probs[i].col_scale % 16 != 0)
            return false;
        if (wfmt == WFMT_S4_PACKED && (k % 128 != 0 || probs[i].scales == nullptr))
            return false;
    }
    (void)out_f16;
    return true;
}

size_t dq_gemm_workspace_bytes(int num_probs, uint32_t n, uint32_t k)
{
    return (size_t)num_probs * (((size_t)k * n * sizeof(__half) + 255) & ~(size_t)255);
}

template <bool PAIR, bool OUT_F16>
static cudaError_t launch_f16_gemm(const DeviceCtx& ctx, const f16g::TensorMaps& maps,
                                   const f16g::Params& p, cudaStream_t stream)
{
    using namespace f16g;
    using C = Cfg<PAIR>;
    static bool attr_set[64] = {};
    cudaError_t err;
    if (!attr_set[ctx.device]) {
        err = cudaFuncSetAttribute(f16_gemm_kernel<PAIR, OUT_F16>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (err != cudaSuccess)
            return err;
        attr_set[ctx.device] = true;
    }
    const uint32_t tiles =
        ((p.m + C::BM - 1) / C::BM) * ((p.n + BN - 1) / BN) * p.num_probs;
    const uint32_t max_workers = PAIR ? (uint32_t)ctx.num_sms / 2 : (uint32_t)ctx.num_sms;
    const uint32_t workers = tiles < max_workers ? tiles : max_workers;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(PAIR ? workers * 2 : workers);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, f16_gemm_kernel<PAIR, OUT_F16>, maps, p);
}

cudaError_t launch_dequant_s4(const uint32_t* w_packed, const __half* scales, __half* out,
                              uint32_t n, uint32_t k, cudaStream_t stream)
{
    DequantArgs da = {};
    da.w[0] = w_packed;
    da.scales[0] = scales;
    da.out[0] = out;
    launch_dequant_s4_any(da, n, k, 1, stream);
    return cudaGetLastError();
}

cudaError_t launch_dq_gemm(const DeviceCtx& ctx, int wfmt, const __half* x, const DqProblem* probs,
                           int num_probs, bool out_f16, bool post_scale, uint32_t m, uint32_t n,
                           uint32_t k, void* dq_workspace, cudaStream_t stream,
                           const OutputCopies* copies, bool silu_gate)
{
    using namespace f16g;
    const size_t per = dq_gemm_workspace_bytes(1, n, k);
    DequantArgs da = {};
    for (int i = 0; i < num_probs; ++i) {
        da.w[i] = probs[i].w;
        da.scales[i] = probs[i].scales;
        da.out[i] = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(dq_workspace) + per * i);
    }
    if (wfmt == WFMT_F16) {
        for (int i = 0; i < num_probs; ++i)  // the weights are the f16 operand already
            da.out[i] = const_cast<__half*>(reinterpret_cast<const __half*>(probs[i].w));
    } else if (wfmt == WFMT_S4_PACKED) {
        launch_dequant_s4_any(da, n, k, num_probs, stream);
    } else {
        const size_t count = (size_t)k * n;
        dim3 grid((unsigned)((count / 8 + 255) / 256 < 4096 ? (count / 8 + 255) / 256 : 4096), num_probs);
        dequant_s8_kernel<<<grid, 256, 0, stream>>>(da, count);
    }
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
        return err;

    // KAIO_B200_PAIR=0/1 forces single-CTA / CTA-pair tiles (tuning aid); default: pairs for M > 128
    bool pair = m > 128;
    if (const char* e = getenv("KAIO_B200_PAIR"))
        pair = (e[0] == '1');
    TensorMaps maps;
    err = encode_tensor_map_2d(&maps.x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, k, m,
                               (uint64_t)k * 2, BK, BM_CTA, CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess)
        return err;
    for (int i = 0; i < MAX_PROBS; ++i) {
        const int j = i < num_probs ? i : 0;
        err = encode_tensor_map_2d(&maps.w[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, da.out[j], n, k,
                                   (uint64_t)n * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
        if (err != cudaSuccess)
            return err;
    }
    // output maps: one per projection, or one per destination of the single output.  A destination
    // map covers only this call's n columns of a wider row (row stride ld), so TMA clips at the
    // shard's edge.
    const uint32_t num_copies = copies ? copies->count : 1u;
    for (int i = 0; i < MAX_OUT_MAPS; ++i) {
        void* base;
        uint64_t ld;
        if (copies) {
            base = copies->ptrs[(uint32_t)i < num_copies ? i : 0];
            ld = copies->ld;
        } else {
            base = probs[i < num_probs ? i : 0].out;
            ld = n;
        }
        // in the scatter form a destination holds one block of scatter_cols columns
        uint64_t width = (copies && copies->scatter_cols) ? copies->scatter_cols : n;
        if (silu_gate) {  // the activation is half as wide as the two interleaved projections
            width = n / 2;
            ld = n / 2;
        }
        if (out_f16)
            err = encode_tensor_map_2d(&maps.out[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, width,
                                       m, ld * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
        else
            err = encode_tensor_map_2d(&maps.out[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, width,
                                       m, ld * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
        if (err != cudaSuccess)
            return err;
    }
    Params p = {};
    for (int i = 0; i < num_probs; ++i) {
        p.probs[i].col_scale = probs[i].col_scale;
        p.probs[i].scale = probs[i].scale;
    }
    p.num_probs = (uint32_t)num_probs;
    p.copies = num_copies;
    p.scatter_cols = copies ? copies->scatter_cols : 0u;
    p.m = m;
    p.n = n;
    p.k = k;
    p.post_scale = post_scale ? 1 : 0;
    p.nt_rot = copies ? (copies->start_col / BN) % ((n + BN - 1) / BN) : 0u;
    p.mc_out = (copies && !copies->scatter_cols && !silu_gate) ? copies->multicast : nullptr;
    p.mc_ld = copies ? copies->ld : 0;
    p.silu_gate = silu_gate ? 1 : 0;
    p.status = ctx.status;
    if (pair)
        return out_f16 ? launch_f16_gemm<true, true>(ctx, maps, p, stream)
                       : launch_f16_gemm<true, false>(ctx, maps, p, stream);
    return out_f16 ? launch_f16_gemm<false, true>(ctx, maps, p, stream)
                   : launch_f16_gemm<false, false>(ctx, maps, p, stream);
}

}  // namespace kaio
