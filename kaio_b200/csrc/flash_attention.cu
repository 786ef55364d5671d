// Flash attention forward for head_dim 128 on the 5th-generation tensor cores:
//   out = softmax(Q K^T / sqrt(d) [+ causal mask j > i]) V,  f16 in, f32 accumulation,
//   f32 or f16 out, any seq_k (online softmax over 128-row KV blocks).
//
// Replaces KAIO's `attention_tc` / `attention_tc_causal` kernel
// (kaio-ops/src/attention_tc_kernel.rs:1454-2233: one warp per 16 query rows, the whole score row
// in shared memory, seq_k <= 384) and adds the batched multi-head form that reads Q/K/V in place
// from [batch*seq, heads*128] projection outputs.
//
// Persistent: one CTA per SM walks the work items (batch, head, 256 query rows), heaviest first
// inside groups of (batch, head) pairs whose K and V fit the L2 together (see make_item); Q loads,
// the fill of the K/V ring and the first scores of the next item overlap the softmax tail and the
// output of the current one, and tensor memory and barriers are set up once.
// An item = two query tiles of 128 rows; 320 threads:
//   warp 0     TMA producer: Q once (four [128][64] boxes), then K and V blocks ([128 kv][128 d] as
//              two 64-column boxes each) through a 2-stage ring; 128-byte swizzle.
//   warp 1     MMA issuer (converged warp, elected lane), for tile t in {0, 1}:
//                S_t  = Q_t K_j^T   tcgen05.mma kind::f16 M128 N128 K16 x8, Q and K from shared
//                                   memory (both K-major), S_t in tensor memory
//                O_t += P_t V_j     M128 N128 K16 x8, P_t (f16) from TENSOR MEMORY (it overwrites
//                                   the first 64 columns of S_t), V from shared memory read
//                                   MN-major (d contiguous), O_t in tensor memory
//              issue order per block: PV_0(j), QK_0(j+1), PV_1(j), QK_1(j+1) -- while one tile's
//              softmax runs, the tensor pipe works on the other tile, and serving the tiles in
//              turn keeps them half a period apart (with one issuer per tile the two tiles
//              fell into step: both in softmax, then both queueing for the tensor pipe).  P is
//              handed over in two halves (kv 0-63, 64-127): the first four P V steps run while
//              the softmax warps still exponentiate the second half.
//   warps 2-5  softmax of tile 0, warps 6-9 softmax of tile 1: thread = query row.  tcgen05.ld of
//              the score row, block max (four independent chains), running reference with lazy
//              rescale: P = 2^(s - ref) may grow to 2^15 before O and the row sum are rescaled,
//              and a new reference is set 2^8 above the max seen, so a row's max can rise by
//              2^23 before the next rescale; when any row of a warp must rescale, every row of
//              the warp moves its reference up to its own running max (the pass over O costs
//              the same for one row as for 32), which makes such passes rare.
//              ex2(s * log2(e)/sqrt(d) - ref) with the scale-and-subtract and the row sum as
//              packed f32x2 instructions (the warps are bound by instruction issue), P packed
//              to f16 and stored to tensor memory; at the end O / sum -> global.  Two warps per
//              scheduler hide each other's dependent chains; a single softmax warp-group left
//              the tensor pipe 27 % busy.
#include "common.cuh"
#include "kernels.h"

namespace kaio {
namespace fa {

constexpr int BQ = 128;   // query rows per tile (two tiles per work item)
constexpr int BKV = 128;  // key/value rows per block
constexpr int D = 128;    // head dim
constexpr int KV_STAGES = 2;
constexpr int Q_TILE_BYTES = BQ * D * 2;      // 32 KiB: two [128][64] sub-tiles
constexpr int Q_BYTES = 2 * Q_TILE_BYTES;     // two query tiles per CTA
constexpr int KV_TILE_BYTES = BKV * D * 2;    // 32 KiB each for K and V
constexpr int STAGE_BYTES = 2 * KV_TILE_BYTES;  // K | V
constexpr int SUB_BYTES = 128 * 128;          // one [128 rows][64 f16] sub-tile
constexpr int NUM_THREADS = 320;
constexpr int SMEM_BYTES = 1024 + Q_BYTES + KV_STAGES * STAGE_BYTES + 256;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_S = 0;      // per tile: 128 columns of f32 scores; P (f16 pairs) reuses the first 64
constexpr uint32_t TMEM_O = 256;    // per tile: 128 columns (f32 output accumulator)

constexpr uint32_t IDESC_QK = make_idesc(1, 0, 0, /*a K-major*/ 0, /*b K-major*/ 0, BQ, BKV);
constexpr uint32_t IDESC_PV = make_idesc(1, 0, 0, /*a K-major*/ 0, /*b MN-major*/ 1, BQ, D);
// lazy rescale: P = 2^(s - ref) <= 2^RESCALE_WINDOW (f16 holds 2^15); a new reference is
// REF_MARGIN above the max seen so far (scores 2^-6 below the max still keep all f16 bits, and
// what lies below is rounded to within 2^-17 of the largest term)
constexpr float RESCALE_WINDOW = 15.0f;
constexpr float REF_MARGIN = 8.0f;

enum : uint32_t {
    SITE_Q_FULL = 1, SITE_KV_FULL = 2, SITE_KV_EMPTY = 3, SITE_S_FULL = 4, SITE_P_FULL = 5,
    SITE_PV_DONE = 6
};

struct Params {
    void* out;
    uint32_t batch, heads, seq_q, seq_k;
    uint64_t o_row, o_head, o_batch;  // element strides of the output
    float scale_log2;                 // log2(e) / sqrt(d)
    int causal;
    int out_f16;
    uint32_t* status;
};

struct TensorMaps {
    CUtensorMap q, k, v;
};

// One work item = (batch, head, 256 query rows).  The (batch, head) pairs are taken in groups of
// gridDim.x / 4 -- few enough that their K and V (1 MB per pair at seq 2048) stay in the L2
// together -- and inside a group the items are numbered heaviest first (causal: the last query block
// of every pair, then the one before, ...).  With eight query blocks per pair a group is two whole
// rounds of the grid, so the snake assignment (see item_of) gives every CTA the same total per
// group, and the query blocks of a pair run within two rounds of each other: K and V come from
// DRAM about once (numbered heaviest first over ALL pairs they were fetched three times: 1.27 GB
// instead of 0.40 GB at config 4, and 326 us instead of 300).
struct Item {
    uint32_t b, h, q0;
    uint32_t nkv0, nkv1;  // KV blocks each query tile attends to (0 for a tile beyond seq_q)
    uint32_t num_kv;
};

__device__ __forceinline__ Item make_item(const Params& p, uint32_t it)
{
    const uint32_t num_qb = (p.seq_q + 2 * BQ - 1) / (2 * BQ);
    const uint32_t bh_count = p.batch * p.heads;
    const uint32_t gsz = gridDim.x >= 4 ? gridDim.x / 4 : 1u;  // pairs per group
    const uint32_t groups = (bh_count + gsz - 1) / gsz;
    uint32_t grp = it / (gsz * num_qb);
    grp = grp < groups - 1 ? grp : groups - 1;
    const uint32_t rem = it - grp * gsz * num_qb;
    const uint32_t gcount = grp == groups - 1 ? bh_count - grp * gsz : gsz;  // the last group is short
    const uint32_t tier = rem / gcount;
    const uint32_t bh = grp * gsz + rem - tier * gcount;
    Item im;
    im.b = bh / p.heads;
    im.h = bh - im.b * p.heads;
    im.q0 = (num_qb - 1 - tier) * 2 * BQ;
    uint32_t nkv[2];
#pragma unroll
    for (uint32_t t = 0; t < 2; ++t) {
        const uint32_t tq0 = im.q0 + t * BQ;
        uint32_t kv_end = p.seq_k;
        if (p.causal) {
            const uint32_t lim = tq0 + BQ;  // columns j <= i < tq0 + BQ
            kv_end = lim < kv_end ? lim : kv_end;
        }
        nkv[t] = tq0 < p.seq_q ? (kv_end + BKV - 1) / BKV : 0u;
    }
    im.nkv0 = nkv[0];
    im.nkv1 = nkv[1];
    im.num_kv = nkv[0] > nkv[1] ? nkv[0] : nkv[1];
    return im;
}

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed f32 pairs (sm_100: one instruction, two f32 operations) and the three-input max: the
// softmax warps are bound by instruction issue, not by a pipe.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi)
{
    uint64_t v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}

__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ float max3_f32(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
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

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
            taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
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


// Three warps share a scheduler's 16 K registers: at most 168 per thread.
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_attention_kernel(const __grid_constant__ TensorMaps maps, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t q_smem = smem_base;
    const uint32_t kv_smem = smem_base + Q_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + Q_BYTES + KV_STAGES * STAGE_BYTES);
    const uint32_t bar_base = smem_base + Q_BYTES + KV_STAGES * STAGE_BYTES;
    const uint32_t q_full = bar_base;
    auto kv_full = [&](uint32_t s) { return bar_base + 8u * (1 + s); };
    auto kv_empty = [&](uint32_t s) { return bar_base + 8u * (3 + s); };
    auto s_full = [&](uint32_t b) { return bar_base + 8u * (5 + b); };
    auto p_lo = [&](uint32_t b) { return bar_base + 8u * (7 + b); };   // P of kv 0-63 stored
    auto p_hi = [&](uint32_t b) { return bar_base + 8u * (9 + b); };   // P of kv 64-127 stored
    auto pv_done = [&](uint32_t b) { return bar_base + 8u * (11 + b); };
    const uint32_t q_empty = bar_base + 8u * 13;  // the item's last Q K^T has read Q
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 14);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    // Persistent CTA: all barrier phases run on through the items (counters, not item-local
    // indices, give the parities); K/V of the next item stream in behind the current one's, its Q
    // lands while the softmax warps finish and write out the current item.
    const uint32_t total_items = ((p.seq_q + 2 * BQ - 1) / (2 * BQ)) * p.batch * p.heads;
    // Round r hands item r * G + c to CTA c in even rounds and to CTA G - 1 - c in odd ones: with the
    // items sorted by weight the CTAs' totals stay within ~1 % of each other (plain round robin:
    // 6 % at config 4), as good as a greedy assignment.
    auto item_of = [&](uint32_t round) {
        const uint32_t c = (round & 1u) ? gridDim.x - 1 - blockIdx.x : blockIdx.x;
        return round * gridDim.x + c;
    };

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (uint32_t s = 0; s < KV_STAGES; ++s) {
            mbar_init(kv_full(s), 1);
            mbar_init(kv_empty(s), 1);
        }
        for (uint32_t i = 0; i < 2; ++i) {
            mbar_init(s_full(i), 1);
            mbar_init(p_lo(i), 4);  // one arrive per softmax warp of the tile
            mbar_init(p_hi(i), 4);
            mbar_init(pv_done(i), 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&maps.q);
        tma_prefetch_desc(&maps.k);
        tma_prefetch_desc(&maps.v);
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
        uint32_t kvc = 0;  // KV blocks loaded so far (all items): stage kvc & 1, use kvc >> 1
        bool ok = true;
        for (uint32_t round = 0; ok && round * gridDim.x < total_items; ++round) {
            const uint32_t it = item_of(round);
            if (it >= total_items)
                continue;  // the last round is not full
            const uint32_t n_item = round;  // every earlier round held an item for this CTA
            const Item im = make_item(p, it);
            const int32_t col0 = (int32_t)(im.h * D);
            const int32_t q_row = (int32_t)(im.b * p.seq_q + im.q0);
            // Q is single-buffered: the previous item's last Q K^T must have read it
            if (!mbar_wait_bounded(q_empty, (n_item & 1u) ^ 1u, abort_flag, p.status, SITE_Q_FULL,
                                   KERNEL_FLASH_ATTN))
                break;
            if (elect_one()) {
                mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    tma_load_2d(q_smem + t * Q_TILE_BYTES, &maps.q, q_full, col0, q_row + t * BQ);
                    tma_load_2d(q_smem + t * Q_TILE_BYTES + SUB_BYTES, &maps.q, q_full, col0 + 64,
                                q_row + t * BQ);
                }
            }
            __syncwarp();
            for (uint32_t j = 0; j < im.num_kv; ++j, ++kvc) {
                const uint32_t s = kvc & 1u, ph = (kvc >> 1) & 1u;
                if (!mbar_wait_bounded(kv_empty(s), ph ^ 1u, abort_flag, p.status, SITE_KV_EMPTY,
                                       KERNEL_FLASH_ATTN)) {
                    ok = false;
                    break;
                }
                if (elect_one()) {
                    const uint32_t stage = kv_smem + s * STAGE_BYTES;
                    const int32_t kv_row = (int32_t)(im.b * p.seq_k + j * BKV);
                    mbar_expect_tx(kv_full(s), STAGE_BYTES);
                    tma_load_2d(stage, &maps.k, kv_full(s), col0, kv_row);
                    tma_load_2d(stage + SUB_BYTES, &maps.k, kv_full(s), col0 + 64, kv_row);
                    tma_load_2d(stage + KV_TILE_BYTES, &maps.v, kv_full(s), col0, kv_row);
                    tma_load_2d(stage + KV_TILE_BYTES + SUB_BYTES, &maps.v, kv_full(s), col0 + 64,
                                kv_row);
                }
                __syncwarp();
            }
        }
        if (*abort_flag)
            for (uint32_t spin = 0; spin < 2000; ++spin)
                __nanosleep(100);
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // g = running number of the KV block (all items): it selects the stage
        auto issue_qk = [&](uint32_t t, uint32_t g) {
            // S_t = Q_t K^T : 8 steps of 16 along d; sub-tile d/64, 32 bytes inside the row
            const uint32_t stage = kv_smem + (g & 1u) * STAGE_BYTES;
            const uint32_t qt = q_smem + t * Q_TILE_BYTES;
            const uint32_t d_tmem = tmem_base + TMEM_S + t * BKV;
            if (elect_one()) {
#pragma unroll
                for (uint32_t kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * SUB_BYTES + (kk & 3u) * 32;
                    umma_f16(d_tmem, make_smem_desc_sw128(qt + off, 16, 1024),
                             make_smem_desc_sw128(stage + off, 16, 1024), IDESC_QK,
                             kk != 0 ? 1u : 0u);
                }
                umma_commit(s_full(t));
            }
            __syncwarp();
        };
        // O_t += P_t V, steps [k0, k0 + 4) of 16 along kv; P in tensor memory (8 columns per
        // step), V MN-major: 16 kv rows of 128 bytes per step, the two 64-column halves
        // SUB_BYTES apart.  j = block inside the item (its first P V overwrites O_t).
        auto issue_pv = [&](uint32_t t, uint32_t j, uint32_t g, uint32_t k0, bool last,
                            bool last_reader) {
            const uint32_t v_smem = kv_smem + (g & 1u) * STAGE_BYTES + KV_TILE_BYTES;
            const uint32_t p_tmem = tmem_base + TMEM_S + t * BKV;
            if (elect_one()) {
#pragma unroll
                for (uint32_t kk = k0; kk < k0 + BKV / 32; ++kk) {
                    umma_f16_ts(tmem_base + TMEM_O + t * D, p_tmem + kk * 8,
                                make_smem_desc_sw128(v_smem + kk * 2048, SUB_BYTES, 1024), IDESC_PV,
                                (j | kk) != 0 ? 1u : 0u);
                }
                if (last) {
                    umma_commit(pv_done(t));
                    if (last_reader)
                        umma_commit(kv_empty(g & 1u));  // this K and V block have been consumed
                }
            }
            __syncwarp();
        };
        uint32_t kvc = 0;           // KV blocks of the items before this one
        uint32_t done[2] = {0, 0};  // blocks each tile's softmax has handed over so far
        bool ok = true;
        for (uint32_t round = 0; ok && round * gridDim.x < total_items; ++round) {
            const uint32_t it = item_of(round);
            if (it >= total_items)
                continue;  // the last round is not full
            const uint32_t n_item = round;  // every earlier round held an item for this CTA
            const Item im = make_item(p, it);
            const uint32_t nkv[2] = {im.nkv0, im.nkv1};
            ok = mbar_wait_bounded(q_full, n_item & 1u, abort_flag, p.status, SITE_Q_FULL,
                                   KERNEL_FLASH_ATTN);
            if (ok && im.num_kv > 0) {
                ok = mbar_wait_bounded(kv_full(kvc & 1u), (kvc >> 1) & 1u, abort_flag, p.status,
                                       SITE_KV_FULL, KERNEL_FLASH_ATTN);
                if (ok) {
                    tc_fence_after_sync();
                    if (nkv[0] > 0)
                        issue_qk(0, kvc);
                    if (nkv[1] > 0)
                        issue_qk(1, kvc);
                }
            }
            if (ok && im.num_kv <= 1) {
                if (elect_one())
                    umma_commit(q_empty);  // no further Q K^T in this item
                __syncwarp();
            }
            for (uint32_t j = 0; ok && j < im.num_kv; ++j) {
                const uint32_t g = kvc + j;
                bool next_ready = false;
#pragma unroll
                for (uint32_t t = 0; t < 2; ++t) {
                    if (j < nkv[t]) {
                        // steps 0-3 go as soon as the first half of P is in
                        if (!mbar_wait_bounded(p_lo(t), done[t] & 1u, abort_flag, p.status,
                                               SITE_P_FULL, KERNEL_FLASH_ATTN)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        issue_pv(t, j, g, 0, false, false);
                        if (!mbar_wait_bounded(p_hi(t), done[t] & 1u, abort_flag, p.status,
                                               SITE_P_FULL, KERNEL_FLASH_ATTN)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        issue_pv(t, j, g, BKV / 32, true, (t == 1) || (j >= nkv[1]));
                        ++done[t];
                    }
                    // scores of the next block for this tile, issued behind its P V so the other
                    // tile's softmax overlaps them (in-order execution on the tensor pipe makes
                    // the overwrite of P_t by S_t safe)
                    if (j + 1 < nkv[t]) {
                        if (!next_ready) {
                            if (!mbar_wait_bounded(kv_full((g + 1) & 1u), ((g + 1) >> 1) & 1u,
                                                   abort_flag, p.status, SITE_KV_FULL,
                                                   KERNEL_FLASH_ATTN)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            next_ready = true;
                        }
                        issue_qk(t, g + 1);
                    }
                }
                // the item's last Q K^T were issued in the step before the last one
                if (ok && j + 2 == im.num_kv) {
                    if (elect_one())
                        umma_commit(q_empty);
                    __syncwarp();
                }
            }
            kvc += im.num_kv;
        }
    } else {
        // ------------------------------------------------------------ softmax + epilogue
        const uint32_t t = (warp - 2) >> 2;  // query tile of this warp-group
        const uint32_t quarter = warp & 3u;
        const uint32_t lane_sel = (quarter * 32u) << 16;
        const uint32_t row_local = quarter * 32 + lane;
        const uint32_t s_tmem = tmem_base + TMEM_S + t * BKV + lane_sel;
        const uint32_t o_tmem = tmem_base + TMEM_O + t * D + lane_sel;
        uint32_t cnt = 0;  // blocks of this tile processed so far (all items): barrier parities
        bool ok = true;
        for (uint32_t round = 0; ok && round * gridDim.x < total_items; ++round) {
        const uint32_t it = item_of(round);
        if (it >= total_items)
            continue;  // the last round is not full
        const Item im = make_item(p, it);
        const uint32_t b = im.b, h = im.h, q0 = im.q0;
        const uint32_t row = q0 + t * BQ + row_local;  // query index inside this (batch, head)
        const uint32_t my_kv = t ? im.nkv1 : im.nkv0;
        float m_ref = 0.0f;  // reference subtracted in the exponent (log2 units)
        float m_run = -INFINITY;  // running max of the scaled scores
        float l_sum = 0.0f;
        for (uint32_t j = 0; j < my_kv; ++j, ++cnt) {
            if (!mbar_wait_bounded(s_full(t), cnt & 1u, abort_flag, p.status, SITE_S_FULL,
                                   KERNEL_FLASH_ATTN)) {
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t col_base = j * BKV;
            // columns allowed for this row: j_abs < seq_k and (causal) j_abs <= row
            uint32_t col_lim = p.seq_k;
            if (p.causal && row + 1 < col_lim)
                col_lim = row + 1;
            const bool need_mask = col_base + BKV > col_lim;
            // only the diagonal block (causal) and the seq_k tail need per-element masks; the
            // test is made warp-uniform so the common blocks run mask-free code
            const bool blk_mask = __any_sync(0xffffffffu, need_mask);

            // ---- the whole score row (128 f32) comes into registers once: four loads in flight,
            // one wait; both softmax passes then run on registers
            uint32_t r0[32], r1[32], r2[32], r3[32];
            tmem_ld_32x32b_x32(s_tmem + 0, r0);
            tmem_ld_32x32b_x32(s_tmem + 32, r1);
            tmem_ld_32x32b_x32(s_tmem + 64, r2);
            tmem_ld_32x32b_x32(s_tmem + 96, r3);
            tmem_ld_wait();
            if (blk_mask) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (col_base + i >= col_lim)
                        r0[i] = 0xff800000u;  // -inf -> p = 0
                    if (col_base + 32 + i >= col_lim)
                        r1[i] = 0xff800000u;
                    if (col_base + 64 + i >= col_lim)
                        r2[i] = 0xff800000u;
                    if (col_base + 96 + i >= col_lim)
                        r3[i] = 0xff800000u;
                }
            }
            // ---- pass 1: block maximum of the raw scores (the scale is positive: scale after)
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {  // four independent chains, two scores per instruction
                mx0 = max3_f32(mx0, __uint_as_float(r0[i]), __uint_as_float(r0[i + 1]));
                mx1 = max3_f32(mx1, __uint_as_float(r1[i]), __uint_as_float(r1[i + 1]));
                mx2 = max3_f32(mx2, __uint_as_float(r2[i]), __uint_as_float(r2[i + 1]));
                mx3 = max3_f32(mx3, __uint_as_float(r3[i]), __uint_as_float(r3[i + 1]));
            }
            const float m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
            // ---- lazy rescale: keep the old reference while P = 2^(s - m_ref) stays inside f16
            // (the row sum and O are f32)
            float alpha = 1.0f;
            bool rescale = false;
            if (j == 0) {
                m_run = m_blk;
                m_ref = (m_blk == -INFINITY) ? 0.0f : m_blk + REF_MARGIN;
            } else {
                m_run = fmaxf(m_run, m_blk);
                rescale = __any_sync(0xffffffffu, m_blk > m_ref + RESCALE_WINDOW);
                if (rescale && m_run + REF_MARGIN > m_ref) {
                    // the pass over O is made for the whole warp: every row uses it to move its
                    // reference up to its own running max
                    alpha = ex2_approx(m_ref - (m_run + REF_MARGIN));
                    m_ref = m_run + REF_MARGIN;
                    l_sum *= alpha;
                }
            }
            // ---- pass 2: p = 2^(s * scale - m_ref), row sum, f16 pairs into tensor memory.  P
            // overwrites the first 64 columns of S, which are all in registers by now.
            // two scores per FMA and per add (packed f32x2); the exponentials stay scalar (MUFU)
            uint64_t lsa = 0, lsb = 0;  // packed row-sum accumulators (two chains)
            const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
            const uint64_t nref2 = pack_f32x2(-m_ref, -m_ref);
            auto exp_chunk = [&](const uint32_t (&r)[32], uint32_t c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float x0, x1, x2, x3;
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                                           scale2, nref2), x0, x1);
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                                           scale2, nref2), x2, x3);
                    const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                    const float p2 = ex2_approx(x2), p3 = ex2_approx(x3);
                    lsa = add_f32x2(lsa, pack_f32x2(p0, p1));
                    lsb = add_f32x2(lsb, pack_f32x2(p2, p3));
                    const __half2 h01 = __floats2half2_rn(p0, p1);
                    const __half2 h23 = __floats2half2_rn(p2, p3);
                    pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h01);
                    pk[(i >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&h23);
                }
                tmem_st_32x32b_x16(s_tmem + c * 16, pk);
            };
            exp_chunk(r0, 0);
            exp_chunk(r1, 1);
            if (!rescale) {
                // first half of P handed over: its P V steps run while the second half is computed
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(p_lo(t));
                }
                // keep the second half's arithmetic behind the hand-over: without a dependence
                // the compiler moves it in front of the store wait and the arrive comes late
#pragma unroll
                for (int i = 0; i < 32; i += 16) {
                    asm volatile("" : "+r"(r2[i]), "+r"(r2[i + 1]), "+r"(r2[i + 2]), "+r"(r2[i + 3]),
                                      "+r"(r2[i + 4]), "+r"(r2[i + 5]), "+r"(r2[i + 6]), "+r"(r2[i + 7]),
                                      "+r"(r2[i + 8]), "+r"(r2[i + 9]), "+r"(r2[i + 10]), "+r"(r2[i + 11]),
                                      "+r"(r2[i + 12]), "+r"(r2[i + 13]), "+r"(r2[i + 14]), "+r"(r2[i + 15])
                                 :: "memory");
                    asm volatile("" : "+r"(r3[i]), "+r"(r3[i + 1]), "+r"(r3[i + 2]), "+r"(r3[i + 3]),
                                      "+r"(r3[i + 4]), "+r"(r3[i + 5]), "+r"(r3[i + 6]), "+r"(r3[i + 7]),
                                      "+r"(r3[i + 8]), "+r"(r3[i + 9]), "+r"(r3[i + 10]), "+r"(r3[i + 11]),
                                      "+r"(r3[i + 12]), "+r"(r3[i + 13]), "+r"(r3[i + 14]), "+r"(r3[i + 15])
                                 :: "memory");
                }
            }
            exp_chunk(r2, 2);
            exp_chunk(r3, 3);
            {
                float a0, a1, b0, b1;
                unpack_f32x2(lsa, a0, a1);
                unpack_f32x2(lsb, b0, b1);
                l_sum += (a0 + a1) + (b0 + b1);
            }
            tmem_st_wait();
            if (rescale) {
                // Some row of this warp moved its reference: O_t (last written by the P V of block
                // j-1, complete since S_j was issued behind them) is scaled before any P V of this
                // block may start, so this block hands both halves over at the end.  The score
                // registers are free by now: four loads in flight.
                if (!mbar_wait_bounded(pv_done(t), (cnt - 1) & 1u, abort_flag, p.status, SITE_PV_DONE,
                                       KERNEL_FLASH_ATTN)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                tmem_ld_32x32b_x32(o_tmem + 0, r0);
                tmem_ld_32x32b_x32(o_tmem + 32, r1);
                tmem_ld_32x32b_x32(o_tmem + 64, r2);
                tmem_ld_32x32b_x32(o_tmem + 96, r3);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    r0[i] = __float_as_uint(__uint_as_float(r0[i]) * alpha);
                    r1[i] = __float_as_uint(__uint_as_float(r1[i]) * alpha);
                    r2[i] = __float_as_uint(__uint_as_float(r2[i]) * alpha);
                    r3[i] = __float_as_uint(__uint_as_float(r3[i]) * alpha);
                }
                tmem_st_32x32b_x32(o_tmem + 0, r0);
                tmem_st_32x32b_x32(o_tmem + 32, r1);
                tmem_st_32x32b_x32(o_tmem + 64, r2);
                tmem_st_32x32b_x32(o_tmem + 96, r3);
                tmem_st_wait();
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (rescale)
                    mbar_arrive(p_lo(t));
                mbar_arrive(p_hi(t));
            }
        }
        // ---- epilogue: O / l -> global
        if (ok && my_kv > 0)
            ok = mbar_wait_bounded(pv_done(t), (cnt - 1) & 1u, abort_flag, p.status, SITE_PV_DONE,
                                   KERNEL_FLASH_ATTN);
        if (ok && q0 + t * BQ < p.seq_q) {
            tc_fence_after_sync();
            const float inv = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
            const size_t obase = (size_t)b * p.o_batch + (size_t)h * p.o_head + (size_t)row * p.o_row;
#pragma unroll 1
            for (uint32_t c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                if (my_kv > 0) {
                    tmem_ld_32x32b_x32(o_tmem + c * 32, r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        r[i] = 0;
                }
                if (row < p.seq_q) {
                    if (p.out_f16) {
                        __half* dst = reinterpret_cast<__half*>(p.out) + obase + c * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 pk;
                            __half2 h0 = __floats2half2_rn(__uint_as_float(r[i]) * inv,
                                                           __uint_as_float(r[i + 1]) * inv);
                            __half2 h1 = __floats2half2_rn(__uint_as_float(r[i + 2]) * inv,
                                                           __uint_as_float(r[i + 3]) * inv);
                            __half2 h2 = __floats2half2_rn(__uint_as_float(r[i + 4]) * inv,
                                                           __uint_as_float(r[i + 5]) * inv);
                            __half2 h3 = __floats2half2_rn(__uint_as_float(r[i + 6]) * inv,
                                                           __uint_as_float(r[i + 7]) * inv);
                            pk.x = *reinterpret_cast<uint32_t*>(&h0);
                            pk.y = *reinterpret_cast<uint32_t*>(&h1);
                            pk.z = *reinterpret_cast<uint32_t*>(&h2);
                            pk.w = *reinterpret_cast<uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(dst + i) = pk;
                        }
                    } else {
                        float* dst = reinterpret_cast<float*>(p.out) + obase + c * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(dst + i) = make_float4(
                                __uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv,
                                __uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                    }
                }
            }
        }
        // the reads of O_t are complete before this warp arrives for the next item's first block
        tc_fence_before_sync();
        }  // items
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<TMEM_COLS>(tmem_base);
    }
}

}  // namespace fa


bool flash_attention_ok(const AttnParams& p)
{
    if (p.d_k != 128 || p.d_v != 128)
        return false;
    const uint64_t strides[] = {p.q_row, p.k_row, p.v_row, p.o_row, p.q_head, p.k_head, p.v_head,
                                p.o_head, p.q_batch, p.k_batch, p.v_batch, p.o_batch};
    for (uint64_t s : strides)
        if (s % 8 != 0)
            return false;
    if ((uintptr_t)p.q % 16 || (uintptr_t)p.k % 16 || (uintptr_t)p.v % 16 || (uintptr_t)p.out % 16)
        return false;
    // the TMA view is [batch*seq rows, heads*128 columns] with one row stride: batch b starts at
    // row b*seq and head h at column h*128
    if (p.heads > 1 && (p.q_head != 128 || p.k_head != 128 || p.v_head != 128))
        return false;
    if (p.batch > 1 &&
        (p.q_batch != (uint64_t)p.seq_q * p.q_row || p.k_batch != (uint64_t)p.seq_k * p.k_row ||
         p.v_batch != (uint64_t)p.seq_k * p.v_row))
        return false;
    if (p.q_row < (uint64_t)p.heads * 128 || p.k_row < (uint64_t)p.heads * 128 ||
        p.v_row < (uint64_t)p.heads * 128)
        return false;
    return true;
}

cudaError_t launch_flash_attention(const DeviceCtx& ctx, const AttnParams& ap, cudaStream_t stream)
{
    using namespace fa;
    TensorMaps maps;
    const uint64_t width = (uint64_t)ap.heads * D;
    cudaError_t err = encode_tensor_map_2d(&maps.q, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ap.q, width,
                                           (uint64_t)ap.batch * ap.seq_q, ap.q_row * 2, 64, BQ,
                                           CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess)
        return err;
    err = encode_tensor_map_2d(&maps.k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ap.k, width,
                               (uint64_t)ap.batch * ap.seq_k, ap.k_row * 2, 64, BKV,
                               CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess)
        return err;
    err = encode_tensor_map_2d(&maps.v, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ap.v, width,
                               (uint64_t)ap.batch * ap.seq_k, ap.v_row * 2, 64, BKV,
                               CU_TENSOR_MAP_SWIZZLE_128B);
    if (err != cudaSuccess)
        return err;
    Params p = {};
    p.out = ap.out;
    p.batch = ap.batch;
    p.heads = ap.heads;
    p.seq_q = ap.seq_q;
    p.seq_k = ap.seq_k;
    p.o_row = ap.o_row;
    p.o_head = ap.o_head;
    p.o_batch = ap.o_batch;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)D);
    p.causal = ap.causal;
    p.out_f16 = ap.out_f16;
    p.status = ctx.status;
    static bool attr_set[64] = {};
    if (!attr_set[ctx.device]) {
        err = cudaFuncSetAttribute(flash_attention_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (err != cudaSuccess)
            return err;
        attr_set[ctx.device] = true;
    }
    // persistent: one CTA per SM walks the (batch, head, 256-row query block) items
    const uint32_t items = ((ap.seq_q + 2 * BQ - 1) / (2 * BQ)) * ap.batch * ap.heads;
    const uint32_t ctas = items < (uint32_t)ctx.num_sms ? items : (uint32_t)ctx.num_sms;
    flash_attention_kernel<<<dim3(ctas), NUM_THREADS, SMEM_BYTES, stream>>>(maps, p);
    return cudaGetLastError();
}

}  // namespace kaio
