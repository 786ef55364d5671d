/*
 * kaio_b200.h -- C ABI of libkaio_b200.so, the sm_100a (B200) implementation of the
 * quantized-inference ops of KAIO's `kaio-ops` crate.
 *
 * Each entry point below replaces the PTX-JIT launch path inside one `kaio-ops`
 * function; the Rust function keeps its signature and its host-side contract and
 * calls the entry point with the raw device pointers, element counts and stream of
 * its `GpuBuffer` / `KaioDevice` arguments (paths are relative to the KAIO tree).
 *
 * Conventions (all entry points):
 *   - pointers are DEVICE pointers owned by the caller; inputs are never written,
 *     outputs are written only in [0, m*n) (or the documented extent);
 *   - `*_len` arguments are element counts of the caller's buffers (GpuBuffer::len());
 *     they are validated exactly like the reference validates them, and a buffer may
 *     be longer than the shape needs;
 *   - `stream` is a CUstream / cudaStream_t (NULL = the legacy default stream).  Work is
 *     enqueued on it and the call returns without synchronising, like the reference
 *     (kaio-ops/src/matmul_int8_kernel.rs:1497-1511);
 *   - the device is the calling thread's current CUDA device, and the output buffer must live
 *     on it: the entry points of the drop-in ops look the pointer's device up
 *     (cudaPointerGetAttributes) and return KAIO_B200_ERR_INVALID_CONFIG on a mismatch, where the
 *     reference compares the buffer's device ordinal with the KaioDevice's;
 *   - scratch the kernels need beyond the caller's buffers (split-K partial tiles, arrival
 *     counters, dequantised weights) is owned by the library, one set per (device, stream), so
 *     calls on different streams may overlap; it grows on demand with cudaFree + cudaMalloc,
 *     which synchronises the device.  Growth is refused (KAIO_B200_ERR_INVALID_CONFIG) while the
 *     stream is being captured into a CUDA graph, and a graph captured earlier keeps the old
 *     address: run every op once at its largest shape before capturing;
 *   - return value: KAIO_B200_OK or an error code; kaio_b200_last_error() returns the
 *     calling thread's last message.  For KAIO_B200_ERR_INVALID_CONFIG the message is
 *     the text the reference puts into KaioError::InvalidConfig;
 *   - there is no CPU fallback: on a machine without an sm_100 GPU every op returns
 *     KAIO_B200_ERR_UNSUPPORTED_ARCH or KAIO_B200_ERR_CUDA.
 *
 * f16 values are IEEE binary16 bit patterns (uint16_t here, `half::f16` / `__half` on
 * either side).
 */
#ifndef KAIO_B200_H
#define KAIO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KAIO_B200_OK 0
#define KAIO_B200_ERR_INVALID_CONFIG 1   /* KaioError::InvalidConfig (kaio-runtime/src/error.rs:4-37) */
#define KAIO_B200_ERR_CUDA 2             /* KaioError::Cuda */
#define KAIO_B200_ERR_UNSUPPORTED_ARCH 3 /* analogue of ValidationError::SmTooLow */
#define KAIO_B200_ERR_TIMEOUT 4          /* a device-side bounded wait gave up (see kaio_b200_device_status) */

typedef uint16_t kaio_f16;

/* ---- W8A8 ------------------------------------------------------------------------ */

/* Replaces kaio_ops::matmul_int8 (kaio-ops/src/matmul_int8_kernel.rs:1468-1512).
 * c[i,j] = ((sum_k a[i,k]*b[k,j]) as f32) * scale; a s8 [m,k], b s8 [k,n], c f32 [m,n],
 * all row-major; k % 32 == 0. */
int32_t kaio_b200_matmul_int8(const int8_t* a, size_t a_len, const int8_t* b, size_t b_len,
                              float* c, size_t c_len, float scale, uint32_t m, uint32_t n,
                              uint32_t k, void* stream);

/* Extension (no reference counterpart): per-row activation and per-column weight scales,
 * c[i,j] = (((acc) as f32) * a_scale[i]) * w_scale[j]. */
int32_t kaio_b200_matmul_int8_scaled(const int8_t* a, size_t a_len, const int8_t* b, size_t b_len,
                                     float* c, size_t c_len, const float* a_scale,
                                     size_t a_scale_len, const float* w_scale, size_t w_scale_len,
                                     uint32_t m, uint32_t n, uint32_t k, void* stream);

/* Extension: the raw s32 accumulators, acc[i,j] = sum_k a[i,k]*b[k,j] (exact). */
int32_t kaio_b200_matmul_int8_acc(const int8_t* a, size_t a_len, const int8_t* b, size_t b_len,
                                  int32_t* acc, size_t acc_len, uint32_t m, uint32_t n, uint32_t k,
                                  void* stream);

/* ---- f16 GEMM --------------------------------------------------------------------- */

/* Replaces kaio_ops::matmul_tc (kaio-ops/src/matmul_tc_kernel.rs:1583-1626) and
 * kaio_ops::matmul_tc_async (kaio-ops/src/matmul_tc_async_kernel.rs, same signature, same
 * validation through validate_dims_tc): a f16 [m,k] row-major, b f16 [k,n] row-major, c f32 [m,n]
 * row-major, f32 accumulation.  k % 16 == 0; m and n are free.  Both entry points run the same
 * kernel here (the reference's two differ only in how they stage shared memory). */
int32_t kaio_b200_matmul_tc(const kaio_f16* a, size_t a_len, const kaio_f16* b, size_t b_len,
                            float* c, size_t c_len, uint32_t m, uint32_t n, uint32_t k,
                            void* stream);
int32_t kaio_b200_matmul_tc_async(const kaio_f16* a, size_t a_len, const kaio_f16* b, size_t b_len,
                                  float* c, size_t c_len, uint32_t m, uint32_t n, uint32_t k,
                                  void* stream);

/* Extension: the same product narrowed to f16 (round to nearest even): c f16 [m,n]. */
int32_t kaio_b200_matmul_tc_f16out(const kaio_f16* a, size_t a_len, const kaio_f16* b, size_t b_len,
                                   kaio_f16* c, size_t c_len, uint32_t m, uint32_t n, uint32_t k,
                                   void* stream);

/* ---- W4A16 ----------------------------------------------------------------------- */

/* Replaces kaio_ops::matmul_int4 (kaio-ops/src/matmul_int4_kernel.rs:2126-2171).
 * a f16 [m,k]; b_packed u32 [(k/8)*n]: word k/8 of column j at (k/8) + j*(k/8), nibble
 * k%8 at bits [4*(k%8), +4), signed; scales f16 [k/128, n]; c f32 [m,n];
 * group_size must be 128 and k % 128 == 0. */
int32_t kaio_b200_matmul_int4(const kaio_f16* a, size_t a_len, const uint32_t* b_packed,
                              size_t b_len, const kaio_f16* scales, size_t scales_len, float* c,
                              size_t c_len, uint32_t m, uint32_t n, uint32_t k,
                              uint32_t group_size, void* stream);

/* Extension (no reference counterpart): the dequantisation step of kaio_b200_matmul_int4 on its
 * own -- w[kk, j] = f16(q[kk, j]) * scales[kk / 128, j] rounded to f16, the reference's mul.f16
 * (kaio-ops/src/matmul_int4_kernel.rs:655-713) -- written as f16 [k, n] row-major.  A caller that
 * runs several products against the same weights in one step (row chunks of a large M whose
 * partial results are exchanged while the next chunk is computed) dequantises once and then calls
 * kaio_b200_matmul_tc / kaio_b200_matmul_tc_f16out: the results equal kaio_b200_matmul_int4's for
 * m > 512 bit for bit, since that op runs these two steps internally.  n even. */
int32_t kaio_b200_dequantize_int4(const uint32_t* b_packed, size_t b_len, const kaio_f16* scales,
                                  size_t scales_len, kaio_f16* w, size_t w_len, uint32_t k,
                                  uint32_t n, uint32_t group_size, void* stream);

/* Extension: same product with the f32 accumulator narrowed to f16 (round to nearest even). */
int32_t kaio_b200_matmul_int4_f16out(const kaio_f16* a, size_t a_len, const uint32_t* b_packed,
                                     size_t b_len, const kaio_f16* scales, size_t scales_len,
                                     kaio_f16* c, size_t c_len, uint32_t m, uint32_t n, uint32_t k,
                                     uint32_t group_size, void* stream);

/* No counterpart in the reference.  kaio_b200_matmul_int4 for decode shapes (m <= 16) that
 * allocates nothing: same arguments, same result bit for bit, but the split-K scratch (partial
 * tiles, arrival counters, status words) lives in a fixed ~5.3 MB array inside the library instead
 * of a cudaMalloc'd workspace.  It is for callers that cannot allocate at call time: a host
 * runtime whose memory pool already owns all device memory (a later cudaMalloc would fail), or a
 * latency-critical loop that must not hit the device-wide synchronisation an allocation implies.
 * Limits (rejected with KAIO_B200_ERR_INVALID_CONFIG): m <= 16, n <= 524288, a device with at
 * most 160 SMs, 16-byte aligned a / b_packed.
 * The first call on each device looks up the array's device address.  With CUDA's lazy module
 * loading that look-up is also what places the array in device memory, so the first call can
 * still claim those ~5.3 MB: make it before a pool reserves the rest of the device and before any
 * stream capture.  Later calls allocate nothing.
 * Every call on a device shares the one array, so calls that may overlap on the GPU (different
 * streams) race: order them.  The call clears the arrival counters on `stream` before launching;
 * the status words persist until kaio_b200_device_status() (which allocates nothing either) has
 * reported them. */
int32_t kaio_b200_matmul_int4_noalloc(const kaio_f16* a, size_t a_len, const uint32_t* b_packed,
                                      size_t b_len, const kaio_f16* scales, size_t scales_len,
                                      float* c, size_t c_len, uint32_t m, uint32_t n, uint32_t k,
                                      uint32_t group_size, void* stream);

/* Extension (no reference counterpart; KAIO is single-device): column-parallel W4A16 GEMM fused
 * with the all-gather of its output.  The caller is rank `rank` of `world` (<= 8) processes, one per
 * GPU of a node; it passes its shard of the weights (columns [rank*N/world, (rank+1)*N/world): a
 * contiguous slice of the packed buffer, and the matching [K/128, N/world] scales) and `out_ptrs`, a
 * HOST array of `world` device pointers: out_ptrs[r] is rank r's f16 [m, n_total] output buffer as
 * mapped in THIS process (peer memory for r != rank, e.g. from torch symmetric memory or CUDA IPC).
 * The kernel's epilogue stores every output block straight into all `world` buffers (TMA bulk
 * stores / plain stores over NVLink), so the transfer overlaps the GEMM tile by tile; no NCCL call
 * is involved.  The caller must synchronise the ranks (all kernels complete) before anyone reads. */
int32_t kaio_b200_matmul_int4_allgather(const kaio_f16* a, size_t a_len,
                                        const uint32_t* b_packed_shard, size_t b_len,
                                        const kaio_f16* scales_shard, size_t scales_len,
                                        void* const* out_ptrs, size_t out_len, uint32_t world,
                                        uint32_t rank, uint32_t m, uint32_t n_total, uint32_t k,
                                        uint32_t group_size, void* stream);

/* The same with the rows above m = 512 written through an NVLink multicast object: multicast_out
 * is the multicast address of the [m, n_total] output that every rank's buffer is bound to (e.g.
 * the multicast pointer of a torch symmetric-memory allocation).  The paired GEMM then stores each
 * output block once as `multimem.st` and the switch delivers it to all ranks (1/world of the
 * egress).  Smaller m use out_ptrs as above, which therefore stay required. */
int32_t kaio_b200_matmul_int4_allgather_multicast(
    const kaio_f16* a, size_t a_len, const uint32_t* b_packed_shard, size_t b_len,
    const kaio_f16* scales_shard, size_t scales_len, void* const* out_ptrs, size_t out_len,
    void* multicast_out, uint32_t world, uint32_t rank, uint32_t m, uint32_t n_total, uint32_t k,
    uint32_t group_size, void* stream);

/* Extension (no reference counterpart; KAIO is single-device): the all-gather of a column-parallel
 * GEMM's output through NCCL.  Every rank passes its [m, n_total / world] shard (row-major,
 * elem_bytes = 2 for f16 or 4 for f32) and receives the row-major [m, n_total] matrix in `out`.
 * `nccl_comm` is the caller's ncclComm_t for the `world` ranks; the op enqueues one ncclAllGather
 * and one copy kernel on `stream`.  NCCL is looked up at the first call (dlopen of libnccl.so.2,
 * i.e. the NCCL already loaded into the process when there is one), so the library itself has no
 * link-time dependency on it; without NCCL the call returns KAIO_B200_ERR_CUDA.  The staging
 * buffer ([world][m][n_total / world]) is library-owned per-stream scratch. */
int32_t kaio_b200_allgather_cols(const void* shard, size_t shard_len, void* out, size_t out_len,
                                 uint32_t m, uint32_t n_total, uint32_t elem_bytes, uint32_t world,
                                 void* nccl_comm, void* stream);

/* ---- fused QKV projection ---------------------------------------------------------- */

/* Replaces kaio_ops::qkv_project_int8 (kaio-ops/src/qkv_project_int8_kernel.rs:2008-2064),
 * W8A16: out_P[i,j] = f16((sum_k x[i,k] * f16(w_P[k,j])) * scale_P) for P in {q,k,v};
 * x f16 [m,k]; w_P s8 [k,n] row-major; outputs f16 [m,n]; k % 16 == 0, n even. */
int32_t kaio_b200_qkv_project_int8(const kaio_f16* x, size_t x_len, const int8_t* w_q,
                                   size_t w_q_len, const int8_t* w_k, size_t w_k_len,
                                   const int8_t* w_v, size_t w_v_len, float scale_q, float scale_k,
                                   float scale_v, kaio_f16* q_out, size_t q_len, kaio_f16* k_out,
                                   size_t k_len, kaio_f16* v_out, size_t v_len, uint32_t m,
                                   uint32_t n, uint32_t k, void* stream);

/* Extension: per-column f32 scales (f32 [n] per projection) instead of scalars. */
int32_t kaio_b200_qkv_project_int8_colscale(const kaio_f16* x, size_t x_len, const int8_t* w_q,
                                            size_t w_q_len, const int8_t* w_k, size_t w_k_len,
                                            const int8_t* w_v, size_t w_v_len,
                                            const float* scale_q, const float* scale_k,
                                            const float* scale_v, size_t scale_len,
                                            kaio_f16* q_out, size_t q_len, kaio_f16* k_out,
                                            size_t k_len, kaio_f16* v_out, size_t v_len,
                                            uint32_t m, uint32_t n, uint32_t k, void* stream);

/* Extension (no reference counterpart: the reference's INT8 QKV op is W8A16,
 * kaio-ops/src/qkv_project_int8_kernel.rs:1965-1985): the W8A8 form.  x is quantised per row on
 * the fly with the reference's symmetric quantiser (examples/int8_matmul/src/main.rs:41-61:
 * s_x[i] = max_k |x[i,k]| / 127, 1 for an all-zero row; xq = clamp(round(x / s_x), -127, 127),
 * round half away from zero), the products accumulate exactly in s32 on the INT8 tensor pipe, and
 * out_P[i,j] = f16((((sum_k xq[i,k] * w_P[k,j]) as f32) * s_x[i]) * scale_P[j]).
 * x f16 [m,k] (16-byte aligned); w_P s8 [k,n] row-major; scale_P f32 [n]; outputs f16 [m,n],
 * three distinct buffers; k % 32 == 0, n even. */
int32_t kaio_b200_qkv_project_w8a8(const kaio_f16* x, size_t x_len, const int8_t* w_q,
                                   size_t w_q_len, const int8_t* w_k, size_t w_k_len,
                                   const int8_t* w_v, size_t w_v_len, const float* scale_q,
                                   const float* scale_k, const float* scale_v, size_t scale_len,
                                   kaio_f16* q_out, size_t q_len, kaio_f16* k_out, size_t k_len,
                                   kaio_f16* v_out, size_t v_len, uint32_t m, uint32_t n,
                                   uint32_t k, void* stream);

/* Replaces kaio_ops::qkv_project_int4 (kaio-ops/src/qkv_project_int4_kernel.rs:1495-1555),
 * W4A16: three matmul_int4-style products sharing x, outputs f16 = f16(acc), no post-scale;
 * packed weights and group scales laid out as for kaio_b200_matmul_int4; n even. */
int32_t kaio_b200_qkv_project_int4(const kaio_f16* x, size_t x_len, const uint32_t* w_q_packed,
                                   size_t w_q_len, const uint32_t* w_k_packed, size_t w_k_len,
                                   const uint32_t* w_v_packed, size_t w_v_len,
                                   const kaio_f16* scales_q, size_t scales_q_len,
                                   const kaio_f16* scales_k, size_t scales_k_len,
                                   const kaio_f16* scales_v, size_t scales_v_len, kaio_f16* q_out,
                                   size_t q_len, kaio_f16* k_out, size_t k_len, kaio_f16* v_out,
                                   size_t v_len, uint32_t m, uint32_t n, uint32_t k,
                                   uint32_t group_size, void* stream);

/* ---- attention --------------------------------------------------------------------- */

/* Replaces kaio_ops::attention_tc and attention_tc_causal
 * (kaio-ops/src/attention_tc_kernel.rs:2240-2333): out = softmax(q k^T / sqrt(d_k) [+ causal
 * mask j > i]) v; q f16 [seq_q,d_k], k f16 [seq_k,d_k], v f16 [seq_k,d_v], out f32
 * [seq_q,d_v]; the reference's shape limits apply (multiples of 16/16/16/8, seq_k <= 384,
 * d_k, d_v <= 128). */
int32_t kaio_b200_attention_tc(const kaio_f16* q, size_t q_len, const kaio_f16* k, size_t k_len,
                               const kaio_f16* v, size_t v_len, float* out, size_t out_len,
                               uint32_t seq_q, uint32_t seq_k, uint32_t d_k, uint32_t d_v,
                               int32_t causal, void* stream);

/* Extension: batched multi-head attention, f16 output, any seq_k.  q/k/v/out are f16
 * [batch*seq, heads*head_dim] row-major with row stride `row_stride` elements (the layout the
 * fused QKV projection writes); head h of batch b starts at row b*seq, column h*head_dim. */
int32_t kaio_b200_attention_mha_f16(const kaio_f16* q, size_t q_len, const kaio_f16* k,
                                    size_t k_len, const kaio_f16* v, size_t v_len, kaio_f16* out,
                                    size_t out_len, uint32_t batch, uint32_t heads, uint32_t seq_q,
                                    uint32_t seq_k, uint32_t head_dim, uint32_t row_stride,
                                    int32_t causal, void* stream);

/* EXT: the gate|up projection of a feed-forward block with the SiLU-gate in the GEMM's epilogue.
 * b_packed / scales describe W4A16 weights [k, 2*cols] in kaio_b200_matmul_int4's layout whose
 * COLUMNS ALTERNATE IN BLOCKS OF 64: block 2b holds columns [64b, 64b+64) of W_gate, block 2b+1
 * the same columns of W_up (cols % 64 == 0).  act f16 [m, cols] = silu(x W_gate) * (x W_up), both
 * projections rounded to f16 first: bit for bit what kaio_b200_matmul_int4_f16out followed by
 * kaio_b200_silu_gate_f16 gives.  For m > 512 the [m, 2*cols] projection never reaches memory;
 * smaller m run the small-M W4A16 kernels into gu_scratch (f16 [m, 2*cols], 16-byte aligned,
 * required there, ignored otherwise) and apply the activation in a second launch. */
int32_t kaio_b200_matmul_int4_silu_gate(const kaio_f16* x, size_t x_len, const uint32_t* b_packed,
                                        size_t b_len, const kaio_f16* scales, size_t scales_len,
                                        kaio_f16* act, size_t act_len, kaio_f16* gu_scratch,
                                        size_t gu_len, uint32_t m, uint32_t cols, uint32_t k,
                                        uint32_t group_size, void* stream);

/* ---- quantisers (the step in front of the GEMMs; host code in the reference's examples) ---- */

/* GPU form of `derive_scale` + `quantize` applied per row
 * (examples/int8_matmul/src/main.rs:41-61): scale[i] = max_k |x[i,k]| / 127 (1 for an all-zero
 * row), q[i,k] = clamp(round(x[i,k] / scale[i]), -127, 127), round half away from zero.
 * x f32 [m,k], q s8 [m,k], scale f32 [m].  Feeds kaio_b200_matmul_int8_scaled. */
int32_t kaio_b200_quantize_rows_int8(const float* x, size_t x_len, int8_t* q, size_t q_len,
                                     float* scale, size_t scale_len, uint32_t m, uint32_t k,
                                     void* stream);

/* GPU form of `quantize_gptq_lite` + `pack_s4_weights` (examples/int4_matmul/src/main.rs:48-99):
 * per (column, group of 128 k): scale = max |w| / 7 (1 if zero) stored as f16,
 * q = clamp(round(w / scale), -8, 7) with the f32 scale; packed as kaio_b200_matmul_int4 expects.
 * w f32 [k,n] row-major, packed u32 [(k/8)*n], scales f16 [k/128, n]. */
int32_t kaio_b200_quantize_pack_int4(const float* w, size_t w_len, uint32_t* packed,
                                     size_t packed_len, kaio_f16* scales, size_t scales_len,
                                     uint32_t k, uint32_t n, uint32_t group_size, void* stream);

/* ---- row-parallel (K-sharded) W4A16 with the reduction fused into the GEMM (EXT) ---------- */

/* This rank's K shard of a W4A16 GEMM (a [m, k] f16, weights packed [k, n], k = this rank's
 * part of the full K): the f32 partial product [m, n] is stored by the GEMM's epilogue into
 * staging slot `rank` of other ranks' staging buffers, tile by tile over peer memory.
 * slot_ptrs[d] is rank d's staging buffer as mapped in this process, f32 [world][m][cols]:
 *   scatter == 0: cols = n, the whole partial goes to every rank (one-step all-reduce);
 *   scatter != 0: cols = n / world, column block d goes to rank d only (reduce-scatter; n / world
 *                 must be a multiple of 64).
 * After all ranks have met at a barrier, kaio_b200_sum_partials_f32 adds the slots. */
int32_t kaio_b200_matmul_int4_peer_partials(const kaio_f16* a, size_t a_len,
                                            const uint32_t* b_packed, size_t b_len,
                                            const kaio_f16* scales, size_t scales_len,
                                            void* const* slot_ptrs, size_t slot_len, uint32_t world,
                                            uint32_t rank, int32_t scatter, uint32_t m, uint32_t n,
                                            uint32_t k, uint32_t group_size, void* stream);

/* out_d[row * out_ld + out_col0 + c] = sum over s < world (ascending) of slots[s][row][c] for each
 * of the num_out (1..8) destinations, which may be peer memory (the all-gather step of a two-step
 * all-reduce).  slots f32 [world][rows][cols]; cols, out_ld, out_col0 multiples of 4. */
int32_t kaio_b200_sum_partials_f32(const float* slots, size_t slots_len, uint32_t world,
                                   uint32_t rows, uint32_t cols, void* const* out_ptrs,
                                   uint32_t num_out, size_t out_len, uint32_t out_ld,
                                   uint32_t out_col0, void* stream);

/* The same sum with ONE destination that is an address of an NVLink multicast object (every
 * rank's output buffer bound to it, e.g. the multicast pointer of a torch symmetric-memory
 * allocation): each vector leaves the GPU once as `multimem.st` and the switch delivers it to all
 * ranks, 1/world of the egress of the form above.  The caller orders the ranks around it
 * (a barrier before reading the outputs), as with peer stores. */
int32_t kaio_b200_sum_partials_f32_multicast(const float* slots, size_t slots_len, uint32_t world,
                                             uint32_t rows, uint32_t cols, void* multicast_out,
                                             size_t out_len, uint32_t out_ld, uint32_t out_col0,
                                             void* stream);

/* All-reduce (sum) of an f32 [rows, ld] buffer that every rank holds at the same offset of a
 * symmetric allocation bound to an NVLink multicast object.  multicast_in / multicast_out are the
 * multicast addresses of the partial buffer and of the output buffer.  This rank reduces the column
 * block [col0, col0 + cols) of all rows: `multimem.ld_reduce` adds the ranks' elements inside the
 * switch, `multimem.st` delivers the sum to every rank.  Every rank calls it with its own block
 * (rank r: col0 = r * ld / world), between two barriers of the caller's (partials complete
 * before, outputs complete after).  One reducer per element: the same bits on every rank; the
 * order of the in-switch additions is the hardware's. */
int32_t kaio_b200_allreduce_multimem_f32(const void* multicast_in, void* multicast_out, size_t len,
                                         uint32_t rows, uint32_t cols, uint32_t ld, uint32_t col0,
                                         void* stream);

/* ---- gated activation (between the up/gate and the down projection of an FFN block) ---- */

/* The user kernel of examples/fused_silu_gate/src/main.rs:13-21:
 * out[i] = x[i] * (1 / (1 + exp(-x[i]))) * gate[i], f32, i < n. */
int32_t kaio_b200_silu_gate_f32(const float* x, size_t x_len, const float* gate, size_t gate_len,
                                float* out, size_t out_len, uint32_t n, void* stream);

/* The same on f16 matrices (EXT, not in the reference): f32 arithmetic on the widened inputs,
 * one rounding to f16.  x, gate and out are [rows, cols] with row strides x_ld, gate_ld, out_ld
 * (elements, >= cols), so x and gate may be the two halves of one [rows, 2*cols] projection
 * output.  Each buffer must hold (rows-1)*ld + cols elements. */
int32_t kaio_b200_silu_gate_f16(const kaio_f16* x, size_t x_len, const kaio_f16* gate,
                                size_t gate_len, kaio_f16* out, size_t out_len, uint32_t rows,
                                uint32_t cols, uint32_t x_ld, uint32_t gate_ld, uint32_t out_ld,
                                void* stream);

/* ---- library state ------------------------------------------------------------------- */

/* Last error message of the calling thread ("" if none). */
const char* kaio_b200_last_error(void);

/* Synchronises `stream` and reads the current device's status blocks (the regular entry points'
 * and the allocation-free entry point's): code[0] = 0 when no kernel reported a problem, else
 * {code, reporting block, site, kernel id} of the first report; that block is cleared and the
 * device's split-K arrival counters are reset, so the next call starts clean.  Returns
 * KAIO_B200_ERR_TIMEOUT when code[0] != 0.  Allocates nothing.
 * No counterpart in the reference, whose kernels have no device-side waits
 * (kaio-runtime/src/error.rs:4-37 has no timeout variant). */
int32_t kaio_b200_device_status(void* stream, uint32_t code[4]);

/* Test hook (no counterpart in the reference): launches one CTA that waits `budget_us`
 * microseconds on a barrier nothing arrives at, gives up and returns normally; the next
 * kaio_b200_device_status() then reports KAIO_B200_ERR_TIMEOUT.  This is the path every kernel of
 * the library takes when a device-side wait runs out: a status code, never a hang or a trap. */
int32_t kaio_b200_selftest_bounded_wait(uint32_t budget_us, void* stream);

/* Diagnostic (no counterpart in the reference): enqueues a probe of the INT8 tensor-pipe rate on
 * `stream` -- one CTA per SM, each issuing `iters` back-to-back tcgen05.mma kind::i8 M128 N256 K32
 * on zeroed shared-memory operands, no loads, no epilogue -- and stores in *ops the integer
 * operations it stands for (2 * 128 * 256 * 32 * iters * SMs).  The caller times it with events:
 * ops / time is the INT8 tensor peak a GEMM on this device can be measured against. */
int32_t kaio_b200_probe_int8_mma_rate(uint32_t iters, uint64_t* ops, void* stream);

/* Name of the kernel variant the last call on this thread dispatched to (for tests and
 * traces): e.g. "w8a8_tcgen05", "int8_generic". */
const char* kaio_b200_last_variant(void);

/* Frees the library's per-device workspaces.  Callers must have synchronised. */
void kaio_b200_shutdown(void);

/* ABI version: major*1000 + minor. */
int32_t kaio_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KAIO_B200_H */
