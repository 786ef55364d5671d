// Internal interface between the C-ABI layer (api.cu) and the kernel translation units.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace kaio {

// Epilogue selectors of the W8A8 GEMM.
enum : int {
    EPI_SCALAR = 0,  // f32 out = (acc as f32) * scale
    EPI_ROWCOL = 1,  // f32 out = ((acc as f32) * a_scale[i]) * w_scale[j]
    EPI_S32 = 2,     // s32 out = acc
    EPI_ROWCOL_F16 = 3,  // f16 out = f16_rn(((acc as f32) * a_scale[i]) * w_scale[j])
};

// Weight encodings of the dequantising GEMM (f16 activations).
enum : int {
    WFMT_S8_ROWMAJOR = 0,  // s8 [K,N] row-major (fused QKV W8A16)
    WFMT_S4_PACKED = 1,    // s4, 8 per u32 along K, words column-major, group-128 f16 scales
    WFMT_F16 = 2,          // f16 [K,N] row-major: used as is (matmul_tc)
};

// Per-device state owned by the library.
struct DeviceCtx {
    int device = -1;
    int num_sms = 0;
    int cc_major = 0, cc_minor = 0;
    uint32_t* status = nullptr;       // uint32[4] status block, zero = no error
};

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda).
cudaError_t encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes,
                                 const void* base, uint64_t inner, uint64_t outer,
                                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                                 CUtensorMapSwizzle swizzle);

// ---------------------------------------------------------------- W8A8
bool w8a8_fast_path_ok(const void* a, const void* b, const void* out, uint32_t m, uint32_t n,
                       uint32_t k);
cudaError_t launch_w8a8_gemm(const DeviceCtx& ctx, int epi, const int8_t* a, const int8_t* b,
                             void* out, float scale, const float* a_scale, const float* w_scale,
                             uint32_t m, uint32_t n, uint32_t k, cudaStream_t stream);
bool w8a8_2cta_ok(uint32_t m, uint32_t n, uint32_t k);
cudaError_t launch_w8a8_gemm_2cta(const DeviceCtx& ctx, int epi, const int8_t* a, const int8_t* b,
                                  void* out, float scale, const float* a_scale,
                                  const float* w_scale, uint32_t m, uint32_t n, uint32_t k,
                                  cudaStream_t stream);
// Fused W8A8 QKV projection on CTA pairs (m > 128): xq s8 [m,k] with per-row scales, three s8
// [k,n] weights with per-column scales, three f16 [m,n] outputs, one launch.
cudaError_t launch_w8a8_qkv_2cta(const DeviceCtx& ctx, const int8_t* xq, const float* x_scale,
                                 const int8_t* const w[3], const float* const col_scale[3],
                                 void* const out[3], uint32_t m, uint32_t n, uint32_t k,
                                 cudaStream_t stream);
cudaError_t launch_int8_generic(int epi, const int8_t* a, const int8_t* b, void* out, float scale,
                                const float* a_scale, const float* w_scale, uint32_t m, uint32_t n,
                                uint32_t k, cudaStream_t stream);

// ---------------------------------------------------------------- dequantising GEMMs
// One "problem" = one weight matrix + one output; the fused QKV ops pass three.
struct DqProblem {
    const void* w;          // s8 [K,N] or packed u32 [(K/8)*N]
    const __half* scales;   // group scales f16 [K/128, N] (WFMT_S4_PACKED) or nullptr
    const float* col_scale; // per-column f32 post-scale or nullptr
    float scale;            // scalar f32 post-scale (used when col_scale == nullptr)
    void* out;              // f32 or f16 [M,N]
};

cudaError_t launch_dq_generic(int wfmt, const __half* x, const DqProblem* probs, int num_probs,
                              bool out_f16, bool post_scale, uint32_t m, uint32_t n, uint32_t k,
                              cudaStream_t stream);

struct OutputCopies;
bool w4a16_decode_ok(const void* x, const DqProblem* probs, int num_probs, uint32_t m, uint32_t n,
                     uint32_t k);
size_t w4a16_decode_workspace_bytes(const DeviceCtx& ctx, uint32_t n, uint32_t k);
size_t w4a16_decode_num_counters(uint32_t n);
cudaError_t launch_w4a16_decode(const DeviceCtx& ctx, const __half* x, const DqProblem& prob,
                                bool out_f16, uint32_t m, uint32_t n, uint32_t k, void* workspace,
                                uint32_t* counters, cudaStream_t stream,
                                const OutputCopies* copies = nullptr);

// Fused W4A16 GEMM for m > 16: int4 -> f16 dequantisation inside the GEMM (weights go from the
// packed words to tensor memory, never to global memory as f16).  Needs no workspace.
bool w4a16_fused_ok(const void* x, const DqProblem* probs, int num_probs, uint32_t m, uint32_t n,
                    uint32_t k);
// Scratch of its stream-K form (f32 partial tiles + arrival counters); 0 when the column tiles
// fill the SMs well enough.  Without scratch (nullptr) every tile runs whole on one CTA.
size_t w4a16_fused_workspace_bytes(const DeviceCtx& ctx, int num_probs, uint32_t m, uint32_t n,
                                   uint32_t k);
size_t w4a16_fused_num_counters(const DeviceCtx& ctx, int num_probs, uint32_t m, uint32_t n,
                                uint32_t k);
cudaError_t launch_w4a16_fused(const DeviceCtx& ctx, const __half* x, const DqProblem* probs,
                               int num_probs, bool out_f16, uint32_t m, uint32_t n, uint32_t k,
                               void* workspace, uint32_t* counters, cudaStream_t stream,
                               const OutputCopies* copies = nullptr);

bool dq_gemm_fast_path_ok(int wfmt, const void* x, const DqProblem* probs, int num_probs,
                          bool out_f16, uint32_t m, uint32_t n, uint32_t k);
// Destinations of a single-output GEMM: the [m, n] result is stored to every ptrs[r] (already
// offset to this call's first column) with row stride ld elements.  Used by the sharded
// all-gather form, where the destinations are the output buffers of all ranks (peer memory).
struct OutputCopies {
    void* ptrs[8];
    uint32_t count;
    uint64_t ld;
    // 0: every output column is stored to every destination at its own column index.
    // > 0: column c is stored only to destination c / scatter_cols, at column c % scatter_cols
    // (each destination receives one block of columns: the reduce-scatter form).
    uint32_t scatter_cols;
    // Column at which this caller starts its walk over the output (the paired f16 GEMM honours it;
    // the small-M kernels ignore it).  In the scatter form every rank works through the same
    // tiles: started at the same column they would all store to the same owner at the same time
    // and that owner's NVLink ingress would set the pace; started one block apart, each owner
    // receives from one or two ranks at a time.  The tiles and their results do not change.
    uint32_t start_col;
    // Non-null: an address of an NVLink multicast object that all destinations' buffers are bound
    // to (already offset to this caller's first column, row stride ld).  The paired f16 GEMM then
    // writes every output block ONCE with multimem.st and the switch delivers it to all ranks
    // (1/count of the egress); ptrs[] stay valid for the kernels that do not take this path.
    void* multicast;
};

size_t dq_gemm_workspace_bytes(int num_probs, uint32_t n, uint32_t k);
// The pre-pass of the M > 512 W4A16 path on its own: packed s4 + group scales -> f16 [K,N]
// row-major with the reference's rounding (f16(q) * f16(scale) in f16).  n even.
cudaError_t launch_dequant_s4(const uint32_t* w_packed, const __half* scales, __half* out,
                              uint32_t n, uint32_t k, cudaStream_t stream);
cudaError_t launch_dq_gemm(const DeviceCtx& ctx, int wfmt, const __half* x, const DqProblem* probs,
                           int num_probs, bool out_f16, bool post_scale, uint32_t m, uint32_t n,
                           uint32_t k, void* dq_workspace, cudaStream_t stream,
                           const OutputCopies* copies = nullptr, bool silu_gate = false);
// silu_gate (one problem, f16 out, n % 128 == 0): the weight columns alternate in blocks of 64
// between two projections; the epilogue rounds both to f16, applies out = silu(a) * b and stores
// [m, n/2] (probs[0].out).

// ---------------------------------------------------------------- quantisers
cudaError_t launch_quantize_rows_int8(const float* x, int8_t* q, float* scale, uint32_t m,
                                      uint32_t k, cudaStream_t stream);
// The same quantiser on f16 activations (widened to f32 exactly, then the same arithmetic).
cudaError_t launch_quantize_rows_int8_f16(const __half* x, int8_t* q, float* scale, uint32_t m,
                                          uint32_t k, cudaStream_t stream);
cudaError_t launch_quantize_pack_s4(const float* w, uint32_t* packed, __half* scales, uint32_t k,
                                    uint32_t n, cudaStream_t stream);

// ---------------------------------------------------------------- sum of partial outputs
cudaError_t launch_sum_partials(const float* slots, uint32_t world, uint32_t rows, uint32_t cols,
                                float* const* outs, uint32_t num_out, uint64_t out_ld,
                                uint32_t out_col0, bool multicast, cudaStream_t stream);

cudaError_t launch_multimem_allreduce_f32(const float* mc_in, float* mc_out, uint32_t rows,
                                          uint32_t cols, uint64_t ld, uint32_t col0,
                                          cudaStream_t stream);

// ---------------------------------------------------------------- gated activation
cudaError_t launch_silu_gate_f32(const float* x, const float* gate, float* out, size_t n,
                                 cudaStream_t stream);
cudaError_t launch_silu_gate_f16(const __half* x, const __half* gate, __half* out, uint32_t rows,
                                 uint32_t cols, uint32_t x_ld, uint32_t gate_ld, uint32_t out_ld,
                                 cudaStream_t stream);
cudaError_t launch_silu_gate_f16_interleaved(const __half* gu, __half* out, uint32_t rows,
                                             uint32_t cols, uint32_t gu_ld, uint32_t out_ld,
                                             cudaStream_t stream);

// ---------------------------------------------------------------- self-test of the bounded wait
cudaError_t launch_selftest_bounded_wait(const DeviceCtx& ctx, uint32_t budget_us,
                                         cudaStream_t stream);

// ---------------------------------------------------------------- NCCL all-gather of column shards
// NCCL is looked up with dlopen at first use; false when no libnccl.so.2 can be loaded.
bool nccl_available();
// ncclAllGather into staging ([P][m][n_loc]) + un-shard copy into out ([m][P * n_loc]).  Returns
// the NCCL result (0 = ok) with its text in *msg; a CUDA launch error in *cuda_err.
int launch_allgather_cols(const void* shard, void* staging, void* out, uint32_t m, uint32_t n_loc,
                          uint32_t elem_bytes, uint32_t world, void* nccl_comm, cudaStream_t stream,
                          const char** msg, cudaError_t* cuda_err);

// ---------------------------------------------------------------- tensor-pipe rate probe
// One CTA per SM issues `iters` back-to-back tcgen05.mma kind::i8 M128 N256 K32.
cudaError_t launch_int8_mma_rate(const DeviceCtx& ctx, uint32_t iters, cudaStream_t stream);

// ---------------------------------------------------------------- attention
struct AttnParams {
    const __half *q, *k, *v;
    void* out;  // f32 or f16
    uint32_t batch, heads, seq_q, seq_k, d_k, d_v;
    // element strides: row stride and per-head / per-batch offsets
    uint64_t q_row, k_row, v_row, o_row;
    uint64_t q_head, k_head, v_head, o_head;
    uint64_t q_batch, k_batch, v_batch, o_batch;
    int causal;
    int out_f16;
};

cudaError_t launch_attention_generic(const AttnParams& p, cudaStream_t stream);
bool flash_attention_ok(const AttnParams& p);
cudaError_t launch_flash_attention(const DeviceCtx& ctx, const AttnParams& p, cudaStream_t stream);

}  // namespace kaio
