// Shape-agnostic CUDA-core kernels.  They serve the shapes the TMA / tcgen05 kernels do not
// take (odd N, unaligned bases, tiny attention heads) and keep the reference's operation
// order exactly: one f32 multiply and one f32 add per term, k ascending, no fused
// multiply-add -- so their results equal the CPU reference functions bit for bit
// (kaio-ops/tests/matmul_int8_e2e.rs:20-34, matmul_int4_e2e.rs:60-95,
// qkv_project_int8_e2e.rs:48-72, qkv_project_int4_e2e.rs:70-100).
#include "kernels.h"

namespace kaio {

// ---------------------------------------------------------------- W8A8, any shape
template <int EPI>
__global__ void __launch_bounds__(256)
int8_generic_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b, void* out,
                    float scale, const float* __restrict__ a_scale,
                    const float* __restrict__ w_scale, uint32_t m, uint32_t n, uint32_t k)
{
    constexpr int T = 16, KC = 32;
    __shared__ int32_t as[T][KC + 1];
    __shared__ int32_t bs[KC][T + 1];
    const uint32_t tx = threadIdx.x, ty = threadIdx.y;
    const uint32_t row = blockIdx.y * T + ty, col = blockIdx.x * T + tx;
    int32_t acc = 0;
    for (uint32_t k0 = 0; k0 < k; k0 += KC) {
        for (uint32_t kk = tx; kk < KC; kk += T)
            as[ty][kk] = (row < m) ? (int32_t)a[(size_t)row * k + k0 + kk] : 0;
        for (uint32_t kk = ty; kk < KC; kk += T)
            bs[kk][tx] = (col < n) ? (int32_t)b[(size_t)(k0 + kk) * n + col] : 0;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < KC; ++kk)
            acc += as[ty][kk] * bs[kk][tx];
        __syncthreads();
    }
    if (row < m && col < n) {
        const size_t idx = (size_t)row * n + col;
        if (EPI == EPI_S32) {
            reinterpret_cast<int32_t*>(out)[idx] = acc;
        } else if (EPI == EPI_SCALAR) {
            reinterpret_cast<float*>(out)[idx] = __fmul_rn(__int2float_rn(acc), scale);
        } else if (EPI == EPI_ROWCOL_F16) {
            reinterpret_cast<__half*>(out)[idx] = __float2half_rn(
                __fmul_rn(__fmul_rn(__int2float_rn(acc), a_scale[row]), w_scale[col]));
        } else {
            reinterpret_cast<float*>(out)[idx] =
                __fmul_rn(__fmul_rn(__int2float_rn(acc), a_scale[row]), w_scale[col]);
        }
    }
}

cudaError_t launch_int8_generic(int epi, const int8_t* a, const int8_t* b, void* out, float scale,
                                const float* a_scale, const float* w_scale, uint32_t m, uint32_t n,
                                uint32_t k, cudaStream_t stream)
{
    dim3 block(16, 16), grid((n + 15) / 16, (m + 15) / 16);
    if (epi == EPI_SCALAR)
        int8_generic_kernel<EPI_SCALAR><<<grid, block, 0, stream>>>(a, b, out, scale, a_scale,
                                                                     w_scale, m, n, k);
    else if (epi == EPI_ROWCOL)
        int8_generic_kernel<EPI_ROWCOL><<<grid, block, 0, stream>>>(a, b, out, scale, a_scale,
                                                                     w_scale, m, n, k);
    else if (epi == EPI_ROWCOL_F16)
        int8_generic_kernel<EPI_ROWCOL_F16><<<grid, block, 0, stream>>>(a, b, out, scale, a_scale,
                                                                         w_scale, m, n, k);
    else
        int8_generic_kernel<EPI_S32><<<grid, block, 0, stream>>>(a, b, out, scale, a_scale, w_scale,
                                                                  m, n, k);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- dequantising GEMM, any shape
struct DqGenericArgs {
    DqProblem probs[3];
};

// Signed nibble kk of column j -> f16(q) * f16(scale) rounded to f16 (the reference's
// cvt.rn.f16 + mul.f16 chain, kaio-ops/src/matmul_int4_kernel.rs:655-713), widened to f32.
__device__ __forceinline__ float dequant_s4_ref(const uint32_t* w, const __half* scales, uint32_t kk,
                                                uint32_t j, uint32_t n, uint32_t k_words)
{
    const uint32_t word = w[(kk >> 3) + (size_t)j * k_words];
    const int32_t q = ((int32_t)(word << (28 - 4 * (kk & 7)))) >> 28;
    const __half raw = __int2half_rn(q);
    const __half sc = scales[(size_t)(kk >> 7) * n + j];
    return __half2float(__hmul(raw, sc));
}

template <int WFMT>
__global__ void __launch_bounds__(256)
dq_generic_kernel(const __half* __restrict__ x, const DqGenericArgs args, int out_f16,
                  int post_scale, uint32_t m, uint32_t n, uint32_t k)
{
    constexpr int T = 16, KC = 64;
    __shared__ float xs[T][KC + 1];
    __shared__ float ws[KC][T + 1];
    const DqProblem& pr = args.probs[blockIdx.z];
    const uint32_t tx = threadIdx.x, ty = threadIdx.y;
    const uint32_t row = blockIdx.y * T + ty, col = blockIdx.x * T + tx;
    const uint32_t k_words = k >> 3;
    float acc = 0.0f;
    for (uint32_t k0 = 0; k0 < k; k0 += KC) {
        for (uint32_t kk = tx; kk < KC; kk += T)
            xs[ty][kk] =
                (row < m && k0 + kk < k) ? __half2float(x[(size_t)row * k + k0 + kk]) : 0.0f;
        for (uint32_t kk = ty; kk < KC; kk += T) {
            float wv = 0.0f;
            if (col < n && k0 + kk < k) {
                if (WFMT == WFMT_S8_ROWMAJOR)
                    wv = (float)reinterpret_cast<const int8_t*>(pr.w)[(size_t)(k0 + kk) * n + col];
                else if (WFMT == WFMT_F16)
                    wv = __half2float(reinterpret_cast<const __half*>(pr.w)[(size_t)(k0 + kk) * n + col]);
                else
                    wv = dequant_s4_ref(reinterpret_cast<const uint32_t*>(pr.w), pr.scales, k0 + kk,
                                        col, n, k_words);
            }
            ws[kk][tx] = wv;
        }
        __syncthreads();
        const uint32_t kmax = (k - k0) < KC ? (k - k0) : KC;
        for (uint32_t kk = 0; kk < kmax; ++kk)
            acc = __fadd_rn(acc, __fmul_rn(xs[ty][kk], ws[kk][tx]));
        __syncthreads();
    }
    if (row < m && col < n) {
        const size_t idx = (size_t)row * n + col;
        float r = acc;
        if (post_scale)
            r = __fmul_rn(acc, pr.col_scale ? pr.col_scale[col] : pr.scale);
        if (out_f16)
            reinterpret_cast<__half*>(pr.out)[idx] = __float2half_rn(r);
        else
            reinterpret_cast<float*>(pr.out)[idx] = r;
    }
}

cudaError_t launch_dq_generic(int wfmt, const __half* x, const DqProblem* probs, int num_probs,
                              bool out_f16, bool post_scale, uint32_t m, uint32_t n, uint32_t k,
                              cudaStream_t stream)
{
    DqGenericArgs args;
    for (int i = 0; i < 3; ++i)
        args.probs[i] = probs[i < num_probs ? i : 0];
    dim3 block(16, 16), grid((n + 15) / 16, (m + 15) / 16, num_probs);
    if (wfmt == WFMT_S8_ROWMAJOR)
        dq_generic_kernel<WFMT_S8_ROWMAJOR><<<grid, block, 0, stream>>>(x, args, out_f16, post_scale,
                                                                         m, n, k);
    else if (wfmt == WFMT_F16)
        dq_generic_kernel<WFMT_F16><<<grid, block, 0, stream>>>(x, args, out_f16, post_scale, m, n, k);
    else
        dq_generic_kernel<WFMT_S4_PACKED><<<grid, block, 0, stream>>>(x, args, out_f16, post_scale,
                                                                       m, n, k);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- attention, any shape
// One warp per query row: scores for the whole key range in shared memory, f32 softmax with
// max subtraction and a true -inf mask, then P.V -- the arithmetic of
// kaio-ops/tests/common/mod.rs:163-235.
constexpr int ATTN_WARPS = 4;

__global__ void __launch_bounds__(ATTN_WARPS * 32)
attention_generic_kernel(const AttnParams p)
{
    extern __shared__ float sm[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* scores = sm + (size_t)warp * (p.seq_k + p.d_k);
    float* qrow = scores + p.seq_k;
    const uint32_t bh = blockIdx.y;
    const uint32_t b = bh / p.heads, h = bh % p.heads;
    const uint32_t i = blockIdx.x * ATTN_WARPS + warp;
    if (i >= p.seq_q)
        return;
    const __half* q = p.q + b * p.q_batch + h * p.q_head + (size_t)i * p.q_row;
    const __half* kbase = p.k + b * p.k_batch + h * p.k_head;
    const __half* vbase = p.v + b * p.v_batch + h * p.v_head;
    const float inv_sqrt_dk = 1.0f / sqrtf((float)p.d_k);

    for (uint32_t d = lane; d < p.d_k; d += 32)
        qrow[d] = __half2float(q[d]);
    __syncwarp();

    float mx = -INFINITY;
    for (uint32_t j = lane; j < p.seq_k; j += 32) {
        const __half* kr = kbase + (size_t)j * p.k_row;
        float dot = 0.0f;
        for (uint32_t d = 0; d < p.d_k; ++d)
            dot = __fadd_rn(dot, __fmul_rn(qrow[d], __half2float(kr[d])));
        float s = __fmul_rn(dot, inv_sqrt_dk);
        if (p.causal && j > i)
            s = -INFINITY;
        scores[j] = s;
        mx = fmaxf(mx, s);
    }
    for (int o = 16; o > 0; o >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
    for (uint32_t j = lane; j < p.seq_k; j += 32) {
        const float s = scores[j];
        const float e = (s == -INFINITY) ? 0.0f : expf(s - mx);
        scores[j] = e;
        sum += e;
    }
    for (int o = 16; o > 0; o >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncwarp();
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    for (uint32_t d = lane; d < p.d_v; d += 32) {
        float o = 0.0f;
        for (uint32_t j = 0; j < p.seq_k; ++j)
            o = fmaf(scores[j] * inv, __half2float(vbase[(size_t)j * p.v_row + d]), o);
        const size_t oi = b * p.o_batch + h * p.o_head + (size_t)i * p.o_row + d;
        if (p.out_f16)
            reinterpret_cast<__half*>(p.out)[oi] = __float2half_rn(o);
        else
            reinterpret_cast<float*>(p.out)[oi] = o;
    }
}

cudaError_t launch_attention_generic(const AttnParams& p, cudaStream_t stream)
{
    const size_t smem = (size_t)ATTN_WARPS * (p.seq_k + p.d_k) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(attention_generic_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem);
        if (err != cudaSuccess)
            return err;
    }
    dim3 grid((p.seq_q + ATTN_WARPS - 1) / ATTN_WARPS, p.batch * p.heads);
    attention_generic_kernel<<<grid, ATTN_WARPS * 32, smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace kaio
