// Sum of the f32 partial outputs of a row-parallel (K-sharded) GEMM.  The GEMM kernels of every
// rank store their partial tiles straight into staging slots of the owning rank (peer memory,
// slot index = source rank); after the ranks have met at a barrier, this kernel adds the slots
// in ascending rank order (so every run and every rank produces the same bits) and stores the
// sum to one or several destinations, which may again be peer memory (the all-gather half of a
// two-step all-reduce).  A streaming pass: (world + copies) * 4 bytes per element.
// With a multicast destination (an address of an NVLink multicast object that every rank's output
// buffer is bound to) the sum leaves the GPU once, as multimem.st, and the switch delivers it to
// every rank: (world + 1) * 4 bytes per element and 1/world of the egress.
// KAIO is single-device; there is no reference counterpart.
#include "kernels.h"

namespace kaio {

struct SumOut {
    float* ptrs[8];
};

// slots: [world][rows][cols] f32.  out_d[row * out_ld + out_col0 + c] = sum_s slots[s][row][c].
// cols, out_ld, out_col0 are multiples of 4 and all bases 16-byte aligned.
// MULTICAST: outs.ptrs[0] is a multicast address; one multimem.st per vector.
template <bool MULTICAST>
__global__ void __launch_bounds__(256)
sum_partials_kernel(const float* __restrict__ slots, uint32_t world, uint32_t rows, uint32_t cols,
                    SumOut outs, uint32_t num_out, uint64_t out_ld, uint32_t out_col0)
{
    const uint32_t v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= cols / 4)
        return;
    const size_t slot_f4 = (size_t)rows * cols / 4;
    const float4* base = reinterpret_cast<const float4*>(slots) + v;
    for (uint32_t r = blockIdx.y; r < rows; r += gridDim.y) {
        const float4* src = base + (size_t)r * (cols / 4);
        // the slots were written by other GPUs: read them from L2, never from a stale L1 line
        float4 acc = __ldcg(src);
        for (uint32_t s = 1; s < world; ++s) {
            const float4 t = __ldcg(src + s * slot_f4);
            acc.x += t.x;
            acc.y += t.y;
            acc.z += t.z;
            acc.w += t.w;
        }
        const size_t o = (size_t)r * out_ld + out_col0 + (size_t)v * 4;
        if constexpr (MULTICAST) {
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                         :
                         : "l"(outs.ptrs[0] + o), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w)
                         : "memory");
        } else {
            for (uint32_t d = 0; d < num_out; ++d)
                *reinterpret_cast<float4*>(outs.ptrs[d] + o) = acc;
        }
    }
}

// All-reduce of a [rows, ld] f32 buffer that every rank holds at the same offset of a symmetric
// allocation bound to an NVLink multicast object: this rank reduces ITS column block
// [col0, col0 + cols) -- multimem.ld_reduce pulls the element from every rank and adds inside the
// switch, so one reduced copy crosses this GPU's link instead of world - 1 partial ones -- and
// multimem.st delivers the sum to every rank's output.  One reducer per element: all ranks end
// with the same bits.  Per rank and direction (world - 1) / world + 1 / world of the buffer
// crosses NVLink; the peer-store form above moves 2 (world - 1) / world of it.
__global__ void __launch_bounds__(256)
multimem_allreduce_f32_kernel(const float* mc_in, float* mc_out, uint32_t rows, uint32_t cols,
                              uint64_t ld, uint32_t col0)
{
    const uint32_t v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= cols / 4)
        return;
    // four rows in flight per thread: a reduction is a round trip through the switch
    for (uint32_t r = blockIdx.y; r < rows; r += 4 * gridDim.y) {
        float4 acc[4];
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u) {
            const uint32_t ru = r + u * gridDim.y;
            if (ru < rows) {
                const size_t o = (size_t)ru * ld + col0 + (size_t)v * 4;
                asm volatile(
                    "multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                    : "=f"(acc[u].x), "=f"(acc[u].y), "=f"(acc[u].z), "=f"(acc[u].w)
                    : "l"(mc_in + o)
                    : "memory");
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u) {
            const uint32_t ru = r + u * gridDim.y;
            if (ru < rows) {
                const size_t o = (size_t)ru * ld + col0 + (size_t)v * 4;
                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                             :
                             : "l"(mc_out + o), "f"(acc[u].x), "f"(acc[u].y), "f"(acc[u].z),
                               "f"(acc[u].w)
                             : "memory");
            }
        }
    }
}

cudaError_t launch_multimem_allreduce_f32(const float* mc_in, float* mc_out, uint32_t rows,
                                          uint32_t cols, uint64_t ld, uint32_t col0,
                                          cudaStream_t stream)
{
    const uint32_t gx = (cols / 4 + 255) / 256;
    uint32_t gy = (148 * 8 + gx - 1) / gx;
    gy = gy > rows ? rows : gy;
    gy = gy < 1 ? 1 : (gy > 65535 ? 65535 : gy);
    multimem_allreduce_f32_kernel<<<dim3(gx, gy, 1), 256, 0, stream>>>(mc_in, mc_out, rows, cols, ld,
                                                                       col0);
    return cudaGetLastError();
}

cudaError_t launch_sum_partials(const float* slots, uint32_t world, uint32_t rows, uint32_t cols,
                                float* const* outs, uint32_t num_out, uint64_t out_ld,
                                uint32_t out_col0, bool multicast, cudaStream_t stream)
{
    SumOut so = {};
    for (uint32_t d = 0; d < num_out && d < 8; ++d)
        so.ptrs[d] = outs[d];
    const uint32_t gx = (cols / 4 + 255) / 256;
    uint32_t gy = (148 * 8 + gx - 1) / gx;
    gy = gy > rows ? rows : gy;
    gy = gy < 1 ? 1 : (gy > 65535 ? 65535 : gy);
    if (multicast)
        sum_partials_kernel<true><<<dim3(gx, gy, 1), 256, 0, stream>>>(slots, world, rows, cols, so,
                                                                       1, out_ld, out_col0);
    else
        sum_partials_kernel<false><<<dim3(gx, gy, 1), 256, 0, stream>>>(slots, world, rows, cols, so,
                                                                        num_out, out_ld, out_col0);
    return cudaGetLastError();
}

}  // namespace kaio
