// Fused SiLU-gate, out = x * sigmoid(x) * gate: the gated activation between the up/gate
// projections and the down projection of a feed-forward block.  KAIO writes it as a user kernel
// (examples/fused_silu_gate/src/main.rs:13-21, f32, sigmoid as 1/(1+exp(-x))); the f32 form
// here is that kernel, the f16 form is the one the quantized FFN chain uses between two W4A16
// GEMMs (f16 in, f32 arithmetic, one rounding to f16 on the way out; row strides so that the
// two inputs may be the halves of one [rows, 2*cols] projection output).
// Both are streaming passes bound by HBM: 12 bytes per element (f32), 6 bytes (f16).
#include "kernels.h"
#include "silu.cuh"

namespace kaio {

__device__ __forceinline__ float silu_gate1(float x, float g)
{
    const float sig = __fdiv_rn(1.0f, 1.0f + expf(-x));
    return x * sig * g;
}

// f32, contiguous.  VEC = 4: 16-byte accesses, n4 = n / 4 vectors; the tail (n % 4) is handled
// by the scalar instantiation launched on the remainder.
template <int VEC>
__global__ void __launch_bounds__(256)
silu_gate_f32_kernel(const float* __restrict__ x, const float* __restrict__ gate,
                     float* __restrict__ out, size_t count)
{
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if constexpr (VEC == 4) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const float4* g4 = reinterpret_cast<const float4*>(gate);
        float4* o4 = reinterpret_cast<float4*>(out);
        // two vectors in flight per thread
        for (; i + stride < count; i += 2 * stride) {
            const float4 a0 = __ldg(x4 + i), b0 = __ldg(g4 + i);
            const float4 a1 = __ldg(x4 + i + stride), b1 = __ldg(g4 + i + stride);
            o4[i] = make_float4(silu_gate1(a0.x, b0.x), silu_gate1(a0.y, b0.y),
                                silu_gate1(a0.z, b0.z), silu_gate1(a0.w, b0.w));
            o4[i + stride] = make_float4(silu_gate1(a1.x, b1.x), silu_gate1(a1.y, b1.y),
                                         silu_gate1(a1.z, b1.z), silu_gate1(a1.w, b1.w));
        }
        if (i < count) {
            const float4 a0 = __ldg(x4 + i), b0 = __ldg(g4 + i);
            o4[i] = make_float4(silu_gate1(a0.x, b0.x), silu_gate1(a0.y, b0.y),
                                silu_gate1(a0.z, b0.z), silu_gate1(a0.w, b0.w));
        }
    } else {
        for (; i < count; i += stride)
            out[i] = silu_gate1(__ldg(x + i), __ldg(gate + i));
    }
}

__device__ __forceinline__ uint4 silu_gate_h8(const uint4& a, const uint4& b)
{
    return make_uint4(silu_gate_h2(a.x, b.x), silu_gate_h2(a.y, b.y), silu_gate_h2(a.z, b.z),
                      silu_gate_h2(a.w, b.w));
}

// f16, [rows, cols] with row strides (elements).  blockIdx.x / threadIdx.x walk the columns,
// blockIdx.y strides over the rows (no index division).  VEC = 8: cols, the strides and the
// base addresses are multiples of 8 halves (16 bytes), one thread per 8 columns and two rows in
// flight per thread; VEC = 1: any shape, one element per thread.
template <int VEC>
__global__ void __launch_bounds__(256)
silu_gate_f16_kernel(const __half* __restrict__ x, const __half* __restrict__ gate,
                     __half* __restrict__ out, uint32_t rows, uint32_t cols, uint32_t x_ld,
                     uint32_t gate_ld, uint32_t out_ld)
{
    const uint32_t vpr = cols / VEC;  // vectors per row
    const uint32_t v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= vpr)
        return;
    const uint32_t c = v * VEC;
    const uint32_t rs = gridDim.y;
    uint32_t r = blockIdx.y;
    if constexpr (VEC == 8) {
        for (; r + rs < rows; r += 2 * rs) {
            const size_t r1 = (size_t)r + rs;
            const uint4 a0 = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * x_ld + c));
            const uint4 b0 = __ldg(reinterpret_cast<const uint4*>(gate + (size_t)r * gate_ld + c));
            const uint4 a1 = __ldg(reinterpret_cast<const uint4*>(x + r1 * x_ld + c));
            const uint4 b1 = __ldg(reinterpret_cast<const uint4*>(gate + r1 * gate_ld + c));
            *reinterpret_cast<uint4*>(out + (size_t)r * out_ld + c) = silu_gate_h8(a0, b0);
            *reinterpret_cast<uint4*>(out + r1 * out_ld + c) = silu_gate_h8(a1, b1);
        }
        if (r < rows) {
            const uint4 a0 = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * x_ld + c));
            const uint4 b0 = __ldg(reinterpret_cast<const uint4*>(gate + (size_t)r * gate_ld + c));
            *reinterpret_cast<uint4*>(out + (size_t)r * out_ld + c) = silu_gate_h8(a0, b0);
        }
    } else {
        for (; r < rows; r += rs)
            out[(size_t)r * out_ld + c] = __float2half_rn(silu_gate1_fast(
                __half2float(x[(size_t)r * x_ld + c]), __half2float(gate[(size_t)r * gate_ld + c])));
    }
}

// The same pass on a projection whose columns alternate in blocks of 64 between the two inputs
// (block 2b = x columns [64b, 64b+64), block 2b+1 = the gate columns of the same range): the
// layout the fused gate|up GEMM takes its weights in.  cols % 64 == 0, 16-byte aligned rows.
__global__ void __launch_bounds__(256)
silu_gate_f16_interleaved_kernel(const __half* __restrict__ gu, __half* __restrict__ out,
                                 uint32_t rows, uint32_t cols, uint32_t gu_ld, uint32_t out_ld)
{
    const uint32_t v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= cols / 8)
        return;
    const uint32_t c = v * 8;
    const uint32_t src = (c >> 6) * 128 + (c & 63u);
    for (uint32_t r = blockIdx.y; r < rows; r += gridDim.y) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(gu + (size_t)r * gu_ld + src));
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(gu + (size_t)r * gu_ld + src + 64));
        *reinterpret_cast<uint4*>(out + (size_t)r * out_ld + c) = silu_gate_h8(a, b);
    }
}

// Column blocks x row slots: about 8 resident blocks of 256 threads on each of the 148 SMs.
static dim3 grid_2d(uint32_t rows, uint32_t vectors_per_row)
{
    const uint32_t gx = (vectors_per_row + 255) / 256;
    uint32_t gy = (148 * 8 + gx - 1) / gx;
    gy = gy < 1 ? 1 : (gy > rows ? rows : gy);
    gy = gy > 65535 ? 65535 : gy;
    return dim3(gx, gy, 1);
}

static int grid_for(size_t work_items)
{
    // up to 8 resident blocks of 256 threads on each of the 148 SMs
    const size_t blocks = (work_items + 255) / 256;
    const size_t cap = 148 * 8;
    return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

cudaError_t launch_silu_gate_f32(const float* x, const float* gate, float* out, size_t n,
                                 cudaStream_t stream)
{
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gate) |
                           reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    size_t done = 0;
    if (aligned && n >= 4) {
        const size_t n4 = n / 4;
        silu_gate_f32_kernel<4><<<grid_for((n4 + 1) / 2), 256, 0, stream>>>(x, gate, out, n4);
        done = n4 * 4;
    }
    if (done < n)
        silu_gate_f32_kernel<1><<<grid_for(n - done), 256, 0, stream>>>(x + done, gate + done,
                                                                        out + done, n - done);
    return cudaGetLastError();
}

cudaError_t launch_silu_gate_f16(const __half* x, const __half* gate, __half* out, uint32_t rows,
                                 uint32_t cols, uint32_t x_ld, uint32_t gate_ld, uint32_t out_ld,
                                 cudaStream_t stream)
{
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gate) |
                       reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                     ((cols | x_ld | gate_ld | out_ld) & 7) == 0;
    if (vec)
        silu_gate_f16_kernel<8><<<grid_2d(rows, cols / 8), 256, 0, stream>>>(
            x, gate, out, rows, cols, x_ld, gate_ld, out_ld);
    else
        silu_gate_f16_kernel<1><<<grid_2d(rows, cols), 256, 0, stream>>>(
            x, gate, out, rows, cols, x_ld, gate_ld, out_ld);
    return cudaGetLastError();
}

cudaError_t launch_silu_gate_f16_interleaved(const __half* gu, __half* out, uint32_t rows,
                                             uint32_t cols, uint32_t gu_ld, uint32_t out_ld,
                                             cudaStream_t stream)
{
    silu_gate_f16_interleaved_kernel<<<grid_2d(rows, cols / 8), 256, 0, stream>>>(gu, out, rows, cols,
                                                                                 gu_ld, out_ld);
    return cudaGetLastError();
}

}  // namespace kaio
