// Quantisers on the GPU: the step in front of the quantized GEMMs.  In KAIO these run on the
// host in the examples (symmetric INT8: examples/int8_matmul/src/main.rs:41-61; group-wise INT4
// "GPTQ-lite" + packer: examples/int4_matmul/src/main.rs:48-99); the arithmetic here is the same,
// operation for operation (IEEE f32 divide, round half away from zero, clamp), so the outputs are
// bit-identical to the host functions.  Both kernels are HBM-bound streaming passes.
#include "kernels.h"

namespace kaio {

// One block per row: scale[i] = max_k |x[i,k]| / 127 (1 if the row is all zero),
// q[i,k] = clamp(round(x[i,k] / scale[i]), -127, 127).
__global__ void __launch_bounds__(256)
quantize_rows_int8_kernel(const float* __restrict__ x, int8_t* __restrict__ q,
                          float* __restrict__ scale, uint32_t m, uint32_t k)
{
    __shared__ float red[8];
    const uint32_t row = blockIdx.x;
    if (row >= m)
        return;
    const float* xr = x + (size_t)row * k;
    float mx = 0.0f;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x)
        mx = fmaxf(mx, fabsf(xr[i]));
    for (int o = 16; o > 0; o >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w)
        mx = fmaxf(mx, red[w]);
    const float s = (mx == 0.0f) ? 1.0f : __fdiv_rn(mx, 127.0f);
    if (threadIdx.x == 0)
        scale[row] = s;
    int8_t* qr = q + (size_t)row * k;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
        const float v = fminf(fmaxf(roundf(__fdiv_rn(xr[i], s)), -127.0f), 127.0f);
        qr[i] = (int8_t)(int)v;
    }
}

// The same quantiser on f16 activations (the input of the W8A8 fused QKV projection): every f16
// widens to f32 exactly, after which the arithmetic is the one above.  One block per row; a row
// of up to 4096 values stays in registers between the max pass and the quantising pass, longer
// rows are read a second time (from L1/L2).  16-byte loads, 8-byte stores.
__global__ void __launch_bounds__(256)
quantize_rows_int8_f16_kernel(const __half* __restrict__ x, int8_t* __restrict__ q,
                              float* __restrict__ scale, uint32_t m, uint32_t k)
{
    __shared__ float red[8];
    const uint32_t row = blockIdx.x;
    if (row >= m)
        return;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * k);
    const uint32_t nvec = k >> 3;
    constexpr uint32_t CACHED = 2;
    uint4 cache[CACHED];
    __half2 mx2 = __float2half2_rn(0.0f);
#pragma unroll
    for (uint32_t j = 0; j < CACHED; ++j) {
        const uint32_t i = threadIdx.x + j * 256;
        cache[j] = make_uint4(0, 0, 0, 0);
        if (i < nvec)
            cache[j] = __ldg(xr + i);
        const __half2* h = reinterpret_cast<const __half2*>(&cache[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e)
            mx2 = __hmax2(mx2, __habs2(h[e]));
    }
    for (uint32_t i = threadIdx.x + CACHED * 256; i < nvec; i += 256) {
        const uint4 v = __ldg(xr + i);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e)
            mx2 = __hmax2(mx2, __habs2(h[e]));
    }
    float mx = fmaxf(__low2float(mx2), __high2float(mx2));  // max of |f16| values: exact
    for (int o = 16; o > 0; o >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w)
        mx = fmaxf(mx, red[w]);
    const float s = (mx == 0.0f) ? 1.0f : __fdiv_rn(mx, 127.0f);
    if (threadIdx.x == 0)
        scale[row] = s;
    uint2* qr = reinterpret_cast<uint2*>(q + (size_t)row * k);
    auto quantise8 = [&](const uint4& v) {
        const __half* h = reinterpret_cast<const __half*>(&v);
        uint32_t out[2] = {0, 0};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float f = fminf(fmaxf(roundf(__fdiv_rn(__half2float(h[e]), s)), -127.0f), 127.0f);
            out[e >> 2] |= ((uint32_t)(int)f & 0xFFu) << (8 * (e & 3));
        }
        return make_uint2(out[0], out[1]);
    };
#pragma unroll
    for (uint32_t j = 0; j < CACHED; ++j) {
        const uint32_t i = threadIdx.x + j * 256;
        if (i < nvec)
            qr[i] = quantise8(cache[j]);
    }
    for (uint32_t i = threadIdx.x + CACHED * 256; i < nvec; i += 256)
        qr[i] = quantise8(__ldg(xr + i));
}

// One warp per (column, group of 128 k): scale = max|w| / 7 (1 if zero) stored as f16;
// q = clamp(round(w / scale_f32), -8, 7) packed 8 per u32 at word (k/8) + col*(K/8).
__global__ void __launch_bounds__(256)
quantize_pack_s4_kernel(const float* __restrict__ w, uint32_t* __restrict__ packed,
                        __half* __restrict__ scales, uint32_t k, uint32_t n)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t col = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t g = blockIdx.y;
    if (col >= n)
        return;
    const uint32_t k0 = g * 128;
    // lane holds k = k0 + 4*lane .. +3 (column-strided reads; the 8 warps of a block cover 8
    // adjacent columns, so a block touches full 32-byte sectors)
    float v[4];
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = w[(size_t)(k0 + 4 * lane + i) * n + col];
        mx = fmaxf(mx, fabsf(v[i]));
    }
    for (int o = 16; o > 0; o >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float s = (mx == 0.0f) ? 1.0f : __fdiv_rn(mx, 7.0f);
    if (lane == 0)
        scales[(size_t)g * n + col] = __float2half_rn(s);
    uint32_t nib = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qi = (int)fminf(fmaxf(roundf(__fdiv_rn(v[i], s)), -8.0f), 7.0f);
        nib |= ((uint32_t)qi & 0xFu) << (4 * i);
    }
    // two lanes make one word: even lane = nibbles 0-3, odd lane = nibbles 4-7
    const uint32_t other = __shfl_xor_sync(0xffffffffu, nib, 1);
    if ((lane & 1) == 0)
        packed[(size_t)col * (k >> 3) + (k0 >> 3) + (lane >> 1)] = nib | (other << 16);
}

cudaError_t launch_quantize_rows_int8(const float* x, int8_t* q, float* scale, uint32_t m,
                                      uint32_t k, cudaStream_t stream)
{
    quantize_rows_int8_kernel<<<m, 256, 0, stream>>>(x, q, scale, m, k);
    return cudaGetLastError();
}

cudaError_t launch_quantize_rows_int8_f16(const __half* x, int8_t* q, float* scale, uint32_t m,
                                          uint32_t k, cudaStream_t stream)
{
    // k % 8 == 0 and 16-byte aligned x, 8-byte aligned q: checked by the caller
    quantize_rows_int8_f16_kernel<<<m, 256, 0, stream>>>(x, q, scale, m, k);
    return cudaGetLastError();
}

cudaError_t launch_quantize_pack_s4(const float* w, uint32_t* packed, __half* scales, uint32_t k,
                                    uint32_t n, cudaStream_t stream)
{
    dim3 grid((n + 7) / 8, k / 128);
    quantize_pack_s4_kernel<<<grid, 256, 0, stream>>>(w, packed, scales, k, n);
    return cudaGetLastError();
}

}  // namespace kaio
