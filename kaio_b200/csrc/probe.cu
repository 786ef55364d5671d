// Tensor-pipe rate probe: how fast does this GPU retire dense tcgen05.mma kind::i8 work when
// nothing else is in the way?  Every SM runs one CTA whose elected thread issues `iters`
// M128 N256 K32 MMAs back to back on zeroed operands in shared memory (no TMA, no epilogue),
// so the result is the INT8 tensor peak a GEMM kernel on this part can be measured against:
// 128 * 256 * 32 multiply-accumulates per instruction per SM.  bench.py runs it beside the W8A8
// GEMMs and divides by the SM clock it samples, which gives MAC per clock per SM.
#include "common.cuh"
#include "kernels.h"

namespace kaio {
namespace probe {

constexpr int SMEM_BYTES = 1024 + 128 * 128 + 128 * 256;  // A [128][128 B], B [128 k][256 B], zeros
constexpr uint32_t IDESC = make_idesc(/*d=s32*/ 2, /*a=s8*/ 1, /*b=s8*/ 1, /*a K-major*/ 0,
                                      /*b K-major*/ 0, 128, 256);

__global__ void __launch_bounds__(128, 1) int8_mma_rate_kernel(uint32_t iters, uint32_t* status)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;
    for (uint32_t i = threadIdx.x; i < (SMEM_BYTES - 1024) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(gen)[i] = 0;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    fence_proxy_async_smem();
    if (threadIdx.x < 32) {
        tmem_alloc<256>(smem_u32(&tmem_slot));
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x < 32) {
        // K-major operands, 128-byte swizzle: four K32 steps inside a 128-byte row
        const uint64_t a_desc = make_smem_desc_sw128(base, 16, 1024);
        const uint64_t b_desc = make_smem_desc_sw128(base + 128 * 128, 16, 1024);
        if (elect_one()) {
#pragma unroll 8
            for (uint32_t i = 0; i < iters; ++i)
                umma_i8(tmem, a_desc + (uint64_t)((i & 3u) * 2), b_desc + (uint64_t)((i & 3u) * 2),
                        IDESC, 1u);
            umma_commit(smem_u32(&bar));
        }
        __syncwarp();
        (void)mbar_wait_bounded(smem_u32(&bar), 0, &abort_flag, status, 98, KERNEL_SELFTEST);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after_sync();
        tmem_dealloc<256>(tmem);
    }
}

}  // namespace probe

cudaError_t launch_int8_mma_rate(const DeviceCtx& ctx, uint32_t iters, cudaStream_t stream)
{
    using namespace probe;
    static bool attr_set[64] = {};
    if (!attr_set[ctx.device]) {
        cudaError_t err = cudaFuncSetAttribute(int8_mma_rate_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (err != cudaSuccess)
            return err;
        attr_set[ctx.device] = true;
    }
    int8_mma_rate_kernel<<<ctx.num_sms, 128, SMEM_BYTES, stream>>>(iters, ctx.status);
    return cudaGetLastError();
}

}  // namespace kaio
