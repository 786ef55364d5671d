// The SiLU-gate arithmetic shared by the stand-alone pass (silu_gate.cu) and the GEMM epilogue that
// applies it to its own accumulators (dq_gemm.cu): one definition, so both give the same bits.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace kaio {

// The f16 form rounds its result to 11 significant bits, so the hardware approximations
// (ex2.approx inside __expf, rcp.approx inside __fdividef; a few f32 units in the last place)
// are invisible after the rounding except on rare ties; with the IEEE divide and expf the pass
// is bound by instruction issue, not by HBM.
__device__ __forceinline__ float silu_gate1_fast(float x, float g)
{
    return __fdividef(x, 1.0f + __expf(-x)) * g;
}

// two f16 pairs in, one f16 pair out: f32 arithmetic, one rounding
__device__ __forceinline__ uint32_t silu_gate_h2(uint32_t xw, uint32_t gw)
{
    const float2 xf = __half22float2(*reinterpret_cast<const __half2*>(&xw));
    const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(&gw));
    const __half2 r = __floats2half2_rn(silu_gate1_fast(xf.x, gf.x), silu_gate1_fast(xf.y, gf.y));
    return *reinterpret_cast<const uint32_t*>(&r);
}

}  // namespace kaio
