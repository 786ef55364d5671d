// kaio_ops.hpp -- header-only C++ mirror of the `kaio-ops` quantized entry points over the C ABI
// of libkaio_b200.so.  Names, argument order and error behaviour follow the Rust functions
// (kaio-ops/src/lib.rs:92-123): `GpuBuffer<T>` is a non-owning (device pointer, length) view here,
// `KaioDevice` carries the ordinal and the stream, errors are thrown as `KaioError` with the
// reference's message text.  For C++ hosts that want the reference's call shapes without Rust.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "kaio_b200.h"

namespace kaio_ops {

// kaio-runtime/src/error.rs:4-37
struct KaioError : std::runtime_error {
    int32_t code;
    KaioError(int32_t c, const std::string& msg) : std::runtime_error(msg), code(c) {}
    bool is_invalid_config() const { return code == KAIO_B200_ERR_INVALID_CONFIG; }
};

// kaio-runtime/src/buffer.rs:31-101 (view only: the caller owns the allocation)
template <typename T>
struct GpuBuffer {
    T* ptr = nullptr;
    size_t length = 0;
    GpuBuffer() = default;
    GpuBuffer(T* p, size_t n) : ptr(p), length(n) {}
    size_t len() const { return length; }
};

// kaio-runtime/src/device.rs:59-115
struct KaioDevice {
    int ordinal = 0;
    void* stream = nullptr;  // cudaStream_t / CUstream; nullptr = default stream
    explicit KaioDevice(int ord = 0, void* s = nullptr) : ordinal(ord), stream(s) {}
};

using f16 = kaio_f16;  // IEEE binary16 bits

inline void check(int32_t code)
{
    if (code != KAIO_B200_OK)
        throw KaioError(code, kaio_b200_last_error());
}

// kaio-ops/src/matmul_int8_kernel.rs:1468-1477
inline void matmul_int8(const KaioDevice& device, const GpuBuffer<const int8_t>& a,
                        const GpuBuffer<const int8_t>& b, GpuBuffer<float>& c, float scale, uint32_t m,
                        uint32_t n, uint32_t k)
{
    check(kaio_b200_matmul_int8(a.ptr, a.len(), b.ptr, b.len(), c.ptr, c.len(), scale, m, n, k,
                                device.stream));
}

// kaio-ops/src/matmul_int4_kernel.rs:2126-2136
// kaio_ops::matmul_tc / matmul_tc_async (kaio-ops/src/matmul_tc_kernel.rs:1583, matmul_tc_async_kernel.rs)
inline void matmul_tc(const KaioDevice& device, const GpuBuffer<const f16>& a, const GpuBuffer<const f16>& b,
                      GpuBuffer<float>& c, uint32_t m, uint32_t n, uint32_t k)
{
    check(kaio_b200_matmul_tc(a.ptr, a.len(), b.ptr, b.len(), c.ptr, c.len(), m, n, k, device.stream));
}

inline void matmul_tc_async(const KaioDevice& device, const GpuBuffer<const f16>& a,
                            const GpuBuffer<const f16>& b, GpuBuffer<float>& c, uint32_t m, uint32_t n,
                            uint32_t k)
{
    check(kaio_b200_matmul_tc_async(a.ptr, a.len(), b.ptr, b.len(), c.ptr, c.len(), m, n, k, device.stream));
}

inline void matmul_int4(const KaioDevice& device, const GpuBuffer<const f16>& a,
                        const GpuBuffer<const uint32_t>& b_packed, const GpuBuffer<const f16>& scales,
                        GpuBuffer<float>& c, uint32_t m, uint32_t n, uint32_t k, uint32_t group_size)
{
    check(kaio_b200_matmul_int4(a.ptr, a.len(), b_packed.ptr, b_packed.len(), scales.ptr, scales.len(),
                                c.ptr, c.len(), m, n, k, group_size, device.stream));
}

// kaio-ops/src/qkv_project_int8_kernel.rs:2008-2023
inline void qkv_project_int8(const KaioDevice& device, const GpuBuffer<const f16>& x,
                             const GpuBuffer<const int8_t>& w_q, const GpuBuffer<const int8_t>& w_k,
                             const GpuBuffer<const int8_t>& w_v, float scale_q, float scale_k,
                             float scale_v, GpuBuffer<f16>& q_out, GpuBuffer<f16>& k_out,
                             GpuBuffer<f16>& v_out, uint32_t m, uint32_t n, uint32_t k)
{
    check(kaio_b200_qkv_project_int8(x.ptr, x.len(), w_q.ptr, w_q.len(), w_k.ptr, w_k.len(), w_v.ptr,
                                     w_v.len(), scale_q, scale_k, scale_v, q_out.ptr, q_out.len(),
                                     k_out.ptr, k_out.len(), v_out.ptr, v_out.len(), m, n, k,
                                     device.stream));
}

// kaio-ops/src/qkv_project_int4_kernel.rs:1495-1511
inline void qkv_project_int4(const KaioDevice& device, const GpuBuffer<const f16>& x,
                             const GpuBuffer<const uint32_t>& w_q_packed,
                             const GpuBuffer<const uint32_t>& w_k_packed,
                             const GpuBuffer<const uint32_t>& w_v_packed,
                             const GpuBuffer<const f16>& scales_q, const GpuBuffer<const f16>& scales_k,
                             const GpuBuffer<const f16>& scales_v, GpuBuffer<f16>& q_out,
                             GpuBuffer<f16>& k_out, GpuBuffer<f16>& v_out, uint32_t m, uint32_t n,
                             uint32_t k, uint32_t group_size)
{
    check(kaio_b200_qkv_project_int4(x.ptr, x.len(), w_q_packed.ptr, w_q_packed.len(), w_k_packed.ptr,
                                     w_k_packed.len(), w_v_packed.ptr, w_v_packed.len(), scales_q.ptr,
                                     scales_q.len(), scales_k.ptr, scales_k.len(), scales_v.ptr,
                                     scales_v.len(), q_out.ptr, q_out.len(), k_out.ptr, k_out.len(),
                                     v_out.ptr, v_out.len(), m, n, k, group_size, device.stream));
}

// kaio-ops/src/attention_tc_kernel.rs:2240-2254
inline void attention_tc(const KaioDevice& device, const GpuBuffer<const f16>& q,
                         const GpuBuffer<const f16>& k, const GpuBuffer<const f16>& v,
                         GpuBuffer<float>& out, uint32_t seq_q, uint32_t seq_k, uint32_t d_k,
                         uint32_t d_v)
{
    check(kaio_b200_attention_tc(q.ptr, q.len(), k.ptr, k.len(), v.ptr, v.len(), out.ptr, out.len(),
                                 seq_q, seq_k, d_k, d_v, 0, device.stream));
}

// kaio-ops/src/attention_tc_kernel.rs:2257-2271
inline void attention_tc_causal(const KaioDevice& device, const GpuBuffer<const f16>& q,
                                const GpuBuffer<const f16>& k, const GpuBuffer<const f16>& v,
                                GpuBuffer<float>& out, uint32_t seq_q, uint32_t seq_k, uint32_t d_k,
                                uint32_t d_v)
{
    check(kaio_b200_attention_tc(q.ptr, q.len(), k.ptr, k.len(), v.ptr, v.len(), out.ptr, out.len(),
                                 seq_q, seq_k, d_k, d_v, 1, device.stream));
}

// The `fused_silu_gate` user kernel's launch wrapper (examples/fused_silu_gate/src/main.rs:13-21,
// called as `fused_silu_gate::launch(&device, &x, &gate, &mut out, n)` at :59).
inline void fused_silu_gate(const KaioDevice& device, const GpuBuffer<const float>& x,
                            const GpuBuffer<const float>& gate, GpuBuffer<float>& out, uint32_t n)
{
    check(kaio_b200_silu_gate_f32(x.ptr, x.len(), gate.ptr, gate.len(), out.ptr, out.len(), n,
                                  device.stream));
}

}  // namespace kaio_ops
