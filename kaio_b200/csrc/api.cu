// C ABI of libkaio_b200.so: argument validation with the reference's contracts and error
// texts, per-device state, and dispatch to the sm_100a kernels.
//
// The validation functions restate, message for message,
//   validate_dims_int8          kaio-ops/src/matmul_int8_kernel.rs:108-150
//   validate_dims_int4          kaio-ops/src/matmul_int4_kernel.rs:112-174
//   validate_dims_qkv_int8      kaio-ops/src/qkv_project_int8_kernel.rs:1894-1953
//   validate_dims_qkv_int4      kaio-ops/src/qkv_project_int4_kernel.rs:1344-1433
//   validate_attention_tc_dims  kaio-ops/src/attention_tc_kernel.rs:139-223
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/kaio_b200.h"
#include "kernels.h"

#define KAIO_API extern "C" __attribute__((visibility("default")))

namespace kaio {

// ---------------------------------------------------------------- thread-local error state
static thread_local std::string g_last_error;
static thread_local const char* g_last_variant = "";

static int32_t fail(int32_t code, const char* fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

static int32_t fail_cuda(cudaError_t err, const char* what)
{
    return fail(KAIO_B200_ERR_CUDA, "%s: CUDA error %d (%s)", what, (int)err,
                cudaGetErrorString(err));
}

// ---------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Encoded tensor maps are a pure function of (type, base, extents, stride, box, swizzle), so the
// calling thread keeps the maps of its recent calls: a decode loop that launches the same few
// GEMMs over and over pays for cuTensorMapEncodeTiled once per operand, not once per launch.
struct TensorMapKey {
    const void* base;
    uint64_t inner, outer, stride;
    uint32_t dtype, box_inner, box_outer, swizzle;
};
struct TensorMapSlot {
    TensorMapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int TMAP_CACHE_SLOTS = 128;  // direct-mapped
static thread_local TensorMapSlot g_tmap_cache[TMAP_CACHE_SLOTS];

cudaError_t encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes,
                                 const void* base, uint64_t inner, uint64_t outer,
                                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                                 CUtensorMapSwizzle swizzle)
{
    (void)elem_bytes;
    TensorMapKey key;
    memset(&key, 0, sizeof(key));
    key.base = base;
    key.inner = inner;
    key.outer = outer;
    key.stride = row_stride_bytes;
    key.dtype = (uint32_t)dtype;
    key.box_inner = box_inner;
    key.box_outer = box_outer;
    key.swizzle = (uint32_t)swizzle;
    uint64_t h = (uint64_t)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
    h ^= (inner * 0xC2B2AE3D27D4EB4Full) ^ (outer * 0x165667B19E3779F9ull) ^
         ((uint64_t)box_inner << 40) ^ ((uint64_t)box_outer << 24) ^ ((uint64_t)swizzle << 8) ^ dtype;
    TensorMapSlot& slot = g_tmap_cache[(h >> 32) % TMAP_CACHE_SLOTS];
    if (slot.used && memcmp(&slot.key, &key, sizeof(key)) == 0) {
        *map = slot.map;
        return cudaSuccess;
    }
    EncodeTiledFn fn = get_encode_fn();
    if (!fn)
        return cudaErrorNotSupported;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    slot.key = key;
    slot.map = *map;
    slot.used = true;
    return cudaSuccess;
}

// ---------------------------------------------------------------- per-device context
constexpr int MAX_DEVICES = 64;
static DeviceCtx g_ctx[MAX_DEVICES];
static std::mutex g_ctx_mutex;

// Scratch the kernels need beyond the caller's buffers, one set per (device, stream): calls on
// different streams may overlap on the GPU, so they must not share split-K partial tiles,
// arrival counters or the dequantised-weight buffer.  Calls on one stream run in order and
// share a set.
struct StreamScratch {
    cudaStream_t stream = nullptr;
    void* workspace = nullptr;          // split-K partial sums
    size_t workspace_bytes = 0;
    uint32_t* tile_counters = nullptr;  // split-K arrival counters (self-resetting)
    size_t num_tile_counters = 0;
    void* dq_workspace = nullptr;       // dequantised f16 weights / quantised activations
    size_t dq_workspace_bytes = 0;
};
static std::vector<StreamScratch*> g_scratch[MAX_DEVICES];

// The device's context.  `device_ptr`, when given, must be memory of the current device: a
// caller that holds buffers of several devices gets an error instead of a launch on the wrong
// one (the reference checks the buffer's device ordinal the same way).
static int32_t get_ctx(DeviceCtx** out, const void* device_ptr = nullptr)
{
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess)
        return fail_cuda(err, "cudaGetDevice");
    if (dev < 0 || dev >= MAX_DEVICES)
        return fail(KAIO_B200_ERR_CUDA, "device ordinal %d out of range", dev);
    if (device_ptr != nullptr) {
        cudaPointerAttributes attr;
        err = cudaPointerGetAttributes(&attr, device_ptr);
        if (err != cudaSuccess)
            return fail_cuda(err, "cudaPointerGetAttributes");
        if ((attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) &&
            attr.device != dev)
            return fail(KAIO_B200_ERR_INVALID_CONFIG,
                        "buffer lives on device %d but the calling thread's current device is %d; "
                        "make the buffer's device current before the call",
                        attr.device, dev);
    }
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    DeviceCtx& c = g_ctx[dev];
    if (c.device < 0) {
        cudaDeviceProp prop;
        err = cudaGetDeviceProperties(&prop, dev);
        if (err != cudaSuccess)
            return fail_cuda(err, "cudaGetDeviceProperties");
        if (prop.major != 10)
            return fail(KAIO_B200_ERR_UNSUPPORTED_ARCH,
                        "kaio_b200 kernels are built for sm_100a only; device %d is sm_%d%d", dev,
                        prop.major, prop.minor);
        err = cudaMalloc(&c.status, 4 * sizeof(uint32_t));
        if (err != cudaSuccess)
            return fail_cuda(err, "cudaMalloc(status)");
        err = cudaMemset(c.status, 0, 4 * sizeof(uint32_t));
        if (err != cudaSuccess)
            return fail_cuda(err, "cudaMemset(status)");
        c.num_sms = prop.multiProcessorCount;
        c.cc_major = prop.major;
        c.cc_minor = prop.minor;
        c.device = dev;
    }
    *out = &c;
    return KAIO_B200_OK;
}

// The scratch set of (c->device, stream), created empty on first use.  Caller holds no lock.
static StreamScratch* scratch_for(DeviceCtx* c, cudaStream_t stream)
{
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    for (StreamScratch* sc : g_scratch[c->device])
        if (sc->stream == stream)
            return sc;
    StreamScratch* sc = new StreamScratch();
    sc->stream = stream;
    g_scratch[c->device].push_back(sc);
    return sc;
}

// Growing a scratch block frees the old one with cudaFree, which waits for the work in flight
// on the device, and allocates: neither is allowed while the stream is being captured into a
// CUDA graph, and a graph captured earlier keeps the old address.  So growth during a capture
// is refused; callers warm every op at its largest shape before they capture.
static int32_t refuse_growth_in_capture(cudaStream_t stream, const char* what)
{
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s would have to be allocated while the stream is being captured; run the op "
                    "once at its largest shape before capturing",
                    what);
    return KAIO_B200_OK;
}

static int32_t ensure_workspace(DeviceCtx* c, cudaStream_t stream, size_t bytes, size_t counters,
                                StreamScratch** out)
{
    StreamScratch* sc = scratch_for(c, stream);
    *out = sc;
    if (bytes <= sc->workspace_bytes && counters <= sc->num_tile_counters)
        return KAIO_B200_OK;
    int32_t rc = refuse_growth_in_capture(stream, "split-K scratch");
    if (rc)
        return rc;
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    if (bytes > sc->workspace_bytes) {
        if (sc->workspace)
            cudaFree(sc->workspace);
        sc->workspace = nullptr;
        sc->workspace_bytes = 0;
        cudaError_t err = cudaMalloc(&sc->workspace, bytes);
        if (err != cudaSuccess)
            return fail_cuda(err, "cudaMalloc(workspace)");
        sc->workspace_bytes = bytes;
    }
    if (counters > sc->num_tile_counters) {
        if (sc->tile_counters)
            cudaFree(sc->tile_counters);
        sc->tile_counters = nullptr;
        sc->num_tile_counters = 0;
        cudaError_t err = cudaMalloc(&sc->tile_counters, counters * sizeof(uint32_t));
        if (err != cudaSuccess)
            return fail_cuda(err, "cudaMalloc(counters)");
        err = cudaMemset(sc->tile_counters, 0, counters * sizeof(uint32_t));
        if (err != cudaSuccess)
            return fail_cuda(err, "cudaMemset(counters)");
        sc->num_tile_counters = counters;
    }
    return KAIO_B200_OK;
}

// The dequantised-weight workspace is written and read by the dequantising GEMM calls of one
// stream, in stream order.
static int32_t ensure_dq_workspace(DeviceCtx* c, cudaStream_t stream, size_t bytes,
                                   StreamScratch** out)
{
    StreamScratch* sc = scratch_for(c, stream);
    *out = sc;
    if (bytes <= sc->dq_workspace_bytes)
        return KAIO_B200_OK;
    int32_t rc = refuse_growth_in_capture(stream, "the dequantised-weight workspace");
    if (rc)
        return rc;
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    if (sc->dq_workspace)
        cudaFree(sc->dq_workspace);
    sc->dq_workspace = nullptr;
    sc->dq_workspace_bytes = 0;
    cudaError_t err = cudaMalloc(&sc->dq_workspace, bytes);
    if (err != cudaSuccess)
        return fail_cuda(err, "cudaMalloc(dequantised weights)");
    sc->dq_workspace_bytes = bytes;
    return KAIO_B200_OK;
}

static int32_t finish(cudaError_t err, const char* op, const char* variant)
{
    g_last_variant = variant;
    if (err != cudaSuccess)
        return fail_cuda(err, op);
    return KAIO_B200_OK;
}

// ---------------------------------------------------------------- validation
#define INVALID(...) return fail(KAIO_B200_ERR_INVALID_CONFIG, __VA_ARGS__)

static int32_t validate_int8(const char* c_kind, size_t a_len, size_t b_len, size_t c_len,
                             uint32_t m, uint32_t n, uint32_t k)
{
    if (m == 0 || n == 0 || k == 0)
        INVALID("matmul_int8 dimensions must be non-zero");
    if (k % 32 != 0)
        INVALID("matmul_int8: K must be a multiple of 32 (got %u). The "
                "mma.sync.m16n8k32.s8.s8.s32 instance shape requires K-tile "
                "size 32; K is not edge-padded inside a K-tile.",
                k);
    const size_t mk = (size_t)m * k, kn = (size_t)k * n, mn = (size_t)m * n;
    if (a_len < mk)
        INVALID("matmul_int8: A buffer too small: need %zu i8 (%u\xC3\x97%u), got %zu", mk, m, k,
                a_len);
    if (b_len < kn)
        INVALID("matmul_int8: B buffer too small: need %zu i8 (%u\xC3\x97%u), got %zu", kn, k, n,
                b_len);
    if (c_len < mn)
        INVALID("matmul_int8: C buffer too small: need %zu %s (%u\xC3\x97%u), got %zu", mn, c_kind, m,
                n, c_len);
    return KAIO_B200_OK;
}

static int32_t validate_int4(const char* c_kind, size_t a_len, size_t b_len, size_t s_len,
                             size_t c_len, uint32_t m, uint32_t n, uint32_t k, uint32_t group_size)
{
    if (m == 0 || n == 0 || k == 0)
        INVALID("matmul_int4: M, N, K dimensions must be non-zero");
    if (group_size != 128)
        INVALID("matmul_int4: group_size must be 128 (got %u). Non-128 "
                "group sizes are deferred to a follow-up sprint.",
                group_size);
    if (k % 128 != 0)
        INVALID("matmul_int4: K must be a multiple of group_size=128 (got %u). "
                "Partial groups are not supported.",
                k);
    const size_t mk = (size_t)m * k, words = (size_t)(k / 8) * n, groups = k / group_size,
                 cells = groups * n, mn = (size_t)m * n;
    if (a_len < mk)
        INVALID("matmul_int4: A buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu", mk, m, k,
                a_len);
    if (b_len < words)
        INVALID("matmul_int4: B packed buffer too small: need %zu u32 "
                "(%u cols \xC3\x97 %u K-words), got %zu",
                words, n, k / 8, b_len);
    if (s_len < cells)
        INVALID("matmul_int4: scales buffer too small: need %zu f16 "
                "(%zu groups \xC3\x97 %u cols), got %zu",
                cells, groups, n, s_len);
    if (c_len < mn)
        INVALID("matmul_int4: C buffer too small: need %zu %s (%u\xC3\x97%u), got %zu", mn, c_kind, m,
                n, c_len);
    return KAIO_B200_OK;
}

static int32_t validate_qkv_int8(size_t x_len, const size_t w_len[3], const size_t o_len[3],
                                 uint32_t m, uint32_t n, uint32_t k)
{
    if (m == 0 || n == 0 || k == 0)
        INVALID("qkv_project_int8: M, N, K dimensions must be non-zero");
    if (k % 16 != 0)
        INVALID("qkv_project_int8: K must be a multiple of K_TILE_SHARED=16 "
                "(got %u). The mma.sync.m16n8k16 instance shape requires K-tile size 16; "
                "K is not edge-padded inside a K-tile.",
                k);
    if (n % 2 != 0)
        INVALID("qkv_project_int8: N must be even (got %u). The store-out path packs "
                "adjacent f16 output pairs into one .b32; odd N would leave a ragged "
                "last column that the current store epilogue does not handle.",
                n);
    const size_t mk = (size_t)m * k, kn = (size_t)k * n, mn = (size_t)m * n;
    if (x_len < mk)
        INVALID("qkv_project_int8: X buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu", mk, m,
                k, x_len);
    static const char* wl[3] = {"W_Q", "W_K", "W_V"};
    static const char* ol[3] = {"Q_out", "K_out", "V_out"};
    for (int i = 0; i < 3; ++i)
        if (w_len[i] < kn)
            INVALID("qkv_project_int8: %s buffer too small: need %zu i8 (%u\xC3\x97%u), got %zu",
                    wl[i], kn, k, n, w_len[i]);
    for (int i = 0; i < 3; ++i)
        if (o_len[i] < mn)
            INVALID("qkv_project_int8: %s buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu",
                    ol[i], mn, m, n, o_len[i]);
    return KAIO_B200_OK;
}

static int32_t validate_qkv_int4(size_t x_len, const size_t w_len[3], const size_t s_len[3],
                                 const size_t o_len[3], uint32_t m, uint32_t n, uint32_t k,
                                 uint32_t group_size)
{
    if (m == 0 || n == 0 || k == 0)
        INVALID("qkv_project_int4: M, N, K dimensions must be non-zero");
    if (group_size != 128)
        INVALID("qkv_project_int4: group_size must be 128 (got %u). "
                "Non-128 group sizes are deferred to a follow-up sprint.",
                group_size);
    if (k % 128 != 0)
        INVALID("qkv_project_int4: K must be a multiple of group_size=128 (got %u). "
                "Partial groups are not supported.",
                k);
    if (n % 2 != 0)
        INVALID("qkv_project_int4: N must be even (got %u). The store-out path packs "
                "adjacent f16 output pairs into one .b32; odd N would leave a ragged "
                "last column that the current store epilogue does not handle.",
                n);
    const size_t mk = (size_t)m * k, words = (size_t)(k / 8) * n, groups = k / group_size,
                 cells = groups * n, mn = (size_t)m * n;
    if (x_len < mk)
        INVALID("qkv_project_int4: X buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu", mk, m,
                k, x_len);
    static const char* wl[3] = {"W_Q_packed", "W_K_packed", "W_V_packed"};
    static const char* sl[3] = {"scales_q", "scales_k", "scales_v"};
    static const char* ol[3] = {"Q_out", "K_out", "V_out"};
    for (int i = 0; i < 3; ++i)
        if (w_len[i] < words)
            INVALID("qkv_project_int4: %s buffer too small: need %zu u32 "
                    "(%u cols \xC3\x97 %u K-words), got %zu",
                    wl[i], words, n, k / 8, w_len[i]);
    for (int i = 0; i < 3; ++i)
        if (s_len[i] < cells)
            INVALID("qkv_project_int4: %s buffer too small: need %zu f16 "
                    "(%zu groups \xC3\x97 %u cols), got %zu",
                    sl[i], cells, groups, n, s_len[i]);
    for (int i = 0; i < 3; ++i)
        if (o_len[i] < mn)
            INVALID("qkv_project_int4: %s buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu",
                    ol[i], mn, m, n, o_len[i]);
    return KAIO_B200_OK;
}

static const char* WHY_CONSTRAINED =
    "Either pad inputs to valid shapes, or use the existing f32 `attention` / `attention_flash` "
    "path instead.";

static int32_t validate_attention_tc(size_t q_len, size_t k_len, size_t v_len, size_t out_len,
                                     uint32_t seq_q, uint32_t seq_k, uint32_t d_k, uint32_t d_v)
{
    if (seq_q == 0 || seq_k == 0 || d_k == 0 || d_v == 0)
        INVALID("attention_tc dimensions must be non-zero");
    if (seq_q % 16 != 0)
        INVALID("attention_tc: seq_q must be a multiple of 16 (got %u). %s", seq_q,
                WHY_CONSTRAINED);
    if (seq_k % 16 != 0)
        INVALID("attention_tc: seq_k must be a multiple of 16 (got %u). %s", seq_k,
                WHY_CONSTRAINED);
    if (d_k % 16 != 0)
        INVALID("attention_tc: d_k must be a multiple of 16 (got %u). %s", d_k, WHY_CONSTRAINED);
    if (d_v % 8 != 0)
        INVALID("attention_tc: d_v must be a multiple of 8 (got %u). %s", d_v, WHY_CONSTRAINED);
    if (seq_k > 384)
        INVALID("attention_tc: seq_k must be \xE2\x89\xA4 384 (got %u). "
                "The shared-memory scores buffer caps the sequence length; "
                "Phase 7's FlashAttention-TC lifts this constraint. %s",
                seq_k, WHY_CONSTRAINED);
    if (d_k > 128)
        INVALID("attention_tc: d_k must be \xE2\x89\xA4 128 (got %u). %s", d_k, WHY_CONSTRAINED);
    if (d_v > 128)
        INVALID("attention_tc: d_v must be \xE2\x89\xA4 128 (got %u). %s", d_v, WHY_CONSTRAINED);
    const size_t qe = (size_t)seq_q * d_k, ke = (size_t)seq_k * d_k, ve = (size_t)seq_k * d_v,
                 oe = (size_t)seq_q * d_v;
    if (q_len < qe)
        INVALID("attention_tc: Q buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu", qe, seq_q,
                d_k, q_len);
    if (k_len < ke)
        INVALID("attention_tc: K buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu", ke, seq_k,
                d_k, k_len);
    if (v_len < ve)
        INVALID("attention_tc: V buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu", ve, seq_k,
                d_v, v_len);
    if (out_len < oe)
        INVALID("attention_tc: out buffer too small: need %zu f32 (%u\xC3\x97%u), got %zu", oe,
                seq_q, d_v, out_len);
    return KAIO_B200_OK;
}

#define REQUIRE_PTR(p, op, name)                                                   \
    if ((p) == nullptr)                                                            \
    return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: %s pointer is null", op, name)

// ---------------------------------------------------------------- op bodies
static int32_t run_int8(int epi, const int8_t* a, size_t a_len, const int8_t* b, size_t b_len,
                        void* c, size_t c_len, float scale, const float* a_scale,
                        const float* w_scale, uint32_t m, uint32_t n, uint32_t k, void* stream)
{
    int32_t rc = validate_int8(epi == EPI_S32 ? "i32" : "f32", a_len, b_len, c_len, m, n, k);
    if (rc)
        return rc;
    REQUIRE_PTR(a, "matmul_int8", "A");
    REQUIRE_PTR(b, "matmul_int8", "B");
    REQUIRE_PTR(c, "matmul_int8", "C");
    DeviceCtx* ctx;
    if ((rc = get_ctx(&ctx, c)))
        return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool scales_aligned = epi != EPI_ROWCOL || ((uintptr_t)w_scale % 16 == 0);
    if (w8a8_fast_path_ok(a, b, c, m, n, k) && scales_aligned) {
        bool pair = w8a8_2cta_ok(m, n, k);
        if (const char* e = getenv("KAIO_B200_PAIR"))  // tuning aid: 0/1 forces single CTA / pair
            pair = (e[0] == '1');
        if (pair)
            return finish(launch_w8a8_gemm_2cta(*ctx, epi, a, b, c, scale, a_scale, w_scale, m, n,
                                                k, s),
                          "matmul_int8", "w8a8_tcgen05_2cta");
        return finish(launch_w8a8_gemm(*ctx, epi, a, b, c, scale, a_scale, w_scale, m, n, k, s),
                      "matmul_int8", "w8a8_tcgen05");
    }
    return finish(launch_int8_generic(epi, a, b, c, scale, a_scale, w_scale, m, n, k, s),
                  "matmul_int8", "int8_generic");
}

// Largest M the fused-dequant W4A16 kernel takes; above it the weights are dequantised once to
// f16 and the paired f16 GEMM runs.  KAIO_B200_FUSED_MAX_M overrides it (tuning aid).
static uint32_t fused_max_m()
{
    static const uint32_t v = [] {
        if (const char* e = getenv("KAIO_B200_FUSED_MAX_M"))
            return (uint32_t)strtoul(e, nullptr, 10);
        return 512u;
    }();
    return v;
}

static int32_t run_int4(const kaio_f16* a, size_t a_len, const uint32_t* b, size_t b_len,
                        const kaio_f16* scales, size_t s_len, void* c, size_t c_len, bool out_f16,
                        uint32_t m, uint32_t n, uint32_t k, uint32_t group_size, void* stream)
{
    int32_t rc =
        validate_int4(out_f16 ? "f16" : "f32", a_len, b_len, s_len, c_len, m, n, k, group_size);
    if (rc)
        return rc;
    REQUIRE_PTR(a, "matmul_int4", "A");
    REQUIRE_PTR(b, "matmul_int4", "B packed");
    REQUIRE_PTR(scales, "matmul_int4", "scales");
    REQUIRE_PTR(c, "matmul_int4", "C");
    DeviceCtx* ctx;
    if ((rc = get_ctx(&ctx, c)))
        return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamScratch* sc = nullptr;
    DqProblem pr;
    pr.w = b;
    pr.scales = reinterpret_cast<const __half*>(scales);
    pr.col_scale = nullptr;
    pr.scale = 1.0f;
    pr.out = c;
    const __half* x = reinterpret_cast<const __half*>(a);
    if (w4a16_decode_ok(x, &pr, 1, m, n, k)) {
        const size_t ws = w4a16_decode_workspace_bytes(*ctx, n, k);
        if ((rc = ensure_workspace(ctx, s, ws, w4a16_decode_num_counters(n), &sc)))
            return rc;
        return finish(launch_w4a16_decode(*ctx, x, pr, out_f16, m, n, k, sc->workspace,
                                          sc->tile_counters, s),
                      "matmul_int4", "w4a16_decode_splitk");
    }
    if (m <= fused_max_m() && w4a16_fused_ok(x, &pr, 1, m, n, k)) {
        const size_t ws = w4a16_fused_workspace_bytes(*ctx, 1, m, n, k);
        if (ws && (rc = ensure_workspace(ctx, s, ws, w4a16_fused_num_counters(*ctx, 1, m, n, k), &sc)))
            return rc;
        return finish(launch_w4a16_fused(*ctx, x, &pr, 1, out_f16, m, n, k,
                                         ws ? sc->workspace : nullptr,
                                         ws ? sc->tile_counters : nullptr, s),
                      "matmul_int4", ws ? "w4a16_fused_dequant_splitk" : "w4a16_fused_dequant");
    }
    if (dq_gemm_fast_path_ok(WFMT_S4_PACKED, x, &pr, 1, out_f16, m, n, k)) {
        if ((rc = ensure_dq_workspace(ctx, s, dq_gemm_workspace_bytes(1, n, k), &sc)))
            return rc;
        return finish(launch_dq_gemm(*ctx, WFMT_S4_PACKED, x, &pr, 1, out_f16, false, m, n, k,
                                     sc->dq_workspace, s),
                      "matmul_int4", "w4a16_tcgen05");
    }
    return finish(launch_dq_generic(WFMT_S4_PACKED, x, &pr, 1, out_f16, false, m, n, k, s),
                  "matmul_int4", "w4a16_generic");
}

static int32_t run_qkv(int wfmt, const char* op, const __half* x, DqProblem probs[3],
                       bool post_scale, uint32_t m, uint32_t n, uint32_t k, void* stream)
{
    for (int i = 0; i < 3; ++i)
        for (int j = i + 1; j < 3; ++j)
            if (probs[i].out == probs[j].out)
                return fail(KAIO_B200_ERR_INVALID_CONFIG,
                            "%s: the three output buffers must be distinct allocations", op);
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx, probs[0].out)))
        return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamScratch* sc = nullptr;
    if (wfmt == WFMT_S4_PACKED && !post_scale && m <= fused_max_m() &&
        w4a16_fused_ok(x, probs, 3, m, n, k)) {
        const size_t ws = w4a16_fused_workspace_bytes(*ctx, 3, m, n, k);
        if (ws && (rc = ensure_workspace(ctx, s, ws, w4a16_fused_num_counters(*ctx, 3, m, n, k), &sc)))
            return rc;
        return finish(launch_w4a16_fused(*ctx, x, probs, 3, true, m, n, k,
                                         ws ? sc->workspace : nullptr,
                                         ws ? sc->tile_counters : nullptr, s),
                      op, ws ? "qkv_w4a16_fused_dequant_splitk" : "qkv_w4a16_fused_dequant");
    }
    if (dq_gemm_fast_path_ok(wfmt, x, probs, 3, true, m, n, k)) {
        if ((rc = ensure_dq_workspace(ctx, s, dq_gemm_workspace_bytes(3, n, k), &sc)))
            return rc;
        return finish(launch_dq_gemm(*ctx, wfmt, x, probs, 3, true, post_scale, m, n, k,
                                     sc->dq_workspace, s),
                      op, wfmt == WFMT_S8_ROWMAJOR ? "qkv_w8a16_tcgen05" : "qkv_w4a16_tcgen05");
    }
    return finish(launch_dq_generic(wfmt, x, probs, 3, true, post_scale, m, n, k, s), op,
                  wfmt == WFMT_S8_ROWMAJOR ? "qkv_w8a16_generic" : "qkv_w4a16_generic");
}

}  // namespace kaio

using namespace kaio;

// ==================================================================== exported entry points

KAIO_API int32_t kaio_b200_matmul_int8(const int8_t* a, size_t a_len, const int8_t* b, size_t b_len,
                                       float* c, size_t c_len, float scale, uint32_t m, uint32_t n,
                                       uint32_t k, void* stream)
{
    return run_int8(EPI_SCALAR, a, a_len, b, b_len, c, c_len, scale, nullptr, nullptr, m, n, k,
                    stream);
}

KAIO_API int32_t kaio_b200_matmul_int8_scaled(const int8_t* a, size_t a_len, const int8_t* b,
                                              size_t b_len, float* c, size_t c_len,
                                              const float* a_scale, size_t a_scale_len,
                                              const float* w_scale, size_t w_scale_len, uint32_t m,
                                              uint32_t n, uint32_t k, void* stream)
{
    if (a_scale == nullptr || w_scale == nullptr)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "matmul_int8_scaled: scale pointer is null");
    if (a_scale_len < m)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "matmul_int8_scaled: a_scale buffer too small: need %u f32, got %zu", m,
                    a_scale_len);
    if (w_scale_len < n)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "matmul_int8_scaled: w_scale buffer too small: need %u f32, got %zu", n,
                    w_scale_len);
    return run_int8(EPI_ROWCOL, a, a_len, b, b_len, c, c_len, 1.0f, a_scale, w_scale, m, n, k,
                    stream);
}

KAIO_API int32_t kaio_b200_matmul_int8_acc(const int8_t* a, size_t a_len, const int8_t* b,
                                           size_t b_len, int32_t* acc, size_t acc_len, uint32_t m,
                                           uint32_t n, uint32_t k, void* stream)
{
    return run_int8(EPI_S32, a, a_len, b, b_len, acc, acc_len, 1.0f, nullptr, nullptr, m, n, k,
                    stream);
}

// ---------------------------------------------------------------- matmul_tc (f16 x f16 -> f32)
// Messages restate validate_dims_tc (kaio-ops/src/matmul_tc_kernel.rs:123-164).
static int32_t run_matmul_tc(const kaio_f16* a, size_t a_len, const kaio_f16* b, size_t b_len,
                             void* c, size_t c_len, bool out_f16, uint32_t m, uint32_t n, uint32_t k,
                             void* stream)
{
    if (m == 0 || n == 0 || k == 0)
        INVALID("matmul_tc dimensions must be non-zero");
    if (k % 16 != 0)
        INVALID("matmul_tc: K must be a multiple of 16 (got %u). The mma.sync.m16n8k16 "
                "instance shape requires K-tile size 16; K is not edge-padded inside a K-tile.",
                k);
    const size_t mk = (size_t)m * k, kn = (size_t)k * n, mn = (size_t)m * n;
    if (a_len < mk)
        INVALID("matmul_tc: A buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu", mk, m, k, a_len);
    if (b_len < kn)
        INVALID("matmul_tc: B buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu", kn, k, n, b_len);
    if (c_len < mn)
        INVALID("matmul_tc: C buffer too small: need %zu %s (%u\xC3\x97%u), got %zu", mn,
                out_f16 ? "f16" : "f32", m, n, c_len);
    REQUIRE_PTR(a, "matmul_tc", "A");
    REQUIRE_PTR(b, "matmul_tc", "B");
    REQUIRE_PTR(c, "matmul_tc", "C");
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx, c)))
        return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DqProblem pr;
    pr.w = b;
    pr.scales = nullptr;
    pr.col_scale = nullptr;
    pr.scale = 1.0f;
    pr.out = c;
    const __half* x = reinterpret_cast<const __half*>(a);
    if (dq_gemm_fast_path_ok(WFMT_F16, x, &pr, 1, out_f16, m, n, k))
        return finish(launch_dq_gemm(*ctx, WFMT_F16, x, &pr, 1, out_f16, false, m, n, k, nullptr, s),
                      "matmul_tc", "f16_tcgen05");
    return finish(launch_dq_generic(WFMT_F16, x, &pr, 1, out_f16, false, m, n, k, s), "matmul_tc",
                  "f16_generic");
}

KAIO_API int32_t kaio_b200_matmul_tc(const kaio_f16* a, size_t a_len, const kaio_f16* b, size_t b_len,
                                     float* c, size_t c_len, uint32_t m, uint32_t n, uint32_t k,
                                     void* stream)
{
    return run_matmul_tc(a, a_len, b, b_len, c, c_len, false, m, n, k, stream);
}

KAIO_API int32_t kaio_b200_matmul_tc_f16out(const kaio_f16* a, size_t a_len, const kaio_f16* b,
                                            size_t b_len, kaio_f16* c, size_t c_len, uint32_t m,
                                            uint32_t n, uint32_t k, void* stream)
{
    return run_matmul_tc(a, a_len, b, b_len, c, c_len, true, m, n, k, stream);
}

KAIO_API int32_t kaio_b200_dequantize_int4(const uint32_t* b_packed, size_t b_len,
                                           const kaio_f16* scales, size_t scales_len, kaio_f16* w,
                                           size_t w_len, uint32_t k, uint32_t n,
                                           uint32_t group_size, void* stream)
{
    const char* op = "dequantize_int4";
    if (k == 0 || n == 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s dimensions must be non-zero", op);
    if (group_size != 128)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: group_size must be 128 (got %u)", op, group_size);
    if (k % 128 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: K must be a multiple of group_size=128 (got %u)", op, k);
    if (n % 2 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: N must be even (got %u)", op, n);
    const size_t words = (size_t)(k / 8) * n, cells = (size_t)(k / 128) * n, kn = (size_t)k * n;
    if (b_len < words)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: packed buffer too small: need %zu u32, got %zu",
                    op, words, b_len);
    if (scales_len < cells)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: scales buffer too small: need %zu f16, got %zu",
                    op, cells, scales_len);
    if (w_len < kn)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: W buffer too small: need %zu f16 (%u\xC3\x97%u), got %zu", op, kn, k, n, w_len);
    REQUIRE_PTR(b_packed, op, "packed");
    REQUIRE_PTR(scales, op, "scales");
    REQUIRE_PTR(w, op, "W");
    if ((uintptr_t)w % 4 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: W must be 4-byte aligned", op);
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx, w)))
        return rc;
    return finish(launch_dequant_s4(b_packed, reinterpret_cast<const __half*>(scales),
                                    reinterpret_cast<__half*>(w), n, k,
                                    static_cast<cudaStream_t>(stream)),
                  op, "dequant_s4");
}

KAIO_API int32_t kaio_b200_matmul_tc_async(const kaio_f16* a, size_t a_len, const kaio_f16* b,
                                           size_t b_len, float* c, size_t c_len, uint32_t m,
                                           uint32_t n, uint32_t k, void* stream)
{
    return run_matmul_tc(a, a_len, b, b_len, c, c_len, false, m, n, k, stream);
}

KAIO_API int32_t kaio_b200_matmul_int4(const kaio_f16* a, size_t a_len, const uint32_t* b_packed,
                                       size_t b_len, const kaio_f16* scales, size_t scales_len,
                                       float* c, size_t c_len, uint32_t m, uint32_t n, uint32_t k,
                                       uint32_t group_size, void* stream)
{
    return run_int4(a, a_len, b_packed, b_len, scales, scales_len, c, c_len, false, m, n, k,
                    group_size, stream);
}

KAIO_API int32_t kaio_b200_matmul_int4_f16out(const kaio_f16* a, size_t a_len,
                                              const uint32_t* b_packed, size_t b_len,
                                              const kaio_f16* scales, size_t scales_len,
                                              kaio_f16* c, size_t c_len, uint32_t m, uint32_t n,
                                              uint32_t k, uint32_t group_size, void* stream)
{
    return run_int4(a, a_len, b_packed, b_len, scales, scales_len, c, c_len, true, m, n, k,
                    group_size, stream);
}

static int32_t qkv_int8_common(const kaio_f16* x, size_t x_len, const int8_t* const w[3],
                               const size_t w_len[3], const float scalar[3],
                               const float* const col[3], kaio_f16* const out[3],
                               const size_t o_len[3], uint32_t m, uint32_t n, uint32_t k,
                               void* stream)
{
    int32_t rc = validate_qkv_int8(x_len, w_len, o_len, m, n, k);
    if (rc)
        return rc;
    REQUIRE_PTR(x, "qkv_project_int8", "X");
    DqProblem probs[3];
    for (int i = 0; i < 3; ++i) {
        REQUIRE_PTR(w[i], "qkv_project_int8", "W");
        REQUIRE_PTR(out[i], "qkv_project_int8", "output");
        probs[i].w = w[i];
        probs[i].scales = nullptr;
        probs[i].col_scale = col ? col[i] : nullptr;
        probs[i].scale = scalar ? scalar[i] : 1.0f;
        probs[i].out = out[i];
    }
    return run_qkv(WFMT_S8_ROWMAJOR, "qkv_project_int8", reinterpret_cast<const __half*>(x), probs,
                   true, m, n, k, stream);
}

KAIO_API int32_t kaio_b200_qkv_project_int8(const kaio_f16* x, size_t x_len, const int8_t* w_q,
                                            size_t w_q_len, const int8_t* w_k, size_t w_k_len,
                                            const int8_t* w_v, size_t w_v_len, float scale_q,
                                            float scale_k, float scale_v, kaio_f16* q_out,
                                            size_t q_len, kaio_f16* k_out, size_t k_len,
                                            kaio_f16* v_out, size_t v_len, uint32_t m, uint32_t n,
                                            uint32_t k, void* stream)
{
    const int8_t* w[3] = {w_q, w_k, w_v};
    const size_t wl[3] = {w_q_len, w_k_len, w_v_len};
    const float sc[3] = {scale_q, scale_k, scale_v};
    kaio_f16* out[3] = {q_out, k_out, v_out};
    const size_t ol[3] = {q_len, k_len, v_len};
    return qkv_int8_common(x, x_len, w, wl, sc, nullptr, out, ol, m, n, k, stream);
}

KAIO_API int32_t kaio_b200_qkv_project_int8_colscale(
    const kaio_f16* x, size_t x_len, const int8_t* w_q, size_t w_q_len, const int8_t* w_k,
    size_t w_k_len, const int8_t* w_v, size_t w_v_len, const float* scale_q, const float* scale_k,
    const float* scale_v, size_t scale_len, kaio_f16* q_out, size_t q_len, kaio_f16* k_out,
    size_t k_len, kaio_f16* v_out, size_t v_len, uint32_t m, uint32_t n, uint32_t k, void* stream)
{
    if (scale_q == nullptr || scale_k == nullptr || scale_v == nullptr)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "qkv_project_int8_colscale: scale pointer is null");
    if (scale_len < n)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "qkv_project_int8_colscale: scale buffers too small: need %u f32, got %zu", n,
                    scale_len);
    const int8_t* w[3] = {w_q, w_k, w_v};
    const size_t wl[3] = {w_q_len, w_k_len, w_v_len};
    const float* col[3] = {scale_q, scale_k, scale_v};
    kaio_f16* out[3] = {q_out, k_out, v_out};
    const size_t ol[3] = {q_len, k_len, v_len};
    return qkv_int8_common(x, x_len, w, wl, nullptr, col, out, ol, m, n, k, stream);
}

// W8A8 form of the fused QKV projection: x is quantised per row to s8 on the fly, the three
// products run on the INT8 tensor pipe, the per-row and per-column scales are applied to the
// exact s32 accumulators.  Validation follows validate_dims_qkv_int8 (the reference's W8A16
// op), with K a multiple of 32 as kind::i8 needs.
KAIO_API int32_t kaio_b200_qkv_project_w8a8(
    const kaio_f16* x, size_t x_len, const int8_t* w_q, size_t w_q_len, const int8_t* w_k,
    size_t w_k_len, const int8_t* w_v, size_t w_v_len, const float* scale_q, const float* scale_k,
    const float* scale_v, size_t scale_len, kaio_f16* q_out, size_t q_len, kaio_f16* k_out,
    size_t k_len, kaio_f16* v_out, size_t v_len, uint32_t m, uint32_t n, uint32_t k, void* stream)
{
    const char* op = "qkv_project_w8a8";
    const size_t wl[3] = {w_q_len, w_k_len, w_v_len};
    const size_t ol[3] = {q_len, k_len, v_len};
    int32_t rc = validate_qkv_int8(x_len, wl, ol, m, n, k);
    if (rc)
        return rc;
    if (k % 32 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: K must be a multiple of 32 (got %u): the INT8 tensor-core instruction "
                    "consumes 32 k per step and K is not edge-padded", op, k);
    if (scale_q == nullptr || scale_k == nullptr || scale_v == nullptr)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: scale pointer is null", op);
    if (scale_len < n)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: scale buffers too small: need %u f32, got %zu", op, n, scale_len);
    REQUIRE_PTR(x, op, "X");
    const int8_t* w[3] = {w_q, w_k, w_v};
    const float* col[3] = {scale_q, scale_k, scale_v};
    void* out[3] = {q_out, k_out, v_out};
    for (int i = 0; i < 3; ++i) {
        REQUIRE_PTR(w[i], op, "W");
        REQUIRE_PTR(out[i], op, "output");
    }
    for (int i = 0; i < 3; ++i)
        for (int j = i + 1; j < 3; ++j)
            if (out[i] == out[j])
                return fail(KAIO_B200_ERR_INVALID_CONFIG,
                            "%s: the three output buffers must be distinct allocations", op);
    if ((uintptr_t)x % 16 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: X must be 16-byte aligned", op);
    DeviceCtx* ctx;
    if ((rc = get_ctx(&ctx, q_out)))
        return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // scratch: the quantised activations (m*k s8, rounded up to 256 bytes) and their row scales
    const size_t xq_bytes = (((size_t)m * k + 255) / 256) * 256;
    StreamScratch* sc = nullptr;
    if ((rc = ensure_dq_workspace(ctx, s, xq_bytes + (size_t)m * sizeof(float), &sc)))
        return rc;
    int8_t* xq = reinterpret_cast<int8_t*>(sc->dq_workspace);
    float* x_scale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sc->dq_workspace) + xq_bytes);
    cudaError_t err = launch_quantize_rows_int8_f16(reinterpret_cast<const __half*>(x), xq, x_scale,
                                                    m, k, s);
    if (err != cudaSuccess)
        return fail_cuda(err, op);
    bool fast = m > 128 && (n % 16 == 0);
    for (int i = 0; i < 3; ++i)
        fast = fast && ((uintptr_t)w[i] % 16 == 0) && ((uintptr_t)out[i] % 16 == 0) &&
               ((uintptr_t)col[i] % 16 == 0);
    if (fast)
        return finish(launch_w8a8_qkv_2cta(*ctx, xq, x_scale, w, col, out, m, n, k, s), op,
                      "qkv_w8a8_tcgen05_2cta");
    for (int i = 0; i < 3; ++i) {
        err = launch_int8_generic(EPI_ROWCOL_F16, xq, w[i], out[i], 1.0f, x_scale, col[i], m, n, k, s);
        if (err != cudaSuccess)
            return fail_cuda(err, op);
    }
    return finish(cudaSuccess, op, "qkv_w8a8_generic");
}

KAIO_API int32_t kaio_b200_qkv_project_int4(
    const kaio_f16* x, size_t x_len, const uint32_t* w_q_packed, size_t w_q_len,
    const uint32_t* w_k_packed, size_t w_k_len, const uint32_t* w_v_packed, size_t w_v_len,
    const kaio_f16* scales_q, size_t scales_q_len, const kaio_f16* scales_k, size_t scales_k_len,
    const kaio_f16* scales_v, size_t scales_v_len, kaio_f16* q_out, size_t q_len, kaio_f16* k_out,
    size_t k_len, kaio_f16* v_out, size_t v_len, uint32_t m, uint32_t n, uint32_t k,
    uint32_t group_size, void* stream)
{
    const size_t wl[3] = {w_q_len, w_k_len, w_v_len};
    const size_t sl[3] = {scales_q_len, scales_k_len, scales_v_len};
    const size_t ol[3] = {q_len, k_len, v_len};
    int32_t rc = validate_qkv_int4(x_len, wl, sl, ol, m, n, k, group_size);
    if (rc)
        return rc;
    const uint32_t* w[3] = {w_q_packed, w_k_packed, w_v_packed};
    const kaio_f16* sc[3] = {scales_q, scales_k, scales_v};
    kaio_f16* out[3] = {q_out, k_out, v_out};
    REQUIRE_PTR(x, "qkv_project_int4", "X");
    DqProblem probs[3];
    for (int i = 0; i < 3; ++i) {
        REQUIRE_PTR(w[i], "qkv_project_int4", "W packed");
        REQUIRE_PTR(sc[i], "qkv_project_int4", "scales");
        REQUIRE_PTR(out[i], "qkv_project_int4", "output");
        probs[i].w = w[i];
        probs[i].scales = reinterpret_cast<const __half*>(sc[i]);
        probs[i].col_scale = nullptr;
        probs[i].scale = 1.0f;
        probs[i].out = out[i];
    }
    return run_qkv(WFMT_S4_PACKED, "qkv_project_int4", reinterpret_cast<const __half*>(x), probs,
                   false, m, n, k, stream);
}

KAIO_API int32_t kaio_b200_attention_tc(const kaio_f16* q, size_t q_len, const kaio_f16* k,
                                        size_t k_len, const kaio_f16* v, size_t v_len, float* out,
                                        size_t out_len, uint32_t seq_q, uint32_t seq_k,
                                        uint32_t d_k, uint32_t d_v, int32_t causal, void* stream)
{
    int32_t rc = validate_attention_tc(q_len, k_len, v_len, out_len, seq_q, seq_k, d_k, d_v);
    if (rc)
        return rc;
    REQUIRE_PTR(q, "attention_tc", "Q");
    REQUIRE_PTR(k, "attention_tc", "K");
    REQUIRE_PTR(v, "attention_tc", "V");
    REQUIRE_PTR(out, "attention_tc", "out");
    DeviceCtx* ctx;
    if ((rc = get_ctx(&ctx, out)))
        return rc;
    AttnParams p = {};
    p.q = reinterpret_cast<const __half*>(q);
    p.k = reinterpret_cast<const __half*>(k);
    p.v = reinterpret_cast<const __half*>(v);
    p.out = out;
    p.batch = 1;
    p.heads = 1;
    p.seq_q = seq_q;
    p.seq_k = seq_k;
    p.d_k = d_k;
    p.d_v = d_v;
    p.q_row = d_k;
    p.k_row = d_k;
    p.v_row = d_v;
    p.o_row = d_v;
    p.causal = causal ? 1 : 0;
    p.out_f16 = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (flash_attention_ok(p))
        return finish(launch_flash_attention(*ctx, p, s), "attention_tc", "flash_tcgen05");
    return finish(launch_attention_generic(p, s), "attention_tc", "attention_generic");
}

KAIO_API int32_t kaio_b200_attention_mha_f16(const kaio_f16* q, size_t q_len, const kaio_f16* k,
                                             size_t k_len, const kaio_f16* v, size_t v_len,
                                             kaio_f16* out, size_t out_len, uint32_t batch,
                                             uint32_t heads, uint32_t seq_q, uint32_t seq_k,
                                             uint32_t head_dim, uint32_t row_stride,
                                             int32_t causal, void* stream)
{
    const char* op = "attention_mha_f16";
    if (batch == 0 || heads == 0 || seq_q == 0 || seq_k == 0 || head_dim == 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s dimensions must be non-zero", op);
    if ((uint64_t)heads * head_dim > row_stride)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: row_stride (%u) must be at least heads*head_dim (%llu)", op, row_stride,
                    (unsigned long long)heads * head_dim);
    if (head_dim > 256)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: head_dim must be \xE2\x89\xA4 256 (got %u)",
                    op, head_dim);
    const size_t need_q = ((size_t)batch * seq_q - 1) * row_stride + (size_t)heads * head_dim;
    const size_t need_k = ((size_t)batch * seq_k - 1) * row_stride + (size_t)heads * head_dim;
    if (q_len < need_q)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: Q buffer too small: need %zu f16, got %zu", op, need_q, q_len);
    if (k_len < need_k)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: K buffer too small: need %zu f16, got %zu", op, need_k, k_len);
    if (v_len < need_k)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: V buffer too small: need %zu f16, got %zu", op, need_k, v_len);
    if (out_len < need_q)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: out buffer too small: need %zu f16, got %zu", op, need_q, out_len);
    REQUIRE_PTR(q, op, "Q");
    REQUIRE_PTR(k, op, "K");
    REQUIRE_PTR(v, op, "V");
    REQUIRE_PTR(out, op, "out");
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx, out)))
        return rc;
    AttnParams p = {};
    p.q = reinterpret_cast<const __half*>(q);
    p.k = reinterpret_cast<const __half*>(k);
    p.v = reinterpret_cast<const __half*>(v);
    p.out = out;
    p.batch = batch;
    p.heads = heads;
    p.seq_q = seq_q;
    p.seq_k = seq_k;
    p.d_k = head_dim;
    p.d_v = head_dim;
    p.q_row = p.k_row = p.v_row = p.o_row = row_stride;
    p.q_head = p.k_head = p.v_head = p.o_head = head_dim;
    p.q_batch = p.o_batch = (uint64_t)seq_q * row_stride;
    p.k_batch = p.v_batch = (uint64_t)seq_k * row_stride;
    p.causal = causal ? 1 : 0;
    p.out_f16 = 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (flash_attention_ok(p))
        return finish(launch_flash_attention(*ctx, p, s), op, "flash_tcgen05");
    return finish(launch_attention_generic(p, s), op, "attention_generic");
}

// ---------------------------------------------------------------- quantisers
KAIO_API int32_t kaio_b200_quantize_rows_int8(const float* x, size_t x_len, int8_t* q, size_t q_len,
                                              float* scale, size_t scale_len, uint32_t m,
                                              uint32_t k, void* stream)
{
    const char* op = "quantize_rows_int8";
    if (m == 0 || k == 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s dimensions must be non-zero", op);
    const size_t mk = (size_t)m * k;
    if (x_len < mk)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: X buffer too small: need %zu f32 (%u\xC3\x97%u), got %zu", op, mk, m, k,
                    x_len);
    if (q_len < mk)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: Q buffer too small: need %zu i8 (%u\xC3\x97%u), got %zu", op, mk, m, k,
                    q_len);
    if (scale_len < m)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: scale buffer too small: need %u f32, got %zu", op, m, scale_len);
    REQUIRE_PTR(x, op, "X");
    REQUIRE_PTR(q, op, "Q");
    REQUIRE_PTR(scale, op, "scale");
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx)))
        return rc;
    return finish(launch_quantize_rows_int8(x, q, scale, m, k, static_cast<cudaStream_t>(stream)),
                  op, "quantize_rows_int8");
}

// ---------------------------------------------------------------- gated activation
KAIO_API int32_t kaio_b200_silu_gate_f32(const float* x, size_t x_len, const float* gate,
                                         size_t gate_len, float* out, size_t out_len, uint32_t n,
                                         void* stream)
{
    const char* op = "silu_gate_f32";
    if (n == 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s dimensions must be non-zero", op);
    if (x_len < n)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: X buffer too small: need %u f32, got %zu",
                    op, n, x_len);
    if (gate_len < n)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: gate buffer too small: need %u f32, got %zu", op, n, gate_len);
    if (out_len < n)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: out buffer too small: need %u f32, got %zu", op, n, out_len);
    REQUIRE_PTR(x, op, "X");
    REQUIRE_PTR(gate, op, "gate");
    REQUIRE_PTR(out, op, "out");
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx)))
        return rc;
    return finish(launch_silu_gate_f32(x, gate, out, n, static_cast<cudaStream_t>(stream)), op,
                  "silu_gate_f32");
}

KAIO_API int32_t kaio_b200_silu_gate_f16(const kaio_f16* x, size_t x_len, const kaio_f16* gate,
                                         size_t gate_len, kaio_f16* out, size_t out_len,
                                         uint32_t rows, uint32_t cols, uint32_t x_ld,
                                         uint32_t gate_ld, uint32_t out_ld, void* stream)
{
    const char* op = "silu_gate_f16";
    if (rows == 0 || cols == 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s dimensions must be non-zero", op);
    if (x_ld < cols || gate_ld < cols || out_ld < cols)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: row strides must be at least cols (got x_ld=%u, gate_ld=%u, out_ld=%u, "
                    "cols=%u)", op, x_ld, gate_ld, out_ld, cols);
    const size_t need_x = (size_t)(rows - 1) * x_ld + cols;
    const size_t need_g = (size_t)(rows - 1) * gate_ld + cols;
    const size_t need_o = (size_t)(rows - 1) * out_ld + cols;
    if (x_len < need_x)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: X buffer too small: need %zu f16, got %zu",
                    op, need_x, x_len);
    if (gate_len < need_g)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: gate buffer too small: need %zu f16, got %zu", op, need_g, gate_len);
    if (out_len < need_o)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: out buffer too small: need %zu f16, got %zu", op, need_o, out_len);
    REQUIRE_PTR(x, op, "X");
    REQUIRE_PTR(gate, op, "gate");
    REQUIRE_PTR(out, op, "out");
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx)))
        return rc;
    return finish(launch_silu_gate_f16(reinterpret_cast<const __half*>(x),
                                       reinterpret_cast<const __half*>(gate),
                                       reinterpret_cast<__half*>(out), rows, cols, x_ld, gate_ld,
                                       out_ld, static_cast<cudaStream_t>(stream)),
                  op, "silu_gate_f16");
}

KAIO_API int32_t kaio_b200_matmul_int4_silu_gate(const kaio_f16* x, size_t x_len,
                                                 const uint32_t* b_packed, size_t b_len,
                                                 const kaio_f16* scales, size_t scales_len,
                                                 kaio_f16* act, size_t act_len, kaio_f16* gu_scratch,
                                                 size_t gu_len, uint32_t m, uint32_t cols,
                                                 uint32_t k, uint32_t group_size, void* stream)
{
    const char* op = "matmul_int4_silu_gate";
    if (cols == 0 || cols % 64 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: cols must be a non-zero multiple of 64, the interleave block (got %u)", op,
                    cols);
    const uint32_t n = 2 * cols;
    // the interleaved projection is an ordinary W4A16 product [m, 2*cols]
    int32_t rc = validate_int4("f16", x_len, b_len, scales_len, (size_t)m * n, m, n, k, group_size);
    if (rc)
        return rc;
    if (act_len < (size_t)m * cols)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: act buffer too small: need %zu f16, got %zu", op,
                    (size_t)m * cols, act_len);
    REQUIRE_PTR(x, op, "X");
    REQUIRE_PTR(b_packed, op, "B packed");
    REQUIRE_PTR(scales, op, "scales");
    REQUIRE_PTR(act, op, "act");
    DeviceCtx* ctx;
    if ((rc = get_ctx(&ctx, act)))
        return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DqProblem pr;
    pr.w = b_packed;
    pr.scales = reinterpret_cast<const __half*>(scales);
    pr.col_scale = nullptr;
    pr.scale = 1.0f;
    pr.out = act;
    const __half* xh = reinterpret_cast<const __half*>(x);
    // Large M: the paired f16 GEMM applies the activation in its epilogue (the interleaved
    // [m, 2*cols] projection never reaches memory).  The small-M kernels keep their own epilogues:
    // they write the interleaved projection to the caller's scratch and a second launch applies
    // the activation -- the same bits either way.
    const bool small_m = w4a16_decode_ok(xh, &pr, 1, m, n, k) ||
                         (m <= fused_max_m() && w4a16_fused_ok(xh, &pr, 1, m, n, k));
    if (!small_m && m > 128 && (uintptr_t)act % 16 == 0 &&
        dq_gemm_fast_path_ok(WFMT_S4_PACKED, xh, &pr, 1, true, m, n, k)) {
        StreamScratch* sc = nullptr;
        if ((rc = ensure_dq_workspace(ctx, s, dq_gemm_workspace_bytes(1, n, k), &sc)))
            return rc;
        return finish(launch_dq_gemm(*ctx, WFMT_S4_PACKED, xh, &pr, 1, true, false, m, n, k,
                                     sc->dq_workspace, s, nullptr, true),
                      op, "w4a16_tcgen05_silu_gate");
    }
    if (gu_scratch == nullptr || gu_len < (size_t)m * n || (uintptr_t)gu_scratch % 16 != 0 ||
        (uintptr_t)act % 16 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: this shape needs a 16-byte aligned scratch of %zu f16 for the interleaved "
                    "projection (got %zu) and a 16-byte aligned act", op, (size_t)m * n, gu_len);
    if ((rc = run_int4(x, x_len, b_packed, b_len, scales, scales_len, gu_scratch, gu_len, true, m, n, k,
                       group_size, stream)))
        return rc;
    return finish(launch_silu_gate_f16_interleaved(reinterpret_cast<const __half*>(gu_scratch),
                                                   reinterpret_cast<__half*>(act), m, cols, n, cols, s),
                  op, "w4a16_then_silu_gate");
}

KAIO_API int32_t kaio_b200_quantize_pack_int4(const float* w, size_t w_len, uint32_t* packed,
                                              size_t packed_len, kaio_f16* scales,
                                              size_t scales_len, uint32_t k, uint32_t n,
                                              uint32_t group_size, void* stream)
{
    const char* op = "quantize_pack_int4";
    if (k == 0 || n == 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s dimensions must be non-zero", op);
    if (group_size != 128)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: group_size must be 128 (got %u)", op,
                    group_size);
    if (k % 128 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: K must be a multiple of group_size=128 (got %u)", op, k);
    const size_t kn = (size_t)k * n, words = (size_t)(k / 8) * n, cells = (size_t)(k / 128) * n;
    if (w_len < kn)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: W buffer too small: need %zu f32 (%u\xC3\x97%u), got %zu", op, kn, k, n,
                    w_len);
    if (packed_len < words)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: packed buffer too small: need %zu u32, got %zu", op, words, packed_len);
    if (scales_len < cells)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: scales buffer too small: need %zu f16, got %zu", op, cells, scales_len);
    REQUIRE_PTR(w, op, "W");
    REQUIRE_PTR(packed, op, "packed");
    REQUIRE_PTR(scales, op, "scales");
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx)))
        return rc;
    return finish(launch_quantize_pack_s4(w, packed, reinterpret_cast<__half*>(scales), k, n,
                                          static_cast<cudaStream_t>(stream)),
                  op, "quantize_pack_s4");
}

// ---------------------------------------------------------------- sharded W4A16 + all-gather
static int32_t run_int4_allgather(const char* op, const kaio_f16* a, size_t a_len,
                                  const uint32_t* b_packed_shard, size_t b_len,
                                  const kaio_f16* scales_shard, size_t scales_len,
                                  void* const* out_ptrs, size_t out_len, void* multicast_out,
                                  uint32_t world, uint32_t rank, uint32_t m, uint32_t n_total,
                                  uint32_t k, uint32_t group_size, void* stream)
{
    if (world == 0 || world > 8 || rank >= world)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: world must be 1..8 and rank < world (got %u, %u)",
                    op, world, rank);
    if (n_total == 0 || n_total % world != 0 || (n_total / world) % 8 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: N (%u) must split into %u shards of a multiple of 8 columns", op, n_total,
                    world);
    const uint32_t n_loc = n_total / world;
    const size_t need_out = (size_t)m * n_total;
    int32_t rc = validate_int4("f16", a_len, b_len, scales_len, need_out, m, n_loc, k, group_size);
    if (rc)
        return rc;
    if (out_len < need_out)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: output buffers too small: need %zu f16 (%u\xC3\x97%u), got %zu", op, need_out,
                    m, n_total, out_len);
    REQUIRE_PTR(a, op, "A");
    REQUIRE_PTR(b_packed_shard, op, "B packed");
    REQUIRE_PTR(scales_shard, op, "scales");
    REQUIRE_PTR(out_ptrs, op, "out_ptrs");
    OutputCopies copies = {};
    copies.count = world;
    copies.ld = n_total;
    for (uint32_t r = 0; r < world; ++r) {
        if (out_ptrs[r] == nullptr || (uintptr_t)out_ptrs[r] % 16 != 0)
            return fail(KAIO_B200_ERR_INVALID_CONFIG,
                        "%s: output pointer %u is null or not 16-byte aligned", op, r);
        copies.ptrs[r] = reinterpret_cast<kaio_f16*>(out_ptrs[r]) + (size_t)rank * n_loc;
    }
    if (multicast_out != nullptr) {
        if ((uintptr_t)multicast_out % 16 != 0)
            return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: multicast address is not 16-byte aligned", op);
        copies.multicast = reinterpret_cast<kaio_f16*>(multicast_out) + (size_t)rank * n_loc;
    }
    DeviceCtx* ctx;
    if ((rc = get_ctx(&ctx)))
        return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamScratch* sc = nullptr;
    DqProblem pr;
    pr.w = b_packed_shard;
    pr.scales = reinterpret_cast<const __half*>(scales_shard);
    pr.col_scale = nullptr;
    pr.scale = 1.0f;
    pr.out = copies.ptrs[rank];
    const __half* x = reinterpret_cast<const __half*>(a);
    if (w4a16_decode_ok(x, &pr, 1, m, n_loc, k)) {
        if ((rc = ensure_workspace(ctx, s, w4a16_decode_workspace_bytes(*ctx, n_loc, k),
                                   w4a16_decode_num_counters(n_loc), &sc)))
            return rc;
        return finish(launch_w4a16_decode(*ctx, x, pr, true, m, n_loc, k, sc->workspace,
                                          sc->tile_counters, s, &copies),
                      op, "w4a16_decode_splitk_allgather");
    }
    if (m <= fused_max_m() && w4a16_fused_ok(x, &pr, 1, m, n_loc, k)) {
        const size_t ws = w4a16_fused_workspace_bytes(*ctx, 1, m, n_loc, k);
        if (ws && (rc = ensure_workspace(ctx, s, ws, w4a16_fused_num_counters(*ctx, 1, m, n_loc, k), &sc)))
            return rc;
        return finish(launch_w4a16_fused(*ctx, x, &pr, 1, true, m, n_loc, k,
                                         ws ? sc->workspace : nullptr,
                                         ws ? sc->tile_counters : nullptr, s, &copies),
                      op, "w4a16_fused_dequant_allgather");
    }
    if (!dq_gemm_fast_path_ok(WFMT_S4_PACKED, x, &pr, 1, true, m, n_loc, k))
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: A, B packed and the outputs must be 16-byte aligned", op);
    if ((rc = ensure_dq_workspace(ctx, s, dq_gemm_workspace_bytes(1, n_loc, k), &sc)))
        return rc;
    return finish(launch_dq_gemm(*ctx, WFMT_S4_PACKED, x, &pr, 1, true, false, m, n_loc, k,
                                 sc->dq_workspace, s, &copies),
                  op, multicast_out ? "w4a16_tcgen05_allgather_multicast" : "w4a16_tcgen05_allgather");
}

KAIO_API int32_t kaio_b200_matmul_int4_allgather(const kaio_f16* a, size_t a_len,
                                                 const uint32_t* b_packed_shard, size_t b_len,
                                                 const kaio_f16* scales_shard, size_t scales_len,
                                                 void* const* out_ptrs, size_t out_len,
                                                 uint32_t world, uint32_t rank, uint32_t m,
                                                 uint32_t n_total, uint32_t k, uint32_t group_size,
                                                 void* stream)
{
    return run_int4_allgather("matmul_int4_allgather", a, a_len, b_packed_shard, b_len, scales_shard,
                              scales_len, out_ptrs, out_len, nullptr, world, rank, m, n_total, k,
                              group_size, stream);
}

KAIO_API int32_t kaio_b200_matmul_int4_allgather_multicast(
    const kaio_f16* a, size_t a_len, const uint32_t* b_packed_shard, size_t b_len,
    const kaio_f16* scales_shard, size_t scales_len, void* const* out_ptrs, size_t out_len,
    void* multicast_out, uint32_t world, uint32_t rank, uint32_t m, uint32_t n_total, uint32_t k,
    uint32_t group_size, void* stream)
{
    const char* op = "matmul_int4_allgather_multicast";
    REQUIRE_PTR(multicast_out, op, "multicast_out");
    return run_int4_allgather(op, a, a_len, b_packed_shard, b_len, scales_shard, scales_len, out_ptrs,
                              out_len, multicast_out, world, rank, m, n_total, k, group_size, stream);
}

// ---------------------------------------------------------------- NCCL all-gather of column shards
KAIO_API int32_t kaio_b200_allgather_cols(const void* shard, size_t shard_len, void* out,
                                          size_t out_len, uint32_t m, uint32_t n_total,
                                          uint32_t elem_bytes, uint32_t world, void* nccl_comm,
                                          void* stream)
{
    const char* op = "allgather_cols";
    if (m == 0 || n_total == 0 || world == 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s dimensions must be non-zero", op);
    if (elem_bytes != 2 && elem_bytes != 4)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: elem_bytes must be 2 (f16) or 4 (f32), got %u",
                    op, elem_bytes);
    if (n_total % world != 0 || ((n_total / world) * elem_bytes) % 16 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: N (%u) must split into %u shards whose rows are a multiple of 16 bytes", op,
                    n_total, world);
    const uint32_t n_loc = n_total / world;
    if (shard_len < (size_t)m * n_loc)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: shard buffer too small: need %zu elements (%u\xC3\x97%u), got %zu", op,
                    (size_t)m * n_loc, m, n_loc, shard_len);
    if (out_len < (size_t)m * n_total)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: out buffer too small: need %zu elements (%u\xC3\x97%u), got %zu", op,
                    (size_t)m * n_total, m, n_total, out_len);
    REQUIRE_PTR(shard, op, "shard");
    REQUIRE_PTR(out, op, "out");
    REQUIRE_PTR(nccl_comm, op, "nccl_comm");
    if ((uintptr_t)shard % 16 != 0 || (uintptr_t)out % 16 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: shard and out must be 16-byte aligned", op);
    if (!nccl_available())
        return fail(KAIO_B200_ERR_CUDA, "%s: libnccl.so.2 could not be loaded", op);
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx, out)))
        return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (world == 1) {
        cudaError_t err = cudaMemcpyAsync(out, shard, (size_t)m * n_total * elem_bytes,
                                          cudaMemcpyDeviceToDevice, s);
        return finish(err, op, "allgather_cols_copy");
    }
    StreamScratch* sc = nullptr;
    if ((rc = ensure_dq_workspace(ctx, s, (size_t)m * n_total * elem_bytes, &sc)))
        return rc;
    const char* msg = "";
    cudaError_t cuda_err = cudaSuccess;
    const int nrc = launch_allgather_cols(shard, sc->dq_workspace, out, m, n_loc, elem_bytes, world,
                                          nccl_comm, s, &msg, &cuda_err);
    if (nrc != 0)
        return fail(KAIO_B200_ERR_CUDA, "%s: NCCL error %d (%s)", op, nrc, msg);
    return finish(cuda_err, op, "allgather_cols_nccl");
}

// ---------------------------------------------------------------- row-parallel W4A16 + reduction
KAIO_API int32_t kaio_b200_matmul_int4_peer_partials(const kaio_f16* a, size_t a_len,
                                                     const uint32_t* b_packed, size_t b_len,
                                                     const kaio_f16* scales, size_t scales_len,
                                                     void* const* slot_ptrs, size_t slot_len,
                                                     uint32_t world, uint32_t rank, int32_t scatter,
                                                     uint32_t m, uint32_t n, uint32_t k,
                                                     uint32_t group_size, void* stream)
{
    const char* op = "matmul_int4_peer_partials";
    if (world == 0 || world > 8 || rank >= world)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: world must be 1..8 and rank < world (got %u, %u)",
                    op, world, rank);
    if (scatter && (n == 0 || n % world != 0 || (n / world) % 64 != 0))
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: N (%u) must split into %u blocks of a multiple of 64 columns", op, n, world);
    const uint32_t cols = scatter ? n / world : n;
    const size_t need_slots = (size_t)world * m * cols;
    int32_t rc = validate_int4("f32", a_len, b_len, scales_len, (size_t)m * n, m, n, k, group_size);
    if (rc)
        return rc;
    if (slot_len < need_slots)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: staging buffers too small: need %zu f32 (%u\xC3\x97%u\xC3\x97%u), got %zu", op,
                    need_slots, world, m, cols, slot_len);
    REQUIRE_PTR(a, op, "A");
    REQUIRE_PTR(b_packed, op, "B packed");
    REQUIRE_PTR(scales, op, "scales");
    REQUIRE_PTR(slot_ptrs, op, "slot_ptrs");
    OutputCopies copies = {};
    copies.count = world;
    copies.ld = cols;
    copies.scatter_cols = scatter ? cols : 0u;
    // start the walk at the next rank's block: the ranks then store to different owners at any
    // one time, and this rank's own block (local stores) comes last
    copies.start_col = scatter ? ((rank + 1) % world) * cols : 0u;
    for (uint32_t r = 0; r < world; ++r) {
        if (slot_ptrs[r] == nullptr || (uintptr_t)slot_ptrs[r] % 16 != 0)
            return fail(KAIO_B200_ERR_INVALID_CONFIG,
                        "%s: staging pointer %u is null or not 16-byte aligned", op, r);
        copies.ptrs[r] = reinterpret_cast<float*>(slot_ptrs[r]) + (size_t)rank * m * cols;
    }
    DeviceCtx* ctx;
    if ((rc = get_ctx(&ctx)))
        return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StreamScratch* sc = nullptr;
    DqProblem pr;
    pr.w = b_packed;
    pr.scales = reinterpret_cast<const __half*>(scales);
    pr.col_scale = nullptr;
    pr.scale = 1.0f;
    pr.out = copies.ptrs[rank];
    const __half* x = reinterpret_cast<const __half*>(a);
    if (w4a16_decode_ok(x, &pr, 1, m, n, k)) {
        if ((rc = ensure_workspace(ctx, s, w4a16_decode_workspace_bytes(*ctx, n, k),
                                   w4a16_decode_num_counters(n), &sc)))
            return rc;
        return finish(launch_w4a16_decode(*ctx, x, pr, false, m, n, k, sc->workspace,
                                          sc->tile_counters, s, &copies),
                      op, "w4a16_decode_splitk_peer_partials");
    }
    if (m <= fused_max_m() && w4a16_fused_ok(x, &pr, 1, m, n, k)) {
        const size_t ws = w4a16_fused_workspace_bytes(*ctx, 1, m, n, k);
        if (ws && (rc = ensure_workspace(ctx, s, ws, w4a16_fused_num_counters(*ctx, 1, m, n, k), &sc)))
            return rc;
        return finish(launch_w4a16_fused(*ctx, x, &pr, 1, false, m, n, k,
                                         ws ? sc->workspace : nullptr,
                                         ws ? sc->tile_counters : nullptr, s, &copies),
                      op, "w4a16_fused_dequant_peer_partials");
    }
    if (!dq_gemm_fast_path_ok(WFMT_S4_PACKED, x, &pr, 1, false, m, n, k))
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: A, B packed and the staging buffers must be 16-byte aligned and N a "
                    "multiple of 8", op);
    if ((rc = ensure_dq_workspace(ctx, s, dq_gemm_workspace_bytes(1, n, k), &sc)))
        return rc;
    return finish(launch_dq_gemm(*ctx, WFMT_S4_PACKED, x, &pr, 1, false, false, m, n, k,
                                 sc->dq_workspace, s, &copies),
                  op, "w4a16_tcgen05_peer_partials");
}

static int32_t run_sum_partials(const char* op, const float* slots, size_t slots_len, uint32_t world,
                                uint32_t rows, uint32_t cols, void* const* out_ptrs, uint32_t num_out,
                                size_t out_len, uint32_t out_ld, uint32_t out_col0, bool multicast,
                                void* stream)
{
    if (world == 0 || rows == 0 || cols == 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s dimensions must be non-zero", op);
    if (num_out == 0 || num_out > 8)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: 1..8 destinations (got %u)", op, num_out);
    if (cols % 4 != 0 || out_ld % 4 != 0 || out_col0 % 4 != 0 || out_ld < out_col0 + cols)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: cols, out_ld and out_col0 must be multiples of 4 and out_col0 + cols <= "
                    "out_ld (got %u, %u, %u)", op, cols, out_ld, out_col0);
    const size_t need_slots = (size_t)world * rows * cols;
    if (slots_len < need_slots)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: staging buffer too small: need %zu f32, got %zu", op, need_slots, slots_len);
    const size_t need_out = (size_t)(rows - 1) * out_ld + out_col0 + cols;
    if (out_len < need_out)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: out buffers too small: need %zu f32, got %zu", op, need_out, out_len);
    REQUIRE_PTR(slots, op, "slots");
    REQUIRE_PTR(out_ptrs, op, "out_ptrs");
    float* outs[8] = {};
    for (uint32_t d = 0; d < num_out; ++d) {
        if (out_ptrs[d] == nullptr || (uintptr_t)out_ptrs[d] % 16 != 0)
            return fail(KAIO_B200_ERR_INVALID_CONFIG,
                        "%s: output pointer %u is null or not 16-byte aligned", op, d);
        outs[d] = reinterpret_cast<float*>(out_ptrs[d]);
    }
    if ((uintptr_t)slots % 16 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: staging buffer is not 16-byte aligned", op);
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx)))
        return rc;
    return finish(launch_sum_partials(slots, world, rows, cols, outs, num_out, out_ld, out_col0,
                                      multicast, static_cast<cudaStream_t>(stream)),
                  op, multicast ? "sum_partials_f32_multicast" : "sum_partials_f32");
}

KAIO_API int32_t kaio_b200_sum_partials_f32(const float* slots, size_t slots_len, uint32_t world,
                                            uint32_t rows, uint32_t cols, void* const* out_ptrs,
                                            uint32_t num_out, size_t out_len, uint32_t out_ld,
                                            uint32_t out_col0, void* stream)
{
    return run_sum_partials("sum_partials_f32", slots, slots_len, world, rows, cols, out_ptrs, num_out,
                            out_len, out_ld, out_col0, false, stream);
}

KAIO_API int32_t kaio_b200_sum_partials_f32_multicast(const float* slots, size_t slots_len,
                                                      uint32_t world, uint32_t rows, uint32_t cols,
                                                      void* multicast_out, size_t out_len,
                                                      uint32_t out_ld, uint32_t out_col0, void* stream)
{
    void* outs[1] = {multicast_out};
    return run_sum_partials("sum_partials_f32_multicast", slots, slots_len, world, rows, cols, outs, 1,
                            out_len, out_ld, out_col0, true, stream);
}

KAIO_API int32_t kaio_b200_allreduce_multimem_f32(const void* multicast_in, void* multicast_out,
                                                  size_t len, uint32_t rows, uint32_t cols,
                                                  uint32_t ld, uint32_t col0, void* stream)
{
    const char* op = "allreduce_multimem_f32";
    if (rows == 0 || cols == 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s dimensions must be non-zero", op);
    if (cols % 4 != 0 || ld % 4 != 0 || col0 % 4 != 0 || ld < col0 + cols)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: cols, ld and col0 must be multiples of 4 and col0 + cols <= ld (got %u, %u, "
                    "%u)", op, cols, ld, col0);
    if (len < (size_t)(rows - 1) * ld + col0 + cols)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: buffers too small: need %zu f32, got %zu", op,
                    (size_t)(rows - 1) * ld + col0 + cols, len);
    REQUIRE_PTR(multicast_in, op, "multicast_in");
    REQUIRE_PTR(multicast_out, op, "multicast_out");
    if ((uintptr_t)multicast_in % 16 != 0 || (uintptr_t)multicast_out % 16 != 0)
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "%s: multicast addresses must be 16-byte aligned", op);
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx)))
        return rc;
    return finish(launch_multimem_allreduce_f32(static_cast<const float*>(multicast_in),
                                                static_cast<float*>(multicast_out), rows, cols, ld,
                                                col0, static_cast<cudaStream_t>(stream)),
                  op, "allreduce_multimem_f32");
}

// ---------------------------------------------------------------- allocation-free decode entry
// Scratch of kaio_b200_matmul_int4_noalloc: split-K partial tiles, tile arrival counters and a
// status block, in a fixed array that is part of the loaded module (every GPU that loads the
// library holds these ~5.3 MB until the process exits).
namespace kaio {
constexpr size_t NOALLOC_MAX_CTAS = 320;         // two CTAs per SM; B200 has 148 SMs
constexpr size_t NOALLOC_MAX_TILES = 4096;       // column tiles of 128 -> N <= 524288
constexpr size_t NOALLOC_PARTIAL_BYTES = NOALLOC_MAX_CTAS * 2 * 16 * 128 * sizeof(float);
constexpr size_t NOALLOC_COUNTER_BYTES = NOALLOC_MAX_TILES * sizeof(uint32_t);
constexpr size_t NOALLOC_STATUS_BYTES = 256;
constexpr size_t NOALLOC_SCRATCH_BYTES =
    NOALLOC_PARTIAL_BYTES + NOALLOC_COUNTER_BYTES + NOALLOC_STATUS_BYTES;

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// Device address of g_noalloc_scratch per device.  In host code the array's name is only a
// handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
static unsigned char* g_noalloc_ptr[MAX_DEVICES] = {};
static int g_noalloc_sms[MAX_DEVICES] = {};
static std::mutex g_noalloc_mutex;
}  // namespace kaio

KAIO_API int32_t kaio_b200_matmul_int4_noalloc(const kaio_f16* a, size_t a_len,
                                               const uint32_t* b_packed, size_t b_len,
                                               const kaio_f16* scales, size_t scales_len, float* c,
                                               size_t c_len, uint32_t m, uint32_t n, uint32_t k,
                                               uint32_t group_size, void* stream)
{
    const char* op = "matmul_int4_noalloc";
    int32_t rc = validate_int4("f32", a_len, b_len, scales_len, c_len, m, n, k, group_size);
    if (rc)
        return rc;
    REQUIRE_PTR(a, op, "A");
    REQUIRE_PTR(b_packed, op, "B packed");
    REQUIRE_PTR(scales, op, "scales");
    REQUIRE_PTR(c, op, "C");
    if (m > 16)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: M must be at most 16 (got %u); larger M has no allocation-free variant",
                    op, m);
    if (w4a16_decode_num_counters(n) > NOALLOC_MAX_TILES)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: N must be at most %zu (got %u): the fixed scratch holds %zu tile counters",
                    op, NOALLOC_MAX_TILES * 128, n, NOALLOC_MAX_TILES);
    DqProblem pr;
    pr.w = b_packed;
    pr.scales = reinterpret_cast<const __half*>(scales);
    pr.col_scale = nullptr;
    pr.scale = 1.0f;
    pr.out = c;
    const __half* x = reinterpret_cast<const __half*>(a);
    if (!w4a16_decode_ok(x, &pr, 1, m, n, k))
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: A and B packed must be 16-byte aligned device pointers", op);

    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess)
        return fail_cuda(err, "cudaGetDevice");
    if (dev < 0 || dev >= MAX_DEVICES)
        return fail(KAIO_B200_ERR_CUDA, "device ordinal %d out of range", dev);
    {
        // One-time set-up for this device (first call on it; do it before any stream capture).
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (g_noalloc_ptr[dev] == nullptr) {
            int major = 0, sms = 0;
            err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            if (err != cudaSuccess)
                return fail_cuda(err, "cudaDeviceGetAttribute");
            if (major != 10)
                return fail(KAIO_B200_ERR_UNSUPPORTED_ARCH,
                            "kaio_b200 kernels are built for sm_100a only; device %d is sm_%dx", dev,
                            major);
            err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (err != cudaSuccess)
                return fail_cuda(err, "cudaDeviceGetAttribute");
            unsigned char* ptr = nullptr;
            err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
            if (err != cudaSuccess || ptr == nullptr)
                return fail_cuda(err, "cudaGetSymbolAddress(noalloc scratch)");
            // a __device__ array without an initialiser starts as zeros, so the status words
            // need no clearing here
            g_noalloc_sms[dev] = sms;
            g_noalloc_ptr[dev] = ptr;
        }
    }
    DeviceCtx ctx;
    ctx.device = dev;
    ctx.num_sms = g_noalloc_sms[dev];
    unsigned char* base = g_noalloc_ptr[dev];
    ctx.status = reinterpret_cast<uint32_t*>(base + NOALLOC_PARTIAL_BYTES + NOALLOC_COUNTER_BYTES);
    if (w4a16_decode_workspace_bytes(ctx, n, k) > NOALLOC_PARTIAL_BYTES)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "%s: this device needs %zu bytes of split-K scratch, the fixed array holds %zu",
                    op, w4a16_decode_workspace_bytes(ctx, n, k), NOALLOC_PARTIAL_BYTES);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left: the arrival counters must start at zero.
    // The status words are left alone, so that a wait that gave up in an earlier call stays
    // readable until kaio_b200_device_status() has reported and cleared it.
    err = cudaMemsetAsync(base + NOALLOC_PARTIAL_BYTES, 0, NOALLOC_COUNTER_BYTES, s);
    if (err != cudaSuccess)
        return fail_cuda(err, "cudaMemsetAsync(noalloc scratch)");
    return finish(launch_w4a16_decode(ctx, x, pr, false, m, n, k, base,
                                      reinterpret_cast<uint32_t*>(base + NOALLOC_PARTIAL_BYTES), s),
                  op, "w4a16_decode_splitk_noalloc");
}

KAIO_API const char* kaio_b200_last_error(void)
{
    return g_last_error.c_str();
}

KAIO_API const char* kaio_b200_last_variant(void)
{
    return g_last_variant;
}

// Reads and clears one status block; returns its four words in `host`.
static cudaError_t read_status_block(uint32_t* dev_block, uint32_t host[4])
{
    cudaError_t err = cudaMemcpy(host, dev_block, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (err == cudaSuccess && host[0] != 0)
        err = cudaMemset(dev_block, 0, 4 * sizeof(uint32_t));
    return err;
}

KAIO_API int32_t kaio_b200_device_status(void* stream, uint32_t code[4])
{
    // Allocates nothing: it only reads blocks that earlier calls created (the cudaMalloc'd
    // block of the regular entry points, the fixed array of the allocation-free one).
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess)
        return fail_cuda(err, "cudaGetDevice");
    if (dev < 0 || dev >= MAX_DEVICES)
        return fail(KAIO_B200_ERR_CUDA, "device ordinal %d out of range", dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    err = cudaStreamSynchronize(s);
    if (err != cudaSuccess)
        return fail_cuda(err, "cudaStreamSynchronize");
    uint32_t* regular = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        if (g_ctx[dev].device >= 0)
            regular = g_ctx[dev].status;
    }
    unsigned char* fixed = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        fixed = g_noalloc_ptr[dev];
    }
    uint32_t host[4] = {0, 0, 0, 0};
    const char* where = "";
    if (regular != nullptr) {
        err = read_status_block(regular, host);
        if (err != cudaSuccess)
            return fail_cuda(err, "cudaMemcpy(status)");
    }
    if (host[0] == 0 && fixed != nullptr) {
        err = read_status_block(
            reinterpret_cast<uint32_t*>(fixed + NOALLOC_PARTIAL_BYTES + NOALLOC_COUNTER_BYTES), host);
        if (err != cudaSuccess)
            return fail_cuda(err, "cudaMemcpy(status of the allocation-free entry)");
        where = " (allocation-free entry point)";
    }
    if (code)
        for (int i = 0; i < 4; ++i)
            code[i] = host[i];
    if (host[0] != 0) {
        // A launch that gave up may have left split-K arrival counters half counted; the next
        // split-K launch would then miscount.  Every stream of the device was idle or is
        // suspect now, so all counters of the device go back to zero.
        {
            std::lock_guard<std::mutex> lock(g_ctx_mutex);
            for (StreamScratch* sc : g_scratch[dev])
                if (sc->tile_counters)
                    cudaMemset(sc->tile_counters, 0, sc->num_tile_counters * sizeof(uint32_t));
        }
        if (fixed != nullptr)
            cudaMemset(fixed + NOALLOC_PARTIAL_BYTES, 0, NOALLOC_COUNTER_BYTES);
        return fail(KAIO_B200_ERR_TIMEOUT,
                    "device-side bounded wait gave up%s: code %u, block %u, site %u, kernel %u",
                    where, host[0], host[1], host[2], host[3]);
    }
    return KAIO_B200_OK;
}

// Test hook: one CTA waits, with a budget of `budget_us` microseconds (at 2 GHz), on an
// mbarrier that nothing ever arrives at, gives up, records the timeout in the device's status
// block and returns normally -- the path every kernel of the library takes when a wait runs
// out, exercised without a fault.
KAIO_API int32_t kaio_b200_selftest_bounded_wait(uint32_t budget_us, void* stream)
{
    if (budget_us == 0 || budget_us > 100000)
        return fail(KAIO_B200_ERR_INVALID_CONFIG,
                    "selftest_bounded_wait: budget must be 1..100000 microseconds (got %u)", budget_us);
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx)))
        return rc;
    return finish(launch_selftest_bounded_wait(*ctx, budget_us, static_cast<cudaStream_t>(stream)),
                  "selftest_bounded_wait", "selftest_bounded_wait");
}

// Diagnostic: enqueues the INT8 tensor-pipe rate probe (one CTA per SM, `iters` back-to-back
// M128 N256 K32 MMAs each) and reports the work it represents; the caller times it with events.
KAIO_API int32_t kaio_b200_probe_int8_mma_rate(uint32_t iters, uint64_t* ops, void* stream)
{
    if (iters == 0 || iters > (1u << 24))
        return fail(KAIO_B200_ERR_INVALID_CONFIG, "probe_int8_mma_rate: iters must be 1..2^24 (got %u)",
                    iters);
    DeviceCtx* ctx;
    int32_t rc;
    if ((rc = get_ctx(&ctx)))
        return rc;
    if (ops)
        *ops = 2ull * 128 * 256 * 32 * (uint64_t)iters * (uint64_t)ctx->num_sms;
    return finish(launch_int8_mma_rate(*ctx, iters, static_cast<cudaStream_t>(stream)),
                  "probe_int8_mma_rate", "int8_mma_rate_probe");
}

KAIO_API void kaio_b200_shutdown(void)
{
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    int cur = -1;
    cudaGetDevice(&cur);
    for (int d = 0; d < MAX_DEVICES; ++d) {
        DeviceCtx& c = g_ctx[d];
        if (c.device < 0)
            continue;
        cudaSetDevice(d);
        if (c.status)
            cudaFree(c.status);
        for (StreamScratch* sc : g_scratch[d]) {
            if (sc->workspace)
                cudaFree(sc->workspace);
            if (sc->tile_counters)
                cudaFree(sc->tile_counters);
            if (sc->dq_workspace)
                cudaFree(sc->dq_workspace);
            delete sc;
        }
        g_scratch[d].clear();
        c = DeviceCtx();
    }
    if (cur >= 0)
        cudaSetDevice(cur);
}

KAIO_API int32_t kaio_b200_version(void)
{
    return 1001;
}
