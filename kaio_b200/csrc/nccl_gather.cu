// Column-parallel all-gather behind the C ABI: every rank holds its [m, n/P] output shard and
// ends with the row-major [m, n] matrix.  NCCL gathers the shards rank-major into a staging
// buffer ([P][m][n/P]); a copy kernel interleaves them back into rows.
//
// NCCL is not linked: the library looks `libnccl.so.2` up at the first call (dlopen), so it
// loads and runs on machines without NCCL and uses whichever NCCL the host process already has
// (the communicator the caller passes in must come from that same library).
#include <dlfcn.h>

#include <mutex>

#include "kernels.h"

namespace kaio {

// staging[p][i][j] -> out[i][p * n_loc + j], 16 bytes per thread step (n_loc * elem_bytes % 16 == 0)
__global__ void __launch_bounds__(256)
unshard_rows_kernel(const uint4* __restrict__ staging, uint4* __restrict__ out, uint32_t world,
                    uint32_t m, uint32_t vec_per_shard_row)
{
    const size_t total = (size_t)world * m * vec_per_shard_row;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t v = (uint32_t)(i % vec_per_shard_row);
        const size_t pr = i / vec_per_shard_row;
        const uint32_t row = (uint32_t)(pr % m);
        const uint32_t p = (uint32_t)(pr / m);
        out[((size_t)row * world + p) * vec_per_shard_row + v] = staging[i];
    }
}

typedef int (*NcclAllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef const char* (*NcclGetErrorStringFn)(int);

static NcclAllGatherFn g_all_gather = nullptr;
static NcclGetErrorStringFn g_error_string = nullptr;

static bool load_nccl()
{
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr)
            h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr)
            return;
        g_all_gather = reinterpret_cast<NcclAllGatherFn>(dlsym(h, "ncclAllGather"));
        g_error_string = reinterpret_cast<NcclGetErrorStringFn>(dlsym(h, "ncclGetErrorString"));
    });
    return g_all_gather != nullptr;
}

bool nccl_available()
{
    return load_nccl();
}

// Returns 0 on success; on an NCCL failure a positive NCCL result code and *msg its text.
int launch_allgather_cols(const void* shard, void* staging, void* out, uint32_t m, uint32_t n_loc,
                          uint32_t elem_bytes, uint32_t world, void* nccl_comm, cudaStream_t stream,
                          const char** msg, cudaError_t* cuda_err)
{
    *msg = "";
    *cuda_err = cudaSuccess;
    const int dtype = elem_bytes == 2 ? 6 /* ncclFloat16 */ : 7 /* ncclFloat32 */;
    const int rc = g_all_gather(shard, staging, (size_t)m * n_loc, dtype, nccl_comm, stream);
    if (rc != 0) {
        *msg = g_error_string ? g_error_string(rc) : "NCCL error";
        return rc;
    }
    const uint32_t vec = n_loc * elem_bytes / 16;
    const size_t total = (size_t)world * m * vec;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
    unshard_rows_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(staging),
                                                    reinterpret_cast<uint4*>(out), world, m, vec);
    *cuda_err = cudaGetLastError();
    return 0;
}

}  // namespace kaio
