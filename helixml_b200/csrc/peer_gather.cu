// All-gather of a channel-sharded y over NVLink by peer STORES, one process per GPU.
//
// The wide scan shards d_inner over the GPUs of one node (every (batch, channel) chain is independent; B and C are
// replicated), so each rank ends with y[:, :, c0:c1] and the only exchange of the path is the gather of y.  Here
// every rank pushes its shard into the full [batch, seq_len, d_full] buffer of every peer with plain 16-byte
// st.global through pointers mapped from the peers' allocations (CUDA IPC): one read of the local shard, G
// writes, no staging copy, no receive side.  The result has the natural [B, L, D] layout (a library all-gather
// concatenates on the outermost axis and would give [G][B][L][D/G]).  The push takes a range of batch rows, so a
// caller can scan rows in groups and push a finished group on a second stream while the next one is scanned.
//
// Only stores cross the link: nothing here loads from a peer, no TMA, no cluster, no multicast.  After a push a
// rank's own stream knows its stores were issued; the buffers are complete everywhere once every rank has
// synchronised its stream and the ranks have met at a host barrier.
//
// The reference has no distributed code of any kind; this is the exchange the benchmark configuration adds.
#include <cuda_runtime.h>

#include <cstring>

#include "hx_common.cuh"

namespace hx {
namespace gather {

struct PushParams {
    const uint4 *src;       // local shard, dense rows of `vec_per_row` 16-byte vectors
    uint4 *dst[HX_MAX_PEERS];
    int world;
    int64_t rows;           // token rows to push (batch rows * seq_len)
    int64_t src_row0;       // first token row, in the local shard and in the destinations
    int vec_per_row;        // d_shard * es / 16
    int64_t dst_row_vecs;   // d_full * es / 16
    int64_t dst_col_vec;    // col0 * es / 16
};

__global__ void __launch_bounds__(256) push_kernel(const PushParams p) {
    const int64_t total = p.rows * p.vec_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / p.vec_per_row + p.src_row0;
        const int c = (int)(i % p.vec_per_row);
        const uint4 v = __ldg(p.src + r * p.vec_per_row + c);
        const int64_t o = r * p.dst_row_vecs + p.dst_col_vec + c;
#pragma unroll
        for (int g = 0; g < HX_MAX_PEERS; ++g)
            if (g < p.world) p.dst[g][o] = v;
    }
}

}  // namespace gather
}  // namespace hx

extern "C" {

hx_status hx_ipc_export(const void *dptr, void *handle) {
    HX_REQUIRE(dptr && handle, HX_ERR_INVALID_INPUT, "hx_ipc_export: NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == HX_IPC_HANDLE_BYTES, "handle size");
    HX_CUDA(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle), const_cast<void *>(dptr)));
    return HX_OK;
}

hx_status hx_ipc_open(const void *handle, void **dptr) {
    HX_REQUIRE(dptr && handle, HX_ERR_INVALID_INPUT, "hx_ipc_open: NULL argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    HX_CUDA(cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
    return HX_OK;
}

hx_status hx_ipc_close(void *dptr) {
    if (!dptr) return HX_OK;
    HX_CUDA(cudaIpcCloseMemHandle(dptr));
    return HX_OK;
}

hx_status hx_allgather_y_push(const hx_gather_args *a, void *stream) {
    HX_REQUIRE(a != nullptr, HX_ERR_INVALID_INPUT, "hx_allgather_y_push: args is NULL");
    HX_REQUIRE(a->world >= 1 && a->world <= HX_MAX_PEERS && a->rank >= 0 && a->rank < a->world, HX_ERR_INVALID_INPUT,
               "hx_allgather_y_push: rank %d of world %d (at most %d peers)", a->rank, a->world, HX_MAX_PEERS);
    HX_REQUIRE(a->batch >= 0 && a->seq_len >= 0 && a->d_shard >= 0 && a->d_full >= 0, HX_ERR_INVALID_DIMENSION, "negative dimension");
    HX_REQUIRE(a->io_dtype == HX_F32 || a->io_dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "io_dtype %d unsupported", a->io_dtype);
    HX_REQUIRE(a->col0 >= 0 && a->col0 + a->d_shard <= a->d_full, HX_ERR_SHAPE_MISMATCH,
               "channels [%d, %d) do not fit d_full %d", a->col0, a->col0 + a->d_shard, a->d_full);
    HX_REQUIRE(a->row_begin >= 0 && a->row_begin <= a->row_end && a->row_end <= a->batch, HX_ERR_INVALID_DIMENSION,
               "batch rows [%d, %d) outside [0, %d)", a->row_begin, a->row_end, a->batch);
    if (a->row_begin == a->row_end || a->seq_len == 0 || a->d_shard == 0) return HX_OK;
    const int es = (int)hx::dtype_size(a->io_dtype);
    HX_REQUIRE(((int64_t)a->d_shard * es) % 16 == 0 && ((int64_t)a->d_full * es) % 16 == 0 && ((int64_t)a->col0 * es) % 16 == 0,
               HX_ERR_UNSUPPORTED_OPERATION, "shard width, full width and column offset must be multiples of 16 bytes");
    HX_REQUIRE(a->y_local && (reinterpret_cast<uintptr_t>(a->y_local) & 15) == 0, HX_ERR_INVALID_INPUT, "y_local NULL or not 16-byte aligned");
    hx::gather::PushParams p;
    p.src = static_cast<const uint4 *>(a->y_local);
    for (int g = 0; g < HX_MAX_PEERS; ++g) {
        p.dst[g] = g < a->world ? static_cast<uint4 *>(a->dst[g]) : nullptr;
        if (g < a->world)
            HX_REQUIRE(a->dst[g] && (reinterpret_cast<uintptr_t>(a->dst[g]) & 15) == 0, HX_ERR_INVALID_INPUT,
                       "destination %d NULL or not 16-byte aligned", g);
    }
    p.world = a->world;
    p.rows = (int64_t)(a->row_end - a->row_begin) * a->seq_len;
    p.src_row0 = (int64_t)a->row_begin * a->seq_len;
    p.vec_per_row = a->d_shard * es / 16;
    p.dst_row_vecs = (int64_t)a->d_full * es / 16;
    p.dst_col_vec = (int64_t)a->col0 * es / 16;
    const int64_t total = p.rows * p.vec_per_row;
    // a few CTAs per SM: the kernel is bound by the link, and it shares the GPU with the scan of the next rows
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)hx::sm_count() * (a->max_ctas_per_sm > 0 ? a->max_ctas_per_sm : 4);
    if (blocks > cap) blocks = cap;
    hx::gather::push_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
    return hx::check_launch("push_kernel");
}

}  // extern "C"
