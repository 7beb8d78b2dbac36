// Multi-GPU forms of the two quantized products over NCCL (one process per GPU):
//
//   hf2q_cuda_qmatmul_rowshard   dense weights sharded by OUTPUT ROWS: local product, ncclAllGather of the
//                                column blocks, device-side unpack into y[m][n_total];
//   hf2q_cuda_qmatmul_id_ep      expert-parallel mul_mat_id: experts split in contiguous ranges over the
//                                ranks; routed rows are packed by owner on the device, exchanged with a
//                                group of ncclSend / ncclRecv (an all-to-all), multiplied by the local
//                                grouped product, sent back the same way and unpacked into the caller's
//                                row order.
//
// The reference is single-device (hf2q has no collective), so these have no counterpart there; they
// serve the same call sites as quantized_matmul_ggml / quantized_matmul_id_ggml_pooled
// (src/inference/models/qwen35/gpu_ffn.rs:188-206, 1236-1306).  For 1..8 activation rows the
// all-gather lives in the mat-vec kernel instead (hf2q_cuda_qmatmul_gather); this file is the general
// path.  NCCL is looked up at run time (dlopen of libnccl.so.2 -- the copy a host framework such as
// torch has already loaded, if any), so the library itself has no link-time dependency on it.
// Remote data always lands in local memory (NCCL's receive buffer) before any kernel reads it.
//
// hf2q_cuda_qmatmul_id_ep reads the per-rank row counts back to the host once per call (NCCL's
// point-to-point calls take their sizes from the host), i.e. it synchronises the stream once and is
// not captured in CUDA graphs.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"
#include "kernels.h"

using namespace hf2q;

namespace {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

const NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        auto sym = [&](const char* n) { return dlsym(h, n); };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
        api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.Send && api.Recv && api.GroupStart &&
                 api.GroupEnd;
    });
    return api;
}

// ---- device-side pack / unpack ----------------------------------------------------------------

// y_full[t][r * n_local + c] = gathered[r][t][c]
__global__ void __launch_bounds__(256) unpack_gathered_kernel(const float* __restrict__ g, float* __restrict__ y, uint32_t world, uint32_t m,
                                                              uint32_t n_local) {
    const uint64_t total = static_cast<uint64_t>(world) * m * n_local, stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t c = i % n_local, t = (i / n_local) % m, r = i / (static_cast<uint64_t>(n_local) * m);
        y[static_cast<uint64_t>(t) * world * n_local + static_cast<uint64_t>(r) * n_local + c] = g[i];
    }
}

// One CTA: routed rows grouped by the rank that owns their expert.  counts[world], perm[rows]
// (perm[pos] = routed row at packed position pos), local_ids[pos] = expert index relative to its owner.
__global__ void __launch_bounds__(1024) ep_route_kernel(const uint32_t* __restrict__ ids, uint32_t rows, uint32_t n_experts, uint32_t e_local,
                                                        uint32_t world, uint32_t* __restrict__ counts, uint32_t* __restrict__ perm,
                                                        uint32_t* __restrict__ local_ids, uint32_t* status) {
    __shared__ uint32_t cnt[8], off[9], cur[8];
    if (threadIdx.x < 8) cnt[threadIdx.x] = 0;
    __syncthreads();
    bool bad = false;
    for (uint32_t r = threadIdx.x; r < rows; r += blockDim.x) {
        const uint32_t e = ids[r];
        if (e < n_experts) atomicAdd(&cnt[e / e_local], 1u);
        else bad = true;
    }
    if (bad) atomicOr(status, STATUS_BAD_EXPERT_ID);
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t a = 0;
        for (uint32_t p = 0; p < world; ++p) { off[p] = a; cur[p] = a; a += cnt[p]; counts[p] = cnt[p]; }
        off[world] = a;
    }
    __syncthreads();
    for (uint32_t r = threadIdx.x; r < rows; r += blockDim.x) {
        const uint32_t e = ids[r];
        if (e >= n_experts) continue;                     // rejected rows are zero-filled by the unpack kernel's caller
        const uint32_t p = e / e_local, pos = atomicAdd(&cur[p], 1u);
        perm[pos] = r;
        local_ids[pos] = e - p * e_local;
    }
}

// send[pos][:] = x[perm[pos]][:]  (row_bytes multiple of 4)
__global__ void __launch_bounds__(256) ep_pack_kernel(const uint32_t* __restrict__ x, const uint32_t* __restrict__ perm, uint32_t packed_rows,
                                                      uint32_t row_words, uint32_t* __restrict__ send) {
    for (uint32_t pos = blockIdx.x; pos < packed_rows; pos += gridDim.x) {
        const uint32_t* src = x + static_cast<size_t>(perm[pos]) * row_words;
        uint32_t* dst = send + static_cast<size_t>(pos) * row_words;
        for (uint32_t i = threadIdx.x; i < row_words; i += blockDim.x) dst[i] = src[i];
    }
}

// y[perm[pos]][:] = back[pos][:]
__global__ void __launch_bounds__(256) ep_unpack_kernel(const float* __restrict__ back, const uint32_t* __restrict__ perm, uint32_t packed_rows,
                                                        uint32_t n, float* __restrict__ y) {
    for (uint32_t pos = blockIdx.x; pos < packed_rows; pos += gridDim.x) {
        const float* src = back + static_cast<size_t>(pos) * n;
        float* dst = y + static_cast<size_t>(perm[pos]) * n;
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
    }
}

uint64_t align256(uint64_t v) { return (v + 255) & ~255ull; }

}  // namespace

struct hf2q_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1, device = 0;
    uint32_t* host_counts = nullptr;      // pinned, [world * world]
    char err[256] = {0};
};

namespace {
int32_t comm_fail(hf2q_comm* c, ncclResult_t r, const char* what) {
    if (c) snprintf(c->err, sizeof c->err, "%s: %s", what, nccl().GetErrorString ? nccl().GetErrorString(r) : "NCCL error");
    return HF2Q_ERR_CUDA;
}
}  // namespace

extern "C" {

HF2Q_API int32_t hf2q_cuda_comm_unique_id(uint8_t* id128) {
    if (!id128) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!nccl().ok) return HF2Q_ERR_NO_DEVICE;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    ncclUniqueId id;
    if (nccl().GetUniqueId(&id) != ncclSuccess) return HF2Q_ERR_CUDA;
    memcpy(id128, &id, 128);
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_comm_create(int32_t device, const uint8_t* id128, int32_t rank, int32_t world, hf2q_comm** out) {
    if (!id128 || !out || world < 1 || world > 8 || rank < 0 || rank >= world) return HF2Q_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (!nccl().ok) return HF2Q_ERR_NO_DEVICE;
    hf2q_comm* c = new (std::nothrow) hf2q_comm();
    if (!c) return HF2Q_ERR_OUT_OF_MEMORY;
    c->rank = rank; c->world = world; c->device = device;
    int prev = -1;
    cudaGetDevice(&prev);
    if (cudaSetDevice(device) != cudaSuccess) { delete c; return HF2Q_ERR_CUDA; }
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    const ncclResult_t r = nccl().CommInitRank(&c->comm, world, id, rank);
    const cudaError_t e = cudaMallocHost(&c->host_counts, sizeof(uint32_t) * 64);
    if (prev >= 0) cudaSetDevice(prev);
    if (r != ncclSuccess || e != cudaSuccess) {
        if (c->comm) nccl().CommDestroy(c->comm);
        if (c->host_counts) cudaFreeHost(c->host_counts);
        delete c;
        return HF2Q_ERR_CUDA;
    }
    *out = c;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_comm_destroy(hf2q_comm* c) {
    if (!c) return HF2Q_ERR_INVALID_ARGUMENT;
    if (c->comm) nccl().CommDestroy(c->comm);
    if (c->host_counts) cudaFreeHost(c->host_counts);
    delete c;
    return HF2Q_OK;
}

HF2Q_API const char* hf2q_cuda_comm_last_error(const hf2q_comm* c) { return c ? c->err : "null communicator"; }

// ---- dense, rows sharded ------------------------------------------------------------------------

HF2Q_API int32_t hf2q_cuda_qmatmul_rowshard_workspace_bytes(uint32_t m, uint32_t n_local, uint32_t k, uint32_t type, uint32_t x_dtype,
                                                            uint32_t world, uint64_t* out) {
    if (!out || world == 0) return HF2Q_ERR_INVALID_ARGUMENT;
    uint64_t inner = 0;
    const int32_t rc = hf2q_cuda_qmatmul_workspace_bytes(m, n_local, k, type, x_dtype, &inner);
    if (rc) return rc;
    *out = align256(inner) + align256(static_cast<uint64_t>(m) * n_local * 4) + align256(static_cast<uint64_t>(world) * m * n_local * 4);
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_rowshard(hf2q_ctx* ctx, hf2q_comm* comm, void* stream, const void* x, uint32_t x_dtype,
                                            const void* w_shard, float* y_full, uint32_t m, uint32_t n_local, uint32_t k, uint32_t type,
                                            void* workspace, uint64_t workspace_bytes) {
    if (!ctx || !comm) return HF2Q_ERR_INVALID_ARGUMENT;
    uint64_t need = 0, inner = 0;
    int32_t rc = hf2q_cuda_qmatmul_rowshard_workspace_bytes(m, n_local, k, type, x_dtype, comm->world, &need);
    if (rc) return rc;
    hf2q_cuda_qmatmul_workspace_bytes(m, n_local, k, type, x_dtype, &inner);
    if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256) {
        snprintf(comm->err, sizeof comm->err, "qmatmul_rowshard: needs a 256-byte aligned workspace of %llu bytes", (unsigned long long)need);
        return HF2Q_ERR_WORKSPACE;
    }
    if (m == 0) return HF2Q_OK;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    float* y_local = reinterpret_cast<float*>(ws + align256(inner));
    float* gathered = reinterpret_cast<float*>(ws + align256(inner) + align256(static_cast<uint64_t>(m) * n_local * 4));
    rc = hf2q_cuda_qmatmul(ctx, stream, x, x_dtype, w_shard, y_local, m, n_local, k, type, ws, inner);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (comm->world == 1) {
        const cudaError_t e = cudaMemcpyAsync(y_full, y_local, static_cast<size_t>(m) * n_local * 4, cudaMemcpyDeviceToDevice, st);
        return e == cudaSuccess ? HF2Q_OK : HF2Q_ERR_CUDA;
    }
    const ncclResult_t r = nccl().AllGather(y_local, gathered, static_cast<size_t>(m) * n_local, ncclFloat32, comm->comm, st);
    if (r != ncclSuccess) return comm_fail(comm, r, "qmatmul_rowshard: ncclAllGather");
    const uint64_t total = static_cast<uint64_t>(comm->world) * m * n_local;
    const unsigned grid = static_cast<unsigned>(total / 256 + 1 < 148 * 8 ? total / 256 + 1 : 148 * 8);
    unpack_gathered_kernel<<<grid, 256, 0, st>>>(gathered, y_full, comm->world, m, n_local);
    return cudaGetLastError() == cudaSuccess ? HF2Q_OK : HF2Q_ERR_CUDA;
}

// ---- expert-parallel mul_mat_id ---------------------------------------------------------------

namespace {
struct EpLayout {
    uint64_t counts, all_counts, perm, lids_send, lids_recv, x_send, x_recv, y_recv, y_back, g, u, inner, total;
};
// inter != 0: the expert FFN form (gate, up [inter x k], down [n x inter]); inter == 0: one product [n x k]
EpLayout ep_layout(uint32_t rows, uint32_t cap_recv, uint32_t world, uint32_t n, uint32_t k, uint32_t e_local, uint32_t x_dtype, uint32_t inter = 0) {
    EpLayout L{};
    const uint64_t xs = x_dtype == HF2Q_DT_F32 ? 4 : 2;
    uint64_t o = 0;
    L.counts = o;     o += 256;
    L.all_counts = o; o += 256;
    L.perm = o;       o += align256(static_cast<uint64_t>(rows) * 4);
    L.lids_send = o;  o += align256(static_cast<uint64_t>(rows) * 4);
    L.lids_recv = o;  o += align256(static_cast<uint64_t>(cap_recv) * 4);
    L.x_send = o;     o += align256(static_cast<uint64_t>(rows) * k * xs);
    L.x_recv = o;     o += align256(static_cast<uint64_t>(cap_recv) * k * xs);
    L.y_recv = o;     o += align256(static_cast<uint64_t>(cap_recv) * n * 4);
    L.y_back = o;     o += align256(static_cast<uint64_t>(rows) * n * 4);
    L.g = o;          o += align256(static_cast<uint64_t>(cap_recv) * inter * 4);
    L.u = o;          o += align256(static_cast<uint64_t>(cap_recv) * inter * 4);
    L.inner = o;
    uint64_t inner = 0, inner2 = 0;
    hf2q_cuda_qmatmul_id_scratch_bytes(e_local, cap_recv, k, x_dtype, &inner);
    if (inter) hf2q_cuda_qmatmul_id_scratch_bytes(e_local, cap_recv, inter, HF2Q_DT_F32, &inner2);
    if (inter) {                                      // the four-launch form of the expert FFN (sort + gather, SwiGLU pair, down)
        uint64_t inner3 = 0;
        hf2q_cuda_moe_experts_scratch_bytes(e_local, cap_recv, k, inter, &inner3);
        if (inner3 > inner2) inner2 = inner3;
    }
    o += align256(inner > inner2 ? inner : inner2);
    L.total = o;
    (void)world;
    return L;
}
}  // namespace

HF2Q_API int32_t hf2q_cuda_qmatmul_id_ep_scratch_bytes(uint32_t rows, uint32_t cap_recv, uint32_t world, uint32_t n, uint32_t k,
                                                       uint32_t n_experts, uint32_t x_dtype, uint64_t* out) {
    if (!out || world == 0 || n_experts % world) return HF2Q_ERR_INVALID_ARGUMENT;
    *out = ep_layout(rows, cap_recv, world, n, k, n_experts / world, x_dtype).total;
    return HF2Q_OK;
}

namespace {
// w_up == nullptr: y = x . W_local[id]^T (w_a [n x k]).  Otherwise the expert FFN: w_a = gate, w_up = up ([inter x k] per
// expert, stride_a apart), w_down [n x inter] per expert (stride_down apart): y = down(silu(gate x) * (up x)).
int32_t ep_impl(hf2q_ctx* ctx, hf2q_comm* comm, void* stream, const void* x_rows, uint32_t x_dtype, const uint32_t* ids, const void* w_a,
                const void* w_up, const void* w_down, float* y, uint32_t rows, uint32_t cap_recv, uint32_t n, uint32_t k, uint32_t inter,
                uint32_t n_experts, uint64_t expert_stride, uint64_t stride_down, uint32_t type, uint32_t type_down, void* scratch,
                uint64_t scratch_bytes) {
    const void* w_local = w_a;
    if (!ctx || !comm) return HF2Q_ERR_INVALID_ARGUMENT;
    auto bad = [&](const char* msg) { snprintf(comm->err, sizeof comm->err, "qmatmul_id_ep: %s", msg); return HF2Q_ERR_INVALID_ARGUMENT; };
    if (!x_rows || !ids || !w_local || !y) return bad("null pointer");
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return bad("x_dtype must be F32 or BF16");
    const uint32_t world = comm->world;
    if (n_experts == 0 || n_experts % world) return bad("the experts must divide evenly over the ranks");
    const uint32_t e_local = n_experts / world;
    const uint64_t xs = x_dtype == HF2Q_DT_F32 ? 4 : 2;
    if ((static_cast<uint64_t>(k) * xs) % 4) return bad("activation rows must be a multiple of 4 bytes");
    const EpLayout L = ep_layout(rows, cap_recv, world, n, k, e_local, x_dtype, w_up ? inter : 0);
    if (!scratch || scratch_bytes < L.total || reinterpret_cast<uintptr_t>(scratch) % 256) {
        snprintf(comm->err, sizeof comm->err, "qmatmul_id_ep: needs a 256-byte aligned scratch of %llu bytes", (unsigned long long)L.total);
        return HF2Q_ERR_WORKSPACE;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* sb = static_cast<uint8_t*>(scratch);
    uint32_t* counts = reinterpret_cast<uint32_t*>(sb + L.counts);
    uint32_t* all_counts = reinterpret_cast<uint32_t*>(sb + L.all_counts);
    uint32_t* perm = reinterpret_cast<uint32_t*>(sb + L.perm);
    uint32_t* lids_send = reinterpret_cast<uint32_t*>(sb + L.lids_send);
    uint32_t* lids_recv = reinterpret_cast<uint32_t*>(sb + L.lids_recv);
    uint8_t* x_send = sb + L.x_send;
    uint8_t* x_recv = sb + L.x_recv;
    float* y_recv = reinterpret_cast<float*>(sb + L.y_recv);
    float* y_back = reinterpret_cast<float*>(sb + L.y_back);
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != comm->device) cudaSetDevice(comm->device);
    auto restore = [&] { if (prev >= 0 && prev != comm->device) cudaSetDevice(prev); };

    // 1. who owns which row; packed order; how many rows go where (device), then the count matrix to the host
    cudaMemsetAsync(y, 0, static_cast<size_t>(rows) * n * 4, st);            // rows with a rejected id stay zero
    cudaMemsetAsync(sb + L.counts, 0, 256, st);
    ep_route_kernel<<<1, 1024, 0, st>>>(ids, rows, n_experts, e_local, world, counts, perm, lids_send, ctx_status_word(ctx));
    ncclResult_t r = ncclSuccess;
    if (world > 1) {
        r = nccl().AllGather(counts, all_counts, 8, ncclUint32, comm->comm, st);            // [world][8]
        if (r != ncclSuccess) { restore(); return comm_fail(comm, r, "qmatmul_id_ep: ncclAllGather(counts)"); }
    } else {
        cudaMemcpyAsync(all_counts, counts, 32, cudaMemcpyDeviceToDevice, st);
    }
    cudaMemcpyAsync(comm->host_counts, all_counts, sizeof(uint32_t) * 8 * world, cudaMemcpyDeviceToHost, st);
    if (cudaStreamSynchronize(st) != cudaSuccess) { restore(); return HF2Q_ERR_CUDA; }
    std::vector<uint32_t> send_cnt(world), recv_cnt(world), send_off(world + 1, 0), recv_off(world + 1, 0);
    for (uint32_t p = 0; p < world; ++p) {
        send_cnt[p] = comm->host_counts[8 * comm->rank + p];
        recv_cnt[p] = comm->host_counts[8 * p + comm->rank];
        send_off[p + 1] = send_off[p] + send_cnt[p];
        recv_off[p + 1] = recv_off[p] + recv_cnt[p];
    }
    const uint32_t packed = send_off[world], total_recv = recv_off[world];
    if (total_recv > cap_recv) {
        restore();
        snprintf(comm->err, sizeof comm->err, "qmatmul_id_ep: %u rows arrive at this rank, the scratch was sized for %u", total_recv, cap_recv);
        return HF2Q_ERR_WORKSPACE;
    }
    // 2. pack the activations in owner order
    const uint32_t row_words = static_cast<uint32_t>(static_cast<uint64_t>(k) * xs / 4);
    if (packed) ep_pack_kernel<<<packed < 148 * 8 ? packed : 148 * 8, 256, 0, st>>>(static_cast<const uint32_t*>(x_rows), perm, packed, row_words,
                                                                                     reinterpret_cast<uint32_t*>(x_send));
    // 3. all-to-all of the rows and of their local expert indices
    const ncclDataType_t xt = x_dtype == HF2Q_DT_F32 ? ncclFloat32 : ncclBfloat16;
    nccl().GroupStart();
    for (uint32_t p = 0; p < world; ++p) {
        if (send_cnt[p]) {
            nccl().Send(x_send + static_cast<size_t>(send_off[p]) * k * xs, static_cast<size_t>(send_cnt[p]) * k, xt, p, comm->comm, st);
            nccl().Send(lids_send + send_off[p], send_cnt[p], ncclUint32, p, comm->comm, st);
        }
        if (recv_cnt[p]) {
            nccl().Recv(x_recv + static_cast<size_t>(recv_off[p]) * k * xs, static_cast<size_t>(recv_cnt[p]) * k, xt, p, comm->comm, st);
            nccl().Recv(lids_recv + recv_off[p], recv_cnt[p], ncclUint32, p, comm->comm, st);
        }
    }
    r = nccl().GroupEnd();
    if (r != ncclSuccess) { restore(); return comm_fail(comm, r, "qmatmul_id_ep: exchange of the routed rows"); }
    // 4. the local product on what arrived (one activation row per routed row)
    if (total_recv) {
        uint64_t inner = 0;
        hf2q_cuda_qmatmul_id_scratch_bytes(e_local, cap_recv, k, x_dtype, &inner);
        int32_t rc;
        if (!w_up) {
            rc = hf2q_cuda_qmatmul_id(ctx, stream, x_recv, x_dtype, w_local, lids_recv, y_recv, total_recv, 1, n, k, e_local, expert_stride, type,
                                      inner ? sb + L.inner : nullptr, inner);
        } else if (hf2q_cuda_moe_experts_supported(ctx, total_recv, 1, k, inter, e_local, type, type_down)) {
            uint64_t need = 0;
            hf2q_cuda_moe_experts_scratch_bytes(e_local, total_recv, k, inter, &need);
            rc = hf2q_cuda_moe_experts(ctx, stream, x_recv, x_dtype, w_local, w_up, w_down, lids_recv, y_recv, total_recv, 1, k, inter, e_local,
                                       expert_stride, type, stride_down, type_down, sb + L.inner, need);
        } else {
            float* g = reinterpret_cast<float*>(sb + L.g);
            float* u = reinterpret_cast<float*>(sb + L.u);
            rc = hf2q_cuda_qmatmul_id_pair(ctx, stream, x_recv, x_dtype, w_local, w_up, lids_recv, g, u, total_recv, 1, inter, k, e_local,
                                           expert_stride, type, inner ? sb + L.inner : nullptr, inner);
            if (!rc) rc = hf2q_cuda_silu_mul(ctx, stream, g, u, g, static_cast<uint64_t>(total_recv) * inter);
            uint64_t inner2 = 0;
            hf2q_cuda_qmatmul_id_scratch_bytes(e_local, cap_recv, inter, HF2Q_DT_F32, &inner2);
            if (!rc)
                rc = hf2q_cuda_qmatmul_id(ctx, stream, g, HF2Q_DT_F32, w_down, lids_recv, y_recv, total_recv, 1, n, inter, e_local, stride_down,
                                          type_down, inner2 ? sb + L.inner : nullptr, inner2);
        }
        if (rc) { restore(); return rc; }
    }
    // 5. results back to where the rows came from
    nccl().GroupStart();
    for (uint32_t p = 0; p < world; ++p) {
        if (recv_cnt[p]) nccl().Send(y_recv + static_cast<size_t>(recv_off[p]) * n, static_cast<size_t>(recv_cnt[p]) * n, ncclFloat32, p, comm->comm, st);
        if (send_cnt[p]) nccl().Recv(y_back + static_cast<size_t>(send_off[p]) * n, static_cast<size_t>(send_cnt[p]) * n, ncclFloat32, p, comm->comm, st);
    }
    r = nccl().GroupEnd();
    if (r != ncclSuccess) { restore(); return comm_fail(comm, r, "qmatmul_id_ep: exchange of the results"); }
    // 6. into the caller's row order
    if (packed) ep_unpack_kernel<<<packed < 148 * 8 ? packed : 148 * 8, 256, 0, st>>>(y_back, perm, packed, n, y);
    const cudaError_t e = cudaGetLastError();
    restore();
    return e == cudaSuccess ? HF2Q_OK : HF2Q_ERR_CUDA;
}
}  // namespace

HF2Q_API int32_t hf2q_cuda_qmatmul_id_ep(hf2q_ctx* ctx, hf2q_comm* comm, void* stream, const void* x_rows, uint32_t x_dtype,
                                         const uint32_t* ids, const void* w_local, float* y, uint32_t rows, uint32_t cap_recv, uint32_t n,
                                         uint32_t k, uint32_t n_experts, uint64_t expert_stride, uint32_t type, void* scratch,
                                         uint64_t scratch_bytes) {
    return ep_impl(ctx, comm, stream, x_rows, x_dtype, ids, w_local, nullptr, nullptr, y, rows, cap_recv, n, k, 0, n_experts, expert_stride, 0,
                   type, type, scratch, scratch_bytes);
}

HF2Q_API int32_t hf2q_cuda_moe_experts_ep_scratch_bytes(uint32_t rows, uint32_t cap_recv, uint32_t world, uint32_t hidden, uint32_t inter,
                                                        uint32_t n_experts, uint32_t x_dtype, uint64_t* out) {
    if (!out || world == 0 || n_experts % world) return HF2Q_ERR_INVALID_ARGUMENT;
    *out = ep_layout(rows, cap_recv, world, hidden, hidden, n_experts / world, x_dtype, inter).total;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_moe_experts_ep(hf2q_ctx* ctx, hf2q_comm* comm, void* stream, const void* x_rows, uint32_t x_dtype,
                                          const uint32_t* ids, const void* w_gate_local, const void* w_up_local, const void* w_down_local,
                                          float* y, uint32_t rows, uint32_t cap_recv, uint32_t hidden, uint32_t inter, uint32_t n_experts,
                                          uint64_t stride_gate_up, uint64_t stride_down, uint32_t type_gate_up, uint32_t type_down,
                                          void* scratch, uint64_t scratch_bytes) {
    if (!w_up_local || !w_down_local || inter == 0) return HF2Q_ERR_INVALID_ARGUMENT;
    return ep_impl(ctx, comm, stream, x_rows, x_dtype, ids, w_gate_local, w_up_local, w_down_local, y, rows, cap_recv, hidden, hidden, inter,
                   n_experts, stride_gate_up, stride_down, type_gate_up, type_down, scratch, scratch_bytes);
}

}  // extern "C"
